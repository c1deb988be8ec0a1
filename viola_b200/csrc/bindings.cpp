// torch.ops.viola_b200.* : thin tensor -> raw-pointer adapters over the C ABI in api.h.
// No op here allocates; outputs and workspaces are arguments.  Errors raise.
#include <torch/library.h>
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <optional>
#include "api.h"

namespace {

using at::Tensor;
using OptTensor = std::optional<Tensor>;

inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline int dtype_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return 0;
    case at::kBFloat16: return 1;
    case at::kHalf: return 2;
    default: TORCH_CHECK(false, "viola_b200: unsupported dtype ", t.scalar_type());
  }
}
inline int fp8_code(const Tensor& t) {
  if (t.scalar_type() == at::kFloat8_e4m3fn) return 0;
  if (t.scalar_type() == at::kFloat8_e5m2) return 1;
  TORCH_CHECK(false, "viola_b200: expected an FP8 tensor, got ", t.scalar_type());
}
inline void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "viola_b200::", what, " failed: ", cudaGetErrorString((cudaError_t)rc), " (", rc, ")");
}
inline void* ptr(const OptTensor& t) { return t.has_value() && t->defined() && t->numel() ? t->data_ptr() : nullptr; }
inline void cuda_contig(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "viola_b200: ", name, " must be a contiguous CUDA tensor");
}

void amax_scale(const Tensor& x, const OptTensor& history, int64_t index, bool delayed, double limit,
                Tensor scale_out, Tensor scratch) {
  cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_amax_scale(x.data_ptr(), x.numel(), dtype_code(x), (float*)ptr(history),
                      history.has_value() ? (int)history->numel() : 0, index, delayed, (float)limit,
                      scale_out.data_ptr<float>(), (unsigned int*)scratch.data_ptr(), stream()),
        "amax_scale");
}

void quantize(const Tensor& x, const Tensor& scale, double limit, const OptTensor& q, const OptTensor& qt, int64_t fmt,
              const OptTensor& colsum, const OptTensor& workspace) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 2);
  if (colsum.has_value() && colsum->defined())
    TORCH_CHECK(colsum->scalar_type() == at::kFloat && colsum->is_contiguous() && colsum->numel() == x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_quantize(x.data_ptr(), (int)x.size(0), (int)x.size(1), dtype_code(x), scale.data_ptr<float>(), (float)limit,
                    (int)fmt, ptr(q), ptr(qt), (float*)ptr(colsum), (float*)ptr(workspace),
                    workspace.has_value() && workspace->defined() ? workspace->numel() : 0, stream()),
        "quantize");
}

void scale_from_amax(Tensor amax_bits, const OptTensor& history, int64_t index, bool delayed, double limit,
                     Tensor scale_out) {
  TORCH_CHECK(amax_bits.is_cuda() && amax_bits.element_size() == 4 && scale_out.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(amax_bits.device());
  check(vb_scale_from_amax((unsigned int*)amax_bits.data_ptr(), (float*)ptr(history),
                           history.has_value() && history->defined() ? (int)history->numel() : 0, index, delayed,
                           (float)limit, scale_out.data_ptr<float>(), stream()),
        "scale_from_amax");
}

void transpose_u8(const Tensor& x, Tensor out) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.element_size() == 1 && out.numel() == x.numel());
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_transpose_u8(x.data_ptr(), (int)x.size(0), (int)x.size(1), out.data_ptr(), stream()), "transpose_u8");
}

void group_encode(const Tensor& x, int64_t fmt, double limit, const OptTensor& q, const OptTensor& s, int64_t gr,
                  int64_t gc, int64_t s_row, int64_t s_col, const OptTensor& qt, const OptTensor& st, int64_t tgr,
                  int64_t tgc, int64_t st_row, int64_t st_col, bool pow2) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 2 && gc >= 32 && (!qt.has_value() || tgc >= 32), "group columns must be >= 32");
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_group_encode(x.data_ptr(), (int)x.size(0), (int)x.size(1), dtype_code(x), (int)fmt, (float)limit, ptr(q),
                        (float*)ptr(s), (int)gr, (int)gc, s_row, s_col, ptr(qt), (float*)ptr(st), (int)tgr, (int)tgc,
                        st_row, st_col, pow2 ? 1 : 0, stream()),
        "group_encode");
}

void group_decode(const Tensor& q, const Tensor& s, int64_t gr, int64_t gc, int64_t s_row, int64_t s_col, Tensor out) {
  cuda_contig(q, "q");
  c10::cuda::CUDAGuard guard(q.device());
  check(vb_group_decode(q.data_ptr(), s.data_ptr<float>(), (int)q.size(0), (int)q.size(1), fp8_code(q), (int)gr,
                        (int)gc, s_row, s_col, out.data_ptr<float>(), stream()),
        "group_decode");
}

// scale_layout = [group, sa_row, sa_k, sb_row, sb_k, sb_shift, k_shift]
void gemm(const Tensor& a, const Tensor& b, Tensor out, int64_t epilogue, int64_t n_logical, const OptTensor& sa,
          const OptTensor& sb, at::IntArrayRef scale_layout, const OptTensor& bias, double alpha, double beta,
          const OptTensor& resid, const OptTensor& out_t, bool symmetric, int64_t activation, const OptTensor& aux,
          const OptTensor& expert_offsets, const OptTensor& tile_map, const OptTensor& status, int64_t force_bn,
          int64_t batch, bool a_mn, bool b_mn, const OptTensor& amax_out, bool accumulate) {
  // a_mn: ``a`` holds A transposed, i.e. [batch * K, M]; b_mn: ``b`` holds B transposed, [batch * K, N]
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda());
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.stride(-1) == 1);
  TORCH_CHECK(batch >= 1 && a.size(0) % batch == 0 && b.size(0) % batch == 0);
  const int64_t k_a = a_mn ? a.size(0) / batch : a.size(1);
  const int64_t k_b = b_mn ? b.size(0) / batch : b.size(1);
  // a K-major operand may carry zero padding up to the next 16-byte boundary that the MN-major one lacks
  const int64_t k_major = a_mn == b_mn ? k_a : (a_mn ? k_b : k_a), k_minor = a_mn == b_mn ? k_b : (a_mn ? k_a : k_b);
  TORCH_CHECK(k_major >= k_minor && k_major - k_minor < 16 && ((a_mn != b_mn && batch == 1) || k_major == k_minor),
              "K mismatch");
  TORCH_CHECK(!b_mn || b.size(1) >= n_logical, "MN-major B must hold at least N columns");
  c10::cuda::CUDAGuard guard(a.device());
  VbGemmDesc d{};
  d.a_mn_major = a_mn;
  d.b_mn_major = b_mn;
  if (a.element_size() == 1) {
    d.kind = VB_KIND_F8;
    d.a_fmt = fp8_code(a);
    d.b_fmt = fp8_code(b);
  } else {
    d.kind = VB_KIND_F16;
    TORCH_CHECK(a.scalar_type() == b.scalar_type(), "16-bit GEMM operands must share a dtype");
    d.a_fmt = d.b_fmt = a.scalar_type() == at::kBFloat16 ? 1 : 0;
    TORCH_CHECK(a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf);
  }
  d.epilogue = (int)epilogue;
  d.batch = (int)batch;
  d.M = (int)(a_mn ? a.size(1) : a.size(0) / batch);
  d.N = (int)n_logical;
  d.K = (int)k_major;
  d.k_mn = (int)k_minor;
  d.A = a.data_ptr();
  d.lda = a.stride(0);
  d.B = b.data_ptr();
  d.ldb = b.stride(0);
  TORCH_CHECK(scale_layout.size() == 7);
  d.group = (int)scale_layout[0];
  d.sa = (const float*)ptr(sa);
  d.sb = (const float*)ptr(sb);
  d.sa_row = scale_layout[1]; d.sa_k = scale_layout[2]; d.sb_row = scale_layout[3]; d.sb_k = scale_layout[4];
  d.sb_shift = (int)scale_layout[5]; d.k_shift = (int)scale_layout[6];
  TORCH_CHECK(!d.group || (d.sa && d.sb), "group-scaled GEMM needs both scale tensors");
  d.out = out.data_ptr();
  d.out_dtype = dtype_code(out);
  d.ldo = out.stride(-2);
  d.out_batch_stride = batch > 1 ? out.stride(0) : 0;
  d.bias = ptr(bias);
  d.bias_dtype = bias.has_value() && bias->defined() ? dtype_code(*bias) : 0;
  d.alpha = (float)alpha; d.beta = (float)beta;
  d.resid = ptr(resid);
  d.ldr = resid.has_value() && resid->defined() ? resid->stride(-2) : 0;
  d.resid_batch_stride = batch > 1 && d.resid ? resid->stride(0) : 0;
  if (d.resid) TORCH_CHECK(resid->scalar_type() == out.scalar_type(), "residual dtype must match the output");
  d.out_t = ptr(out_t);
  d.ldot = out_t.has_value() && out_t->defined() ? out_t->stride(-2) : 0;
  d.out_t_batch_stride = batch > 1 && d.out_t ? out_t->stride(0) : 0;
  d.symmetric = symmetric;
  d.activation = (int)activation;
  d.amax_out = (unsigned int*)ptr(amax_out);
  if (d.amax_out) TORCH_CHECK(amax_out->element_size() == 4 && amax_out->numel() >= 1);
  d.aux = ptr(aux);
  d.ldaux = aux.has_value() && aux->defined() ? aux->stride(0) : 0;
  if (d.aux) TORCH_CHECK(aux->scalar_type() == out.scalar_type(), "aux dtype must match the output");
  d.expert_offsets = (const int*)ptr(expert_offsets);
  d.num_experts = d.expert_offsets ? (int)expert_offsets->numel() - 1 : 0;
  d.tile_map = (int*)ptr(tile_map);
  if (d.expert_offsets) {
    TORCH_CHECK(d.tile_map && tile_map->numel() >= 3 * ((d.M + 127) / 128 + d.num_experts), "tile_map too small");
    TORCH_CHECK(b.size(0) == (int64_t)d.N * d.num_experts);
  }
  d.status = (int*)ptr(status);
  d.accumulate_out = accumulate ? 1 : 0;
  d.force_bn = (int)(force_bn & 0xffff);          // low half: tile width; high half: split-K units per tile
  d.force_split = (int)(force_bn >> 16);
  check(vb_gemm(&d, stream()), "gemm");
}

void attention_forward(const Tensor& qkv, Tensor out, Tensor lse, double scale, const OptTensor& status) {
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 5 && qkv.size(2) == 3 && qkv.is_contiguous(), "qkv must be [B, T, 3, H, D]");
  TORCH_CHECK(qkv.scalar_type() == at::kBFloat16 || qkv.scalar_type() == at::kHalf);
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == qkv.scalar_type() && out.numel() == qkv.numel() / 3);
  TORCH_CHECK(lse.is_contiguous() && lse.scalar_type() == at::kFloat && lse.numel() == qkv.size(0) * qkv.size(1) * qkv.size(3));
  c10::cuda::CUDAGuard guard(qkv.device());
  check(vb_attention_forward(qkv.data_ptr(), qkv.scalar_type() == at::kBFloat16 ? 1 : 2, (int)qkv.size(0), (int)qkv.size(1),
                             (int)qkv.size(3), (int)qkv.size(4), (float)scale, out.data_ptr(), lse.data_ptr<float>(),
                             (int*)ptr(status), stream()),
        "attention_forward");
}

void momentum_1d(const Tensor& grad, const Tensor& old_q, const Tensor& old_scale, Tensor new_q, Tensor new_scale,
                 Tensor update, int64_t tile, double beta, double inv_loss_scale, bool nesterov, bool stochastic,
                 int64_t step, int64_t key) {
  cuda_contig(grad, "grad");
  c10::cuda::CUDAGuard guard(grad.device());
  TORCH_CHECK(update.scalar_type() == at::kBFloat16 && update.numel() >= grad.numel());
  check(vb_momentum_1d(grad.data_ptr(), dtype_code(grad), grad.numel(), (const uint8_t*)old_q.data_ptr(),
                       old_scale.data_ptr<float>(), (uint8_t*)new_q.data_ptr(), new_scale.data_ptr<float>(),
                       update.data_ptr(), (int)tile, (float)beta, (float)inv_loss_scale, nesterov, stochastic, step,
                       (unsigned long long)key, stream()),
        "momentum_1d");
}

void momentum_2d(const Tensor& grad, int64_t planes, int64_t rows, int64_t cols, const Tensor& old_q,
                 const Tensor& old_scale, Tensor new_q, Tensor new_scale, Tensor update, int64_t tr, int64_t tc,
                 double beta, double inv_loss_scale, bool nesterov, bool stochastic, int64_t step, int64_t key) {
  cuda_contig(grad, "grad");
  c10::cuda::CUDAGuard guard(grad.device());
  check(vb_momentum_2d(grad.data_ptr(), dtype_code(grad), (int)planes, (int)rows, (int)cols,
                       (const uint8_t*)old_q.data_ptr(), old_scale.data_ptr<float>(), (uint8_t*)new_q.data_ptr(),
                       new_scale.data_ptr<float>(), update.data_ptr(), (int)tr, (int)tc, (float)beta,
                       (float)inv_loss_scale, nesterov, stochastic, step, (unsigned long long)key, stream()),
        "momentum_2d");
}

void weight_update(Tensor weight, const Tensor& update, double lr, double decay, double update_scale, bool stochastic,
                   int64_t step, int64_t key, int64_t offset) {
  cuda_contig(weight, "weight");
  cuda_contig(update, "update");
  TORCH_CHECK(weight.numel() == update.numel());
  c10::cuda::CUDAGuard guard(weight.device());
  check(vb_weight_update(weight.data_ptr(), dtype_code(weight), update.data_ptr(), dtype_code(update), weight.numel(),
                         (float)lr, (float)decay, (float)update_scale, stochastic, step, (unsigned long long)key, offset,
                         stream()),
        "weight_update");
}

void adam_update(Tensor weight, const Tensor& grad, Tensor first, Tensor second, double lr, double decay, double b1,
                 double b2, double inv_c1, double inv_c2, double eps, bool adamw, bool maximize, bool stochastic,
                 int64_t step, int64_t key, int64_t offset) {
  cuda_contig(weight, "weight");
  cuda_contig(grad, "grad");
  TORCH_CHECK(first.scalar_type() == second.scalar_type());
  c10::cuda::CUDAGuard guard(weight.device());
  check(vb_adam_update(weight.data_ptr(), dtype_code(weight), grad.data_ptr(), dtype_code(grad), first.data_ptr(),
                       second.data_ptr(), dtype_code(first), weight.numel(), (float)lr, (float)decay, (float)b1,
                       (float)b2, (float)inv_c1, (float)inv_c2, (float)eps, adamw, maximize, stochastic, step,
                       (unsigned long long)key, offset, stream()),
        "adam_update");
}

void copy_scaled(const Tensor& update, Tensor out, int64_t src, int64_t dst, int64_t count, double scale) {
  c10::cuda::CUDAGuard guard(update.device());
  check(vb_copy_scaled(update.data_ptr(), dtype_code(update), out.data_ptr(), dtype_code(out), src, dst, count,
                       (float)scale, stream()),
        "copy_scaled");
}

void momentum16(const Tensor& grad, Tensor momentum, Tensor update, double beta, bool nesterov) {
  c10::cuda::CUDAGuard guard(grad.device());
  check(vb_momentum16(grad.data_ptr(), dtype_code(grad), momentum.data_ptr(), dtype_code(momentum), update.data_ptr(),
                      grad.numel(), (float)beta, nesterov, stream()),
        "momentum16");
}

void sumsq(const Tensor& x, int64_t round_dtype, Tensor accum) {
  // x: [batch, n] (or [n]); accum: float[batch], pre-zeroed
  cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t batch = accum.numel();
  check(vb_sumsq(x.data_ptr(), dtype_code(x) | ((int)round_dtype << 8), x.numel() / batch, accum.data_ptr<float>(),
                 (int)batch, stream()),
        "sumsq");
}

void ns_prescale(const Tensor& x, const Tensor& sumsq_t, double eps, const OptTensor& out, const OptTensor& out_t) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 2 || x.dim() == 3);
  const Tensor& ref = out.has_value() && out->defined() ? *out : *out_t;
  c10::cuda::CUDAGuard guard(x.device());
  const int batch = x.dim() == 3 ? (int)x.size(0) : 1;
  check(vb_ns_prescale(x.data_ptr(), dtype_code(x), (int)x.size(-2), (int)x.size(-1), sumsq_t.data_ptr<float>(),
                       (float)eps, ptr(out), ptr(out_t), dtype_code(ref), batch, stream()),
        "ns_prescale");
}

void ema_lerp(Tensor ema, const Tensor& master, double decay) {
  cuda_contig(ema, "ema");
  cuda_contig(master, "master");
  c10::cuda::CUDAGuard guard(ema.device());
  check(vb_ema_lerp(ema.data_ptr(), dtype_code(ema), master.data_ptr(), dtype_code(master), ema.numel(), (float)decay,
                    stream()),
        "ema_lerp");
}

void philox_kat(int64_t element, int64_t step, int64_t key, Tensor out) {
  c10::cuda::CUDAGuard guard(out.device());
  check(vb_philox_kat((unsigned long long)element, (unsigned long long)step, (unsigned long long)key,
                      (unsigned int*)out.data_ptr(), (int)out.numel(), stream()),
        "philox_kat");
}

void gated_forward(const Tensor& gu, int64_t activation, Tensor out) {
  cuda_contig(gu, "gu");
  c10::cuda::CUDAGuard guard(gu.device());
  check(vb_gated_forward(gu.data_ptr(), dtype_code(gu), (int)gu.size(0), (int)(gu.size(1) / 2), (int)activation,
                         out.data_ptr(), stream()),
        "gated_forward");
}
void gated_backward(const Tensor& gu, const Tensor& dh, int64_t activation, Tensor dgu) {
  cuda_contig(gu, "gu");
  cuda_contig(dh, "dh");
  c10::cuda::CUDAGuard guard(gu.device());
  check(vb_gated_backward(gu.data_ptr(), dh.data_ptr(), dtype_code(gu), (int)gu.size(0), (int)(gu.size(1) / 2),
                          (int)activation, dgu.data_ptr(), stream()),
        "gated_backward");
}

void hadamard64(const Tensor& x, Tensor out) {
  cuda_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_hadamard64(x.data_ptr(), dtype_code(x), (int)(x.numel() / x.size(-1)), (int)x.size(-1), out.data_ptr(),
                      stream()),
        "hadamard64");
}

void wire_pack(const Tensor& x, int64_t rows, int64_t groups, int64_t tile, int64_t fmt, Tensor packet,
               int64_t row_stride) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_wire_pack(x.data_ptr<float>(), x.numel(), (int)rows, (int)groups, (int)tile, (int)fmt,
                     (uint8_t*)packet.data_ptr(), row_stride, stream()),
        "wire_pack");
}
void wire_unpack(const Tensor& packet, int64_t row_stride, int64_t rows, int64_t groups, int64_t tile, int64_t fmt,
                 bool reduce, Tensor out, bool accumulate) {
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous());
  c10::cuda::CUDAGuard guard(out.device());
  check(vb_wire_unpack((const uint8_t*)packet.data_ptr(), row_stride, (int)rows, (int)groups, (int)tile, (int)fmt,
                       reduce, out.data_ptr<float>(), out.numel(), accumulate, stream()),
        "wire_unpack");
}

// ---- MXFP8 hardware block-scaled GEMM --------------------------------------------------------------
Tensor mx_pack_scales(const Tensor& scales, int64_t row_stride, int64_t group_stride, int64_t rows, int64_t k,
                      int64_t row_shift) {
  TORCH_CHECK(scales.is_cuda() && (scales.scalar_type() == at::kFloat || scales.scalar_type() == at::kByte),
              "scales must be a CUDA fp32 or uint8 tensor");
  c10::cuda::CUDAGuard guard(scales.device());
  Tensor out = at::empty({vb_mx_scale_bytes(rows, k)}, scales.options().dtype(at::kByte));
  check(vb_mx_pack_scales(scales.data_ptr(), scales.scalar_type() == at::kByte ? 1 : 0, row_stride, group_stride, (int)rows,
                          (int)k, (int)row_shift, out.data_ptr<uint8_t>(), stream()),
        "mx_pack_scales");
  return out;
}

void mx_gemm(const Tensor& a, int64_t a_fmt, const Tensor& b, int64_t b_fmt, const Tensor& sfa, const Tensor& sfb, Tensor out,
             const OptTensor& bias, Tensor status) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "A [M, K], B [N, K]");
  TORCH_CHECK(a.element_size() == 1 && b.element_size() == 1 && a.stride(1) == 1 && b.stride(1) == 1, "FP8 codes, K contiguous");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == a.size(0) && out.size(1) == b.size(0) && out.stride(1) == 1);
  TORCH_CHECK(sfa.numel() == vb_mx_scale_bytes(a.size(0), a.size(1)) && sfb.numel() == vb_mx_scale_bytes(b.size(0), b.size(1)),
              "scale tensors must come from mx_pack_scales for these operands");
  c10::cuda::CUDAGuard guard(a.device());
  const bool has_bias = bias.has_value() && bias->defined();
  check(vb_mx_gemm(a.data_ptr(), a.stride(0), (int)a_fmt, b.data_ptr(), b.stride(0), (int)b_fmt, sfa.data_ptr<uint8_t>(),
                   sfb.data_ptr<uint8_t>(), (int)a.size(0), (int)b.size(0), (int)a.size(1), out.data_ptr(), dtype_code(out),
                   out.stride(0), has_bias ? bias->data_ptr() : nullptr, has_bias ? dtype_code(*bias) : 0,
                   (int*)status.data_ptr(), stream()),
        "mx_gemm");
}

// ---- peer-memory kernels -----------------------------------------------------------------------
VbPeerTable peer_table(at::IntArrayRef heaps, int64_t rank) {
  VbPeerTable table{};
  TORCH_CHECK(heaps.size() <= 16, "at most 16 ranks per node");
  table.world = (int)heaps.size();
  table.rank = (int)rank;
  for (size_t i = 0; i < heaps.size(); ++i) table.buffers[i] = reinterpret_cast<void*>(heaps[i]);
  return table;
}

void reduce_push_fp8(const Tensor& bucket, int64_t tile, int64_t fmt, int64_t dst_codes, int64_t dst_scales,
                     int64_t dst_flag, int64_t ack_flag, const Tensor& generation, Tensor counter, int64_t wait_clocks,
                     int64_t max_blocks, Tensor status) {
  cuda_contig(bucket, "bucket");
  c10::cuda::CUDAGuard guard(bucket.device());
  check(vb_reduce_push_fp8(bucket.data_ptr<float>(), bucket.numel(), (int)tile, (int)fmt, reinterpret_cast<void*>(dst_codes),
                           reinterpret_cast<float*>(dst_scales), reinterpret_cast<int*>(dst_flag),
                           reinterpret_cast<const int*>(ack_flag), (const int*)generation.data_ptr(),
                           (unsigned int*)counter.data_ptr(),
                           wait_clocks, (int)max_blocks, (int*)status.data_ptr(), stream()),
        "reduce_push_fp8");
}

void reduce_accumulate_fp8(const Tensor& bucket, int64_t tile, int64_t fmt, int64_t recv, int64_t slot_stride,
                           int64_t scales_offset, int64_t flags, at::IntArrayRef heaps, int64_t rank, int64_t ack_offset,
                           const Tensor& generation, Tensor accum, Tensor counter, int64_t wait_clocks, int64_t max_blocks,
                           Tensor status) {
  cuda_contig(bucket, "bucket");
  TORCH_CHECK(accum.scalar_type() == at::kFloat && accum.numel() >= bucket.numel());
  c10::cuda::CUDAGuard guard(bucket.device());
  VbPeerTable table = peer_table(heaps, rank);
  check(vb_reduce_accumulate_fp8(bucket.data_ptr<float>(), bucket.numel(), (int)tile, (int)fmt,
                                 reinterpret_cast<const void*>(recv), slot_stride, scales_offset,
                                 reinterpret_cast<const int*>(flags), &table, ack_offset,
                                 (const int*)generation.data_ptr(), accum.data_ptr<float>(), (unsigned int*)counter.data_ptr(), wait_clocks, (int)max_blocks,
                                 (int*)status.data_ptr(), stream()),
        "reduce_accumulate_fp8");
}

void reduce_many(const Tensor& table, const Tensor& prefix, int64_t total_tiles, int64_t tile, int64_t fmt, at::IntArrayRef heaps,
                 int64_t rank, bool accumulate, int64_t flags, int64_t flag_offset, const Tensor& generation, Tensor counter,
                 int64_t wait_clocks, int64_t max_blocks, Tensor status) {
  // push: ``flags`` = local acknowledgement flags, ``flag_offset`` = heap offset of the data flags at the owners;
  // accumulate: ``flags`` = local data flags, ``flag_offset`` = heap offset of the acknowledgement flags at the sources
  TORCH_CHECK(table.is_cuda() && table.is_contiguous() && prefix.is_cuda() && prefix.scalar_type() == at::kLong);
  const int64_t buckets = prefix.numel() - 1;
  TORCH_CHECK(buckets >= 0 && table.numel() * table.element_size() >= buckets * 64);
  c10::cuda::CUDAGuard guard(table.device());
  VbPeerTable peers = peer_table(heaps, rank);
  if (accumulate)
    check(vb_reduce_accumulate_many(table.data_ptr(), (const long long*)prefix.data_ptr(), (int)buckets, total_tiles, (int)tile,
                                    (int)fmt, &peers, reinterpret_cast<const int*>(flags), flag_offset,
                                    (const int*)generation.data_ptr(), (unsigned int*)counter.data_ptr(), wait_clocks,
                                    (int)max_blocks, (int*)status.data_ptr(), stream()),
          "reduce_accumulate_many");
  else
    check(vb_reduce_push_many(table.data_ptr(), (const long long*)prefix.data_ptr(), (int)buckets, total_tiles, (int)tile,
                              (int)fmt, &peers, flag_offset, reinterpret_cast<const int*>(flags),
                              (const int*)generation.data_ptr(), (unsigned int*)counter.data_ptr(), wait_clocks,
                              (int)max_blocks, (int*)status.data_ptr(), stream()),
          "reduce_push_many");
}

void allreduce_requant_fp8(Tensor value, int64_t tile, int64_t fmt, at::IntArrayRef heaps, int64_t rank, int64_t a2a_offset,
                           int64_t gather_offset, int64_t slot, int64_t a2a_flag_offset, int64_t gather_flag_offset,
                           int64_t generation, Tensor counters, int64_t wait_clocks, int64_t max_blocks, Tensor status) {
  cuda_contig(value, "value");
  c10::cuda::CUDAGuard guard(value.device());
  VbPeerTable table = peer_table(heaps, rank);
  check(vb_allreduce_requant_fp8(value.data_ptr<float>(), value.numel(), (int)tile, (int)fmt, &table, a2a_offset,
                                 gather_offset, slot, a2a_flag_offset, gather_flag_offset, (int)generation,
                                 (unsigned int*)counters.data_ptr(), wait_clocks, (int)max_blocks, (int*)status.data_ptr(),
                                 stream()),
        "allreduce_requant_fp8");
}

void quantize_push(const Tensor& master, const Tensor& scale, double limit, int64_t fmt, const OptTensor& ema, double decay,
                   at::IntArrayRef heaps, int64_t rank, int64_t dst_offset, int64_t shard_rows, int64_t max_blocks) {
  cuda_contig(master, "master");
  TORCH_CHECK(master.dim() == 2);
  c10::cuda::CUDAGuard guard(master.device());
  VbPeerTable table = peer_table(heaps, rank);
  check(vb_quantize_push(master.data_ptr(), dtype_code(master), master.size(0), master.size(1), scale.data_ptr<float>(),
                         (float)limit, (int)fmt, ptr(ema), ema.has_value() && ema->defined() ? dtype_code(*ema) : 0,
                         (float)decay, &table, dst_offset, shard_rows, (int)max_blocks, stream()),
        "quantize_push");
}

void byte_push(const Tensor& src, at::IntArrayRef heaps, int64_t rank, int64_t dst_offset, int64_t shard_bytes,
               int64_t max_blocks) {
  cuda_contig(src, "src");
  c10::cuda::CUDAGuard guard(src.device());
  VbPeerTable table = peer_table(heaps, rank);
  check(vb_byte_push(src.data_ptr(), (long long)src.numel() * src.element_size(), &table, dst_offset, shard_bytes,
                     (int)max_blocks, stream()),
        "byte_push");
}

void multi_writeback(const Tensor& table, const Tensor& prefix, int64_t blocks, double decay, bool with_ema,
                     at::IntArrayRef heaps, int64_t rank, int64_t calls) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() && table.numel() % 16 == 0,
              "write-back table must be a contiguous CUDA int64 tensor of 16-word rows");
  TORCH_CHECK(prefix.is_cuda() && prefix.scalar_type() == at::kInt && prefix.numel() == table.numel() / 16 + 1);
  c10::cuda::CUDAGuard guard(table.device());
  VbPeerTable peers = peer_table(heaps, rank);
  check(vb_multi_writeback(table.data_ptr(), prefix.data_ptr<int>(), (int)(table.numel() / 16), (int)blocks, (float)decay,
                           with_ema ? 1 : 0, &peers, calls, stream()),
        "multi_writeback");
}

void signal(at::IntArrayRef heaps, int64_t rank, int64_t flag_offset, int64_t value, bool include_self) {
  VbPeerTable table = peer_table(heaps, rank);
  check(vb_signal(&table, flag_offset, (int)value, include_self, stream()), "signal");
}

void wait_flags(int64_t flags, int64_t count, int64_t skip, int64_t expected, int64_t wait_clocks, Tensor status) {
  c10::cuda::CUDAGuard guard(status.device());
  check(vb_wait_flags(reinterpret_cast<const int*>(flags), (int)count, (int)skip, (int)expected, wait_clocks,
                      (int*)status.data_ptr(), stream()),
        "wait_flags");
}

void gather_pull(const Tensor& entries, at::IntArrayRef heaps, int64_t rank, int64_t shard_region_offset, Tensor full,
                 const Tensor& piece_prefix, Tensor piece_counts, Tensor panel_flags, int64_t generation,
                 int64_t total_pieces, int64_t max_blocks) {
  c10::cuda::CUDAGuard guard(full.device());
  VbPeerTable table = peer_table(heaps, rank);
  check(vb_gather_pull(entries.data_ptr(), (int)(entries.numel() / 3), &table, shard_region_offset, full.data_ptr(),
                       (const long long*)piece_prefix.data_ptr(), (unsigned int*)piece_counts.data_ptr(),
                       (int*)panel_flags.data_ptr(), (int)generation, total_pieces, (int)max_blocks, stream()),
        "gather_pull");
}

// ---- producer-fused quantisers -------------------------------------------------------------------
// a per-sample modulation vector: bf16 [samples, cols] with unit column stride (rows may be strided views)
static int64_t mod_rows(const Tensor& t, const char* name, int64_t cols) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2 && t.size(1) == cols && t.stride(1) == 1 && t.scalar_type() == at::kBFloat16,
              name, " must be a bf16 CUDA [samples, cols] tensor with unit column stride");
  return t.stride(0);
}
static int stream_dtype(const Tensor& t, const char* name) {
  TORCH_CHECK(t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16, name, " must be fp32 or bf16");
  return t.scalar_type() == at::kFloat ? 0 : 1;
}

void ln_stats_amax(const Tensor& x, double eps, const Tensor& shift, const Tensor& scale, int64_t tokens, Tensor mean,
                   Tensor rstd, const OptTensor& history, int64_t index, bool delayed, double limit, Tensor scale_out,
                   Tensor scratch) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 2);
  const int64_t stride = mod_rows(shift, "shift", x.size(1));
  TORCH_CHECK(mod_rows(scale, "scale", x.size(1)) == stride, "shift and scale must share a row pitch");
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_ln_stats_amax(x.data_ptr(), stream_dtype(x, "x"), (int)x.size(0), (int)x.size(1), (float)eps, shift.data_ptr(),
                         scale.data_ptr(), stride, (int)tokens, mean.data_ptr<float>(), rstd.data_ptr<float>(),
                         (float*)ptr(history), history.has_value() ? (int)history->numel() : 0, index, delayed,
                         (float)limit, scale_out.data_ptr<float>(), (unsigned int*)scratch.data_ptr(), stream()),
        "ln_stats_amax");
}

void act_amax(const Tensor& z, int64_t mode, const OptTensor& history, int64_t index, bool delayed, double limit,
              Tensor scale_out, Tensor scratch) {
  cuda_contig(z, "z");
  TORCH_CHECK(z.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(z.device());
  check(vb_act_amax(z.data_ptr(), z.numel(), (int)mode, (float*)ptr(history), history.has_value() ? (int)history->numel() : 0,
                    index, delayed, (float)limit, scale_out.data_ptr<float>(), (unsigned int*)scratch.data_ptr(), stream()),
        "act_amax");
}

void fused_quantize(const Tensor& x, int64_t mode, const OptTensor& mean, const OptTensor& rstd, const OptTensor& shift,
                    const OptTensor& scale, int64_t tokens, const Tensor& qscale, double limit, int64_t fmt,
                    const OptTensor& q, const OptTensor& qt, const OptTensor& slope) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 2);
  if (slope.has_value() && slope->defined())
    TORCH_CHECK(slope->scalar_type() == at::kBFloat16 && slope->is_contiguous() && slope->sizes() == x.sizes());
  int64_t stride = 0;
  if (mode == 1) {
    TORCH_CHECK(shift.has_value() && scale.has_value() && mean.has_value() && rstd.has_value());
    stride = mod_rows(*shift, "shift", x.size(1));
    TORCH_CHECK(mod_rows(*scale, "scale", x.size(1)) == stride, "shift and scale must share a row pitch");
  }
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_fused_quantize(x.data_ptr(), stream_dtype(x, "x"), (int)x.size(0), (int)x.size(1), (int)mode,
                          (const float*)ptr(mean), (const float*)ptr(rstd), ptr(shift), ptr(scale), stride, (int)tokens,
                          qscale.data_ptr<float>(), (float)limit, (int)fmt, ptr(q), ptr(qt), ptr(slope), stream()),
        "fused_quantize");
}

void ln_modulate_backward(const Tensor& dh, const Tensor& x, const Tensor& mean, const Tensor& rstd, const Tensor& scale,
                          int64_t tokens, const OptTensor& grad_in, Tensor dx, Tensor dshift, Tensor dscale, Tensor workspace,
                          Tensor tickets) {
  cuda_contig(dh, "dh");
  cuda_contig(x, "x");
  cuda_contig(dx, "dx");
  TORCH_CHECK(dh.scalar_type() == at::kBFloat16 && dx.scalar_type() == x.scalar_type());
  if (grad_in.has_value() && grad_in->defined())
    TORCH_CHECK(grad_in->is_contiguous() && grad_in->scalar_type() == x.scalar_type() && grad_in->sizes() == x.sizes());
  TORCH_CHECK((dshift.scalar_type() == at::kFloat || dshift.scalar_type() == at::kBFloat16) &&
              dscale.scalar_type() == dshift.scalar_type() && dshift.is_contiguous() && dscale.is_contiguous());
  const int64_t stride = mod_rows(scale, "scale", x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_ln_modulate_backward(dh.data_ptr(), x.data_ptr(), stream_dtype(x, "x"), mean.data_ptr<float>(),
                                rstd.data_ptr<float>(), scale.data_ptr(), stride, (int)x.size(0), (int)x.size(1),
                                (int)tokens, ptr(grad_in), dx.data_ptr(), dshift.data_ptr(), dscale.data_ptr(),
                                dshift.scalar_type() == at::kBFloat16 ? 1 : 0, workspace.data_ptr<float>(), workspace.numel(), (unsigned int*)tickets.data_ptr(),
                                (int)tickets.numel(), stream()),
        "ln_modulate_backward");
}

int64_t row_block_count(int64_t rows, int64_t tokens) { return vb_row_block_count((int)rows, (int)tokens); }

void gate_residual(const Tensor& x, const Tensor& gate, const Tensor& y, int64_t tokens, Tensor out) {
  cuda_contig(x, "x");
  cuda_contig(y, "y");
  cuda_contig(out, "out");
  TORCH_CHECK(x.dim() == 2 && y.sizes() == x.sizes() && out.sizes() == x.sizes());
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && out.scalar_type() == x.scalar_type());
  const int64_t stride = mod_rows(gate, "gate", x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  check(vb_gate_residual(x.data_ptr(), stream_dtype(x, "x"), gate.data_ptr(), stride, y.data_ptr(), (int)x.size(0),
                         (int)x.size(1), (int)tokens, out.data_ptr(), stream()),
        "gate_residual");
}

void gate_residual_backward(const Tensor& dout, const Tensor& gate, const Tensor& y, int64_t tokens, Tensor dy,
                            Tensor dgate, Tensor workspace, Tensor tickets) {
  cuda_contig(dout, "dout");
  cuda_contig(y, "y");
  cuda_contig(dy, "dy");
  cuda_contig(dgate, "dgate");
  TORCH_CHECK(dout.dim() == 2 && y.sizes() == dout.sizes() && dy.sizes() == dout.sizes());
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && dy.scalar_type() == at::kBFloat16 &&
              (dgate.scalar_type() == at::kFloat || dgate.scalar_type() == at::kBFloat16));
  const int64_t stride = mod_rows(gate, "gate", dout.size(1));
  c10::cuda::CUDAGuard guard(dout.device());
  check(vb_gate_residual_backward(dout.data_ptr(), stream_dtype(dout, "dout"), gate.data_ptr(), stride, y.data_ptr(),
                                  (int)dout.size(0), (int)dout.size(1), (int)tokens, dy.data_ptr(),
                                  dgate.data_ptr(), dgate.scalar_type() == at::kBFloat16 ? 1 : 0,
                                  workspace.data_ptr<float>(), workspace.numel(),
                                  (unsigned int*)tickets.data_ptr(), (int)tickets.numel(), stream()),
        "gate_residual_backward");
}

// ---- multi-tensor optimizer kernels ---------------------------------------------------------------
void multi_ema(const Tensor& table, const Tensor& prefix, int64_t blocks, double decay) {
  c10::cuda::CUDAGuard guard(table.device());
  check(vb_multi_ema(table.data_ptr(), (const int*)prefix.data_ptr(), (int)table.size(0), (int)blocks, (float)decay, stream()),
        "multi_ema");
}
void multi_adam(const Tensor& table, const Tensor& prefix, int64_t blocks, double lr, double decay, double b1, double b2,
                double inv_c1, double inv_c2, double eps, bool adamw, bool maximize, bool stochastic, int64_t step) {
  c10::cuda::CUDAGuard guard(table.device());
  check(vb_multi_adam(table.data_ptr(), (const int*)prefix.data_ptr(), (int)table.size(0), (int)blocks, (float)lr,
                      (float)decay, (float)b1, (float)b2, (float)inv_c1, (float)inv_c2, (float)eps, adamw, maximize,
                      stochastic, step, stream()),
        "multi_adam");
}
void multi_weight_update(const Tensor& table, const Tensor& prefix, int64_t blocks, double lr, double decay, bool stochastic,
                         int64_t step) {
  c10::cuda::CUDAGuard guard(table.device());
  check(vb_multi_weight_update(table.data_ptr(), (const int*)prefix.data_ptr(), (int)table.size(0), (int)blocks, (float)lr,
                               (float)decay, stochastic, step, stream()),
        "multi_weight_update");
}
void multi_momentum(const Tensor& table, const Tensor& prefix, int64_t blocks, int64_t tile, double beta,
                    double inv_loss_scale, bool nesterov, bool stochastic, int64_t step) {
  c10::cuda::CUDAGuard guard(table.device());
  check(vb_multi_momentum(table.data_ptr(), (const int*)prefix.data_ptr(), (int)table.size(0), (int)blocks, (int)tile,
                          (float)beta, (float)inv_loss_scale, nesterov, stochastic, step, stream()),
        "multi_momentum");
}

}  // namespace

TORCH_LIBRARY(viola_b200, m) {
  m.def("amax_scale", &amax_scale);
  m.def("quantize", &quantize);
  m.def("transpose_u8", &transpose_u8);
  m.def("scale_from_amax", &scale_from_amax);
  m.def("group_encode", &group_encode);
  m.def("group_decode", &group_decode);
  m.def("gemm", &gemm);
  m.def("momentum_1d", &momentum_1d);
  m.def("momentum_2d", &momentum_2d);
  m.def("weight_update", &weight_update);
  m.def("adam_update", &adam_update);
  m.def("copy_scaled", &copy_scaled);
  m.def("momentum16", &momentum16);
  m.def("sumsq", &sumsq);
  m.def("ns_prescale", &ns_prescale);
  m.def("ema_lerp", &ema_lerp);
  m.def("philox_kat", &philox_kat);
  m.def("gated_forward", &gated_forward);
  m.def("gated_backward", &gated_backward);
  m.def("hadamard64", &hadamard64);
  m.def("wire_pack", &wire_pack);
  m.def("wire_unpack", &wire_unpack);
  m.def("reduce_push_fp8", &reduce_push_fp8);
  m.def("reduce_accumulate_fp8", &reduce_accumulate_fp8);
  m.def("allreduce_requant_fp8", &allreduce_requant_fp8);
  m.def("quantize_push", &quantize_push);
  m.def("byte_push", &byte_push);
  m.def("multi_writeback", &multi_writeback);
  m.def("mx_pack_scales", &mx_pack_scales);
  m.def("mx_gemm", &mx_gemm);
  m.def("attention_forward", &attention_forward);
  m.def("reduce_many", &reduce_many);
  m.def("signal", &signal);
  m.def("wait_flags", &wait_flags);
  m.def("gather_pull", &gather_pull);
  m.def("multi_ema", &multi_ema);
  m.def("multi_adam", &multi_adam);
  m.def("multi_weight_update", &multi_weight_update);
  m.def("multi_momentum", &multi_momentum);
  m.def("ln_stats_amax", &ln_stats_amax);
  m.def("act_amax", &act_amax);
  m.def("fused_quantize", &fused_quantize);
  m.def("ln_modulate_backward", &ln_modulate_backward);
  m.def("row_block_count", &row_block_count);
  m.def("gate_residual", &gate_residual);
  m.def("gate_residual_backward", &gate_residual_backward);
}
