// C ABI of the sm_100a kernel library.  Every entry point takes raw device
// pointers and a stream, returns a cudaError_t as int, and allocates nothing:
// workspaces are passed in by the caller (the Python layer owns them).
#pragma once
#include <cstdint>
#include <algorithm>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- quantisation ----------------------------------------------------------
int vb_amax_scale(const void* x, long long n, int dtype, float* history, int history_len,
                  long long index, int delayed, float limit, float* scale_out, unsigned int* scratch,
                  cudaStream_t stream);
// scale from an amax that a producer kernel gathered as float bits (see VbGemmDesc::amax_out); zeroes the word
int vb_scale_from_amax(unsigned int* amax_bits, float* history, int history_len, long long index, int delayed,
                       float limit, float* scale_out, cudaStream_t stream);
// colsum (optional, row-wise output only, cols % 16 == 0): fp32 [cols], the column sums of x are ADDED to it, in a
// fixed order (reproducible).  workspace: 1024 + ceil(rows / 256) * strips * 128 floats with strips =
// ceil(cols / 128) <= 1024; its first 1024 words (tickets) must be zero on first use and are left zero.
int vb_quantize(const void* x, int rows, int cols, int dtype, const float* scale, float limit, int fmt,
                void* q, void* qt, float* colsum, float* workspace, long long workspace_floats, cudaStream_t stream);
int vb_transpose_u8(const void* x, int rows, int cols, void* out, cudaStream_t stream);
int vb_group_encode(const void* x, int rows, int cols, int dtype, int fmt, float limit, void* q, float* s,
                    int gr, int gc, long long s_row, long long s_col, void* qt, float* st, int tgr, int tgc,
                    long long st_row, long long st_col, int pow2 /* 1: round every scale up to a power of two (MXFP8) */, cudaStream_t stream);
int vb_group_decode(const void* q, const float* s, int rows, int cols, int fmt, int gr, int gc,
                    long long s_row, long long s_col, float* out, cudaStream_t stream);

// ---- tcgen05 GEMM family -----------------------------------------------------
// D[M, N] = A[M, K] . B[N, K]^T, both operands K-major (row-major with K contiguous).
enum VbGemmKind { VB_KIND_F16 = 0, VB_KIND_F8 = 1 };
enum VbEpilogue { VB_EPI_LINEAR = 0, VB_EPI_AXPBY = 1, VB_EPI_GATED_FWD = 2, VB_EPI_GATED_BWD = 3, VB_EPI_ACT_BWD = 4 };
enum VbActivation { VB_ACT_SILU = 0, VB_ACT_GELU = 1, VB_ACT_RELU = 2 };

typedef struct VbGemmDesc {
  int kind;              // VbGemmKind
  int a_fmt, b_fmt;      // F16 kind: 0 fp16, 1 bf16 (must match); F8 kind: 0 e4m3, 1 e5m2
  int epilogue;          // VbEpilogue
  int M, N, K;           // N = logical output width (gated forward: hidden width H)
  const void* A; long long lda;   // elements
  const void* B; long long ldb;   // elements; rows = N (2N for gated forward, E*N for experts)
  // scaling: per-tensor (group == 0): alpha = (*sa) * (*sb), null pointer = 1.
  // group (== 1): fp32 scale per 128.2^k_shift K elements;
  //   sa index = row * sa_row + (kb >> k_shift) * sa_k
  //   sb index = (brow >> sb_shift) * sb_row + (kb >> k_shift) * sb_k   (brow = row of B)
  int group;
  const float* sa; const float* sb;
  long long sa_row, sa_k, sb_row, sb_k;
  int sb_shift, k_shift;
  // output
  void* out; int out_dtype; long long ldo;       // 0 fp32, 1 bf16, 2 fp16
  const void* bias; int bias_dtype;              // [N] (gated forward: [2N]) or null
  // AXPBY: out = alpha * round(acc) + beta * R, optional transposed copy / symmetric mirror
  float alpha, beta;
  const void* resid; long long ldr;
  void* out_t; long long ldot;
  int symmetric;         // 1: M == N, only tiles with n_tile >= m_tile are computed and mirrored
  // gated MLP
  int activation;        // VbActivation
  void* aux; long long ldaux;   // [M, 2N] saved (gate | up) in out dtype (fwd: written, bwd: read);
                                // VB_EPI_ACT_BWD: [M, N] activation slope act'(z) saved by the forward pass,
                                // out = round(acc) * aux
  unsigned int* amax_out;       // VB_EPI_ACT_BWD: atomicMax of |out| as float bits (caller zero-initialises)
  // expert GEMM: rows of A are grouped by expert; offsets[e]..offsets[e+1] (device, int32, E+1)
  const int* expert_offsets; int num_experts;
  int* tile_map;         // workspace int32[3 * (ceil(M/128) + E)] when expert_offsets != null
  int* status;           // int32[8] device status word (zeroed by caller) or null
  int force_bn;          // 0 = auto, else 64 / 128 / 256
  // batched problems (LINEAR / AXPBY): A is [batch * M, K], B is [batch * N, K]; strides in elements
  int batch;
  long long out_batch_stride, resid_batch_stride, out_t_batch_stride;
  // operand layouts: 0 = K-major (A is [M, K], B is [N, K]); 1 = MN-major (A stored as [K, M], B as [K, N]);
  // lda / ldb are always the row pitch of the stored matrix
  int a_mn_major, b_mn_major;
  int k_mn;              // rows of K actually stored by an MN-major operand (0: K); K - k_mn < 16 rows read as zero
  int force_split;       // LINEAR epilogue: 0 = choose, 1 = no split-K, k > 1 = k work units per output tile
  int accumulate_out;    // LINEAR, fp32 output through TMA, no bias: out += product (TMA reduce-add) instead of out = product
  int no_tma_store;      // 1: LINEAR epilogue writes with per-thread stores instead of the TMA-store path
} VbGemmDesc;

int vb_gemm(const VbGemmDesc* desc, cudaStream_t stream);

// ---- MXFP8: hardware block-scaled GEMM (mxfp8_gemm_sm100.cu) ---------------------------------
// out[m, n] = sum_k (A[m, k] * 2^(sfa[m, k/32] - 127)) * (B[n, k] * 2^(sfb[n, k/32] - 127)) (+ bias[n]);
// A [M, K], B [N, K]: e4m3 (fmt 0) / e5m2 (fmt 1) codes, K contiguous, row pitches lda / ldb bytes (multiples of 16).
// sfa_tiled / sfb_tiled: UE8M0 scale bytes in the tiled layout written by vb_mx_pack_scales
// (vb_mx_scale_bytes(rows, K) bytes each, 16-byte aligned).  out_dtype: 0 fp32, 1 bf16, 2 fp16.
long long vb_mx_scale_bytes(long long rows, long long k);
// scales: one fp32 power of two (is_bytes = 0) or one UE8M0 byte (is_bytes = 1) per (row >> row_shift, 32 K elements),
// element (r, g) at scales[(r >> row_shift) * row_stride + g * group_stride].
int vb_mx_pack_scales(const void* scales, int is_bytes, long long row_stride, long long group_stride, int rows, int k,
                      int row_shift, uint8_t* out, cudaStream_t stream);
int vb_mx_gemm(const void* a, long long lda, int a_fmt, const void* b, long long ldb, int b_fmt,
               const uint8_t* sfa_tiled, const uint8_t* sfb_tiled, int M, int N, int K, void* out, int out_dtype,
               long long ldo, const void* bias, int bias_dtype, int* status, cudaStream_t stream);

// ---- optimizer kernels ---------------------------------------------------------
int vb_momentum_1d(const void* grad, int grad_dtype, long long n, const uint8_t* old_q,
                   const float* old_scale, uint8_t* new_q, float* new_scale, void* update_bf16,
                   int tile_size, float beta, float inv_loss_scale, int nesterov, int stochastic,
                   long long step, unsigned long long key, cudaStream_t stream);
int vb_momentum_2d(const void* grad, int grad_dtype, int planes, int rows, int cols, const uint8_t* old_q,
                   const float* old_scale, uint8_t* new_q, float* new_scale, void* update_bf16, int tr,
                   int tc, float beta, float inv_loss_scale, int nesterov, int stochastic, long long step,
                   unsigned long long key, cudaStream_t stream);
int vb_weight_update(void* weight, int weight_dtype, const void* update, int update_dtype, long long n,
                     float lr, float decay, float update_scale, int stochastic, long long step,
                     unsigned long long key, long long offset, cudaStream_t stream);
int vb_adam_update(void* weight, int weight_dtype, const void* grad, int grad_dtype, void* first,
                   void* second, int state_dtype, long long n, float lr, float decay, float b1, float b2,
                   float inv_c1, float inv_c2, float eps, int adamw, int maximize, int stochastic,
                   long long step, unsigned long long key, long long offset, cudaStream_t stream);
int vb_copy_scaled(const void* update, int dtype, void* out, int out_dtype, long long src, long long dst,
                   long long count, float scale, cudaStream_t stream);
int vb_momentum16(const void* grad, int grad_dtype, void* momentum, int momentum_dtype, void* update_bf16,
                  long long n, float beta, int nesterov, cudaStream_t stream);
// Frobenius-norm based prescale for Newton-Schulz: out = x / (||x||_F + eps) in `out_dtype`,
// optionally also writing the transpose.  scratch: float[2] (zeroed; self-resetting).
int vb_sumsq(const void* x, int dtype, long long n, float* accum, int batch, cudaStream_t stream);
int vb_ns_prescale(const void* x, int dtype, int rows, int cols, const float* sumsq, float eps, void* out,
                   void* out_t, int out_dtype, int batch, cudaStream_t stream);
// master -> EMA lerp fused with optional dtype casts (owner-side writeback helper)
int vb_ema_lerp(void* ema, int ema_dtype, const void* master, int master_dtype, long long n, float decay,
                cudaStream_t stream);
int vb_philox_kat(unsigned long long element, unsigned long long step, unsigned long long key,
                  unsigned int* out, int count, cudaStream_t stream);

// ---- multi-tensor optimizer kernels (multi.cu) --------------------------------------------
// table: device array of 64-byte descriptors {p0, p1, p2, p3, n, i0, (f0, f1), (d0, d1)};
// prefix: device int32[tensors + 1] prefix sums of 4096-element chunks; blocks = prefix[tensors].
int vb_multi_ema(const void* table, const int* prefix, int tensors, int blocks, float decay, cudaStream_t stream);
int vb_multi_adam(const void* table, const int* prefix, int tensors, int blocks, float lr, float decay, float b1,
                  float b2, float inv_c1, float inv_c2, float eps, int adamw, int maximize, int stochastic,
                  long long step, cudaStream_t stream);
int vb_multi_weight_update(const void* table, const int* prefix, int tensors, int blocks, float lr, float decay,
                           int stochastic, long long step, cudaStream_t stream);
int vb_multi_momentum(const void* table, const int* prefix, int tensors, int blocks, int tile, float beta,
                      float inv_loss_scale, int nesterov, int stochastic, long long step, cudaStream_t stream);

// ---- gated activation (unfused baseline + post-rotation path) ------------------
int vb_gated_forward(const void* gu, int dtype, int rows, int hidden, int activation, void* out,
                     cudaStream_t stream);
int vb_gated_backward(const void* gu, const void* dh, int dtype, int rows, int hidden, int activation,
                      void* dgu, cudaStream_t stream);

// ---- producer-fused quantisers (fused.cu): per-tensor scales ---------------------------------------
// mode: 1 = LayerNorm (no affine) + modulate, 2 = GELU(tanh), 3 = SiLU.  x_dtype: 0 fp32, 1 bf16 (the residual
// stream); modulation vectors are bf16 rows of pitch mod_stride (elements), one row per sample of `tokens` rows.
int vb_ln_stats_amax(const void* x, int x_dtype, int rows, int cols, float eps, const void* mod_shift,
                     const void* mod_scale, long long mod_stride, int tokens, float* mean, float* rstd, float* history,
                     int history_len, long long index, int delayed, float limit, float* scale_out,
                     unsigned int* scratch, cudaStream_t stream);
int vb_act_amax(const void* z, long long n, int mode, float* history, int history_len, long long index,
                int delayed, float limit, float* scale_out, unsigned int* scratch, cudaStream_t stream);
// slope (optional, activation modes, row-wise output only): bf16 [rows, cols] that receives act'(x), which is all
// the backward pass needs of x
int vb_fused_quantize(const void* x, int x_dtype, int rows, int cols, int mode, const float* mean, const float* rstd,
                      const void* mod_shift, const void* mod_scale, long long mod_stride, int tokens,
                      const float* scale, float limit, int fmt, void* q, void* qt, void* slope, cudaStream_t stream);
// The per-sample column sums (dshift, dscale, dgate) are reproducible: blocks park their totals in `workspace`
// (vb_row_block_count(rows, tokens) x (2 * cols | cols) floats) and the last block of a sample (tickets: one zeroed
// word per sample, left zero) adds them in a fixed order; the outputs are written, not accumulated.
int vb_row_block_count(int rows, int tokens);
int vb_ln_modulate_backward(const void* dh, const void* x, int x_dtype, const float* mean, const float* rstd,
                            const void* mod_scale, long long mod_stride, int rows, int cols, int tokens,
                            const void* grad_in /* optional, x's dtype: added to dx */, void* dx,
                            void* dshift, void* dscale, int sums_bf16 /* 0: fp32 sums, 1: bf16 sums */,
                            float* workspace, long long workspace_floats, unsigned int* tickets, int ticket_count,
                            cudaStream_t stream);
// out = x + gate[row / tokens] * y (x, out: x_dtype; y, gate: bf16) and the branch side of its backward:
// dy = dout * gate (bf16), dgate = per-sample column sums of dout * y (fp32, or bf16 with sums_bf16)
int vb_gate_residual(const void* x, int x_dtype, const void* gate, long long gate_stride, const void* y, int rows,
                     int cols, int tokens, void* out, cudaStream_t stream);
int vb_gate_residual_backward(const void* dout, int dout_dtype, const void* gate, long long gate_stride, const void* y,
                              int rows, int cols, int tokens, void* dy, void* dgate, int sums_bf16, float* workspace,
                              long long workspace_floats, unsigned int* tickets, int ticket_count, cudaStream_t stream);

// ---- attention forward for 256-token sequences (tcgen05; one CTA per sample and head) ------------
// qkv: [batch, 256, 3, heads, head_dim] contiguous (dtype 1 = bf16, 2 = fp16), head_dim a multiple of 8 in [16, 128];
// out: [batch, 256, heads, head_dim]; lse: [batch, heads, 256] fp32 = log(sum(exp(score * scale))) per query (optional)
int vb_attention_forward(const void* qkv, int dtype, int batch, int tokens, int heads, int head_dim, float scale,
                         void* out, float* lse, int* status, cudaStream_t stream);

// ---- Hadamard-64 rotation --------------------------------------------------------
int vb_hadamard64(const void* x, int dtype, int rows, int cols, void* out, cudaStream_t stream);

// ---- FP8 wire codec ----------------------------------------------------------------
// packet row = [groups * tile codes][groups fp32 scales], padded to 16 B
int vb_wire_pack(const float* x, long long n, int rows, int groups, int tile, int fmt, uint8_t* packet,
                 long long row_stride, cudaStream_t stream);
int vb_wire_unpack(const uint8_t* packet, long long row_stride, int rows, int groups, int tile, int fmt,
                   int reduce, float* out, long long n, int accumulate, cudaStream_t stream);

// ---- fused communication over peer memory (comm.cu) ---------------------------------
// Every rank maps every rank's symmetric heap; buffers[r] is rank r's heap base in this
// process's address space and offsets are identical on all ranks.
typedef struct VbPeerTable {
  void* buffers[16];
  int world, rank;
} VbPeerTable;

// Path 1 (non-owner): quantise the local fp32 bucket tile by tile and store codes + scales straight
// into the owner's receive slot, then raise the owner's flag for this source rank.
int vb_reduce_push_fp8(const float* bucket, long long n, int tile, int fmt, void* dst_codes, float* dst_scales,
                       int* dst_flag, const int* ack_flag, const int* generation, unsigned int* counter,
                       long long wait_clocks, int max_blocks, int* status, cudaStream_t stream);
// Path 1 (owner): wait for every peer's flag, then accum += sum over ranks (ascending, fp32) of the
// dequantised contributions; the owner's own bucket goes through the same quantise-dequantise.
int vb_reduce_accumulate_fp8(const float* bucket, long long n, int tile, int fmt, const void* recv,
                             long long slot_stride, long long scales_offset, const int* flags,
                             const VbPeerTable* peers, long long ack_offset, const int* generation, float* accum,
                             unsigned int* counter, long long wait_clocks, int max_blocks, int* status,
                             cudaStream_t stream);
// Path 1 over a device table of 64-byte rows {src, n, codes, scales, accum, slot_stride, scales_offset, reserved}
// (prefix: int64[buckets + 1] prefix sums of tiles): one launch pushes all buckets owned elsewhere and raises
// flag[rank] at every peer; one launch accumulates all owned buckets after every peer's flag and acknowledges.
int vb_reduce_push_many(const void* table, const long long* prefix, int buckets, long long total_tiles, int tile, int fmt,
                        const VbPeerTable* peers, long long flag_offset, const int* ack_flags, const int* generation,
                        unsigned int* counter, long long wait_clocks, int max_blocks, int* status, cudaStream_t stream);
int vb_reduce_accumulate_many(const void* table, const long long* prefix, int buckets, long long total_tiles, int tile,
                              int fmt, const VbPeerTable* peers, const int* flags, long long ack_offset,
                              const int* generation, unsigned int* counter, long long wait_clocks, int max_blocks,
                              int* status, cudaStream_t stream);
// Path 2: in-place FP8 all-reduce with a second quantisation of the partial sums.
int vb_allreduce_requant_fp8(float* value, long long n, int tile, int fmt, const VbPeerTable* peers,
                             long long a2a_offset, long long gather_offset, long long slot,
                             long long a2a_flag_offset, long long gather_flag_offset, int generation,
                             unsigned int* counters, long long wait_clocks, int max_blocks, int* status,
                             cudaStream_t stream);
// Path 4: master -> (EMA) -> FP8 codes stored into every rank (shard_rows == 0) or per-row-slab owner.
int vb_quantize_push(const void* master, int master_dtype, long long rows, long long cols, const float* scale,
                     float limit, int fmt, void* ema, int ema_dtype, float decay, const VbPeerTable* peers,
                     long long dst_offset, long long shard_rows, int max_blocks, cudaStream_t stream);
int vb_byte_push(const void* src, long long bytes, const VbPeerTable* peers, long long dst_offset,
                 long long shard_bytes, int max_blocks, cudaStream_t stream);
// Path 4, fused: the whole write-back of an owner in two launches over a device table of 128-byte rows
// {master, ema, amax slot, n, slab_elems, dst_offset, header_offset, base_index, limit, history_len,
//  master_dtype, ema_dtype, mode, out_dtype}: (A) EMA lerp + per-tensor amax, (B) scale + encode / cast +
// stores into the rank that holds each row slab + header (scale, history slot) into every rank.
// prefix: int32[rows + 1] prefix sums of 4096-element chunks; amax slots must be zero on entry.
int vb_multi_writeback(const void* table, const int* prefix, int rows, int blocks, float decay, int with_ema,
                       const VbPeerTable* peers, long long calls, cudaStream_t stream);
// flags[rank] = value on every peer (and optionally on this rank); bounded wait on local flags
int vb_signal(const VbPeerTable* peers, long long flag_offset, int value, int include_self, cudaStream_t stream);
int vb_wait_flags(const int* flags, int count, int skip, int expected, long long wait_clocks, int* status,
                  cudaStream_t stream);
// Path 3: pull every peer's row slab of every parameter of a unit into the local full buffer.
// entries: device array of {shard_offset, shard_bytes, full_offset} (3 x int64 each);
// piece_prefix: device int64[num_entries * world + 1] prefix sums of 64 KiB pieces per (entry, visit slot).
int vb_gather_pull(const void* entries, int num_entries, const VbPeerTable* peers, long long shard_region_offset,
                   void* full, const long long* piece_prefix, unsigned int* piece_counts, int* panel_flags,
                   int generation, long long total_pieces, int max_blocks, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
