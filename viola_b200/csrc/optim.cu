// Optimizer-side elementwise kernels (sm_100a): FP8 momentum (1-D tiles / 2-D blocks,
// nearest or stochastic rounding), master-weight update, Adam(W), copy_scaled, the
// 16-bit momentum diagnostic, Newton-Schulz prescale, EMA lerp, gated activations,
// Hadamard-64 and the Philox known-answer helper.
//
// Arithmetic restates viola/optim/_kernels.py:88-293 (momentum: m = beta*(q*s) +
// (1-beta)*g*inv_loss_scale; scale = max(amax,1e-30)/448; nesterov update (1-beta)g +
// beta*m emitted in bf16 before the state is rounded), experiments/momentum16.py:9-22,
// viola/nn/_gated_kernels.py:16-67 and viola/nn/_rotation_kernels.py:11-25.
#include "api.h"
#include "common/numerics.cuh"

namespace vb {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

// --------------------------------------------------------------------------------
// momentum, 1-D tiles: one warp per tile, TILE/32 elements per lane kept in registers
// --------------------------------------------------------------------------------
template <int TILE, typename G>
__global__ void __launch_bounds__(256)
momentum_1d_kernel(const G* __restrict__ grad, long long n, const uint8_t* __restrict__ old_q,
                   const float* __restrict__ old_scale, uint8_t* __restrict__ new_q,
                   float* __restrict__ new_scale, __nv_bfloat16* __restrict__ update, float beta,
                   float inv_loss_scale, int nesterov, int stochastic, unsigned long long step,
                   unsigned long long key) {
  constexpr int EPL = TILE / 32;
  constexpr int VEC = EPL >= 4 ? 4 : EPL;
  constexpr int IT = EPL / VEC;
  const long long blocks = (n + TILE - 1) / TILE;
  const int lane = threadIdx.x & 31;
  const bool q_vec = ((reinterpret_cast<uintptr_t>(old_q) | reinterpret_cast<uintptr_t>(new_q)) & (VEC - 1)) == 0;
  const bool g_vec = (reinterpret_cast<uintptr_t>(grad) & (VEC * sizeof(G) - 1)) == 0;
  const bool u_vec = (reinterpret_cast<uintptr_t>(update) & (VEC * 2 - 1)) == 0;
  for (long long b = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < blocks;
       b += (long long)gridDim.x * (blockDim.x >> 5)) {
    const long long base = b * TILE;
    const float os = old_scale[b];
    const bool full = base + TILE <= n;
    float g[EPL], m[EPL];
    float amax = 0.f;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const long long i0 = base + it * 32 * VEC + lane * VEC;
      uint8_t qc[VEC];
      if (q_vec && VEC == 4) *reinterpret_cast<uint32_t*>(qc) = *reinterpret_cast<const uint32_t*>(old_q + i0);
      else if (q_vec && VEC == 2) *reinterpret_cast<uint16_t*>(qc) = *reinterpret_cast<const uint16_t*>(old_q + i0);
      else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) qc[e] = old_q[i0 + e];
      }
      G gv[VEC];
      if (full && g_vec) {
        if constexpr (sizeof(G) * VEC == 16) *reinterpret_cast<uint4*>(gv) = *reinterpret_cast<const uint4*>(grad + i0);
        else if constexpr (sizeof(G) * VEC == 8) *reinterpret_cast<uint2*>(gv) = *reinterpret_cast<const uint2*>(grad + i0);
        else *reinterpret_cast<uint32_t*>(gv) = *reinterpret_cast<const uint32_t*>(grad + i0);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) gv[e] = (i0 + e < n) ? grad[i0 + e] : G(0.f);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const bool in = full || (i0 + e < n);
        const float gg = in ? to_f<G>(gv[e]) * inv_loss_scale : 0.f;
        const float mm = in ? fp8_decode(qc[e], kE4M3) * os : 0.f;
        g[it * VEC + e] = gg;
        m[it * VEC + e] = beta * mm + (1.f - beta) * gg;
        amax = fmaxf(amax, fabsf(m[it * VEC + e]));
      }
    }
    amax = warp_max(amax);
    const float scale = fmaxf(amax, 1e-30f) / 448.f;
    if (lane == 0) new_scale[b] = scale;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const long long i0 = base + it * 32 * VEC + lane * VEC;
      uint8_t qc[VEC];
      __nv_bfloat16 uo[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float mm = m[it * VEC + e];
        float c = fminf(fmaxf(mm / scale, -448.f), 448.f);
        if (mm != mm) c = mm;
        if (stochastic) c = stochastic_e4m3(c, (unsigned long long)(i0 + e), step, key);
        qc[e] = fp8_encode(c, kE4M3);
        const float u = nesterov ? (1.f - beta) * g[it * VEC + e] + beta * mm : mm;
        uo[e] = __float2bfloat16_rn(u);
      }
      // the padded tail of the state is written too (it is part of the buffer)
      if (q_vec && VEC == 4) *reinterpret_cast<uint32_t*>(new_q + i0) = *reinterpret_cast<uint32_t*>(qc);
      else if (q_vec && VEC == 2) *reinterpret_cast<uint16_t*>(new_q + i0) = *reinterpret_cast<uint16_t*>(qc);
      else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) new_q[i0 + e] = qc[e];
      }
      if (full && u_vec) {
        if constexpr (VEC == 4) *reinterpret_cast<uint2*>(update + i0) = *reinterpret_cast<uint2*>(uo);
        else *reinterpret_cast<uint32_t*>(update + i0) = *reinterpret_cast<uint32_t*>(uo);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          if (i0 + e < n) update[i0 + e] = uo[e];
      }
    }
  }
}

// --------------------------------------------------------------------------------
// momentum, 2-D blocks: one warp per (plane, block); two passes over the block
// --------------------------------------------------------------------------------
template <typename G>
__global__ void __launch_bounds__(256)
momentum_2d_kernel(const G* __restrict__ grad, int planes, int rows, int cols, const uint8_t* __restrict__ old_q,
                   const float* __restrict__ old_scale, uint8_t* __restrict__ new_q,
                   float* __restrict__ new_scale, __nv_bfloat16* __restrict__ update, int tr, int tc,
                   float beta, float inv_loss_scale, int nesterov, int stochastic, unsigned long long step,
                   unsigned long long key) {
  const int nr = (rows + tr - 1) / tr, nc = (cols + tc - 1) / tc;
  const long long tiles = (long long)planes * nr * nc;
  const int lane = threadIdx.x & 31;
  for (long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < tiles;
       t += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int plane = (int)(t / ((long long)nr * nc));
    const int br = (int)((t / nc) % nr), bc = (int)(t % nc);
    const float os = old_scale[t];
    float amax = 0.f;
    for (int e = lane; e < tr * tc; e += 32) {
      const int y = br * tr + e / tc, x = bc * tc + e % tc;
      if (y < rows && x < cols) {
        const long long i = ((long long)plane * rows + y) * cols + x;
        const float g = to_f<G>(grad[i]) * inv_loss_scale;
        const float m = beta * (fp8_decode(old_q[i], kE4M3) * os) + (1.f - beta) * g;
        amax = fmaxf(amax, fabsf(m));
      }
    }
    amax = warp_max(amax);
    const float scale = fmaxf(amax, 1e-30f) / 448.f;
    __syncwarp();
    for (int e = lane; e < tr * tc; e += 32) {
      const int y = br * tr + e / tc, x = bc * tc + e % tc;
      if (y < rows && x < cols) {
        const long long i = ((long long)plane * rows + y) * cols + x;
        const float g = to_f<G>(grad[i]) * inv_loss_scale;
        const float m = beta * (fp8_decode(old_q[i], kE4M3) * os) + (1.f - beta) * g;
        float c = fminf(fmaxf(m / scale, -448.f), 448.f);
        if (m != m) c = m;
        if (stochastic) c = stochastic_e4m3(c, (unsigned long long)i, step, key);
        new_q[i] = fp8_encode(c, kE4M3);
        update[i] = __float2bfloat16_rn(nesterov ? (1.f - beta) * g + beta * m : m);
      }
    }
    __syncwarp();
    if (lane == 0) new_scale[t] = scale;
  }
}

// --------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
weight_update_kernel(void* __restrict__ weight, int wdt, const void* __restrict__ update, int udt, long long n,
                     float lr, float decay, float update_scale, int stochastic, unsigned long long step,
                     unsigned long long key, long long offset) {
  const float keep = 1.f - lr * decay, rate = lr * update_scale;
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (long long)gridDim.x * blockDim.x) {
    const float v = load_as_float(weight, j, wdt) * keep - rate * load_as_float(update, j, udt);
    store_rounded(weight, j, wdt, v, stochastic != 0, (unsigned long long)(j + offset), step, key);
  }
}

__global__ void __launch_bounds__(256)
adam_kernel(void* __restrict__ weight, int wdt, const void* __restrict__ grad, int gdt, void* __restrict__ first,
            void* __restrict__ second, int sdt, long long n, float lr, float decay, float b1, float b2,
            float inv_c1, float inv_c2, float eps, int adamw, int maximize, int stochastic,
            unsigned long long step, unsigned long long key, long long offset) {
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (long long)gridDim.x * blockDim.x) {
    float w = load_as_float(weight, j, wdt);
    float g = load_as_float(grad, j, gdt);
    if (maximize) g = -g;
    if (!adamw) g = g + decay * w;
    const float m = b1 * load_as_float(first, j, sdt) + (1.f - b1) * g;
    const float v = b2 * load_as_float(second, j, sdt) + (1.f - b2) * g * g;
    store_from_float(first, j, sdt, m);
    store_from_float(second, j, sdt, v);
    if (adamw) w = w * (1.f - lr * decay);
    const float value = w - lr * (m * inv_c1) / (sqrtf(v * inv_c2) + eps);
    store_rounded(weight, j, wdt, value, stochastic != 0, (unsigned long long)(j + offset), step, key);
  }
}

__global__ void __launch_bounds__(256)
copy_scaled_kernel(const void* __restrict__ update, int dt, void* __restrict__ out, int odt, long long src,
                   long long dst, long long count, float scale) {
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < count; j += (long long)gridDim.x * blockDim.x)
    store_from_float(out, dst + j, odt, load_as_float(update, src + j, dt) * scale);
}

__global__ void __launch_bounds__(256)
momentum16_kernel(const void* __restrict__ grad, int gdt, void* __restrict__ mom, int mdt,
                  __nv_bfloat16* __restrict__ out, long long n, float beta, int nesterov) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float g = load_as_float(grad, i, gdt);
    const float fresh = beta * load_as_float(mom, i, mdt) + (1.f - beta) * g;
    out[i] = __float2bfloat16_rn(nesterov ? (1.f - beta) * g + beta * fresh : fresh);
    store_from_float(mom, i, mdt, fresh);
  }
}

// sum of squares of x rounded to `round_dt` first (Newton-Schulz normalises the bf16/fp16 copy).  Reproducible:
// every block parks its partial sum, the last block of a tensor (ticket, self-resetting) adds them in block order.
// The scratch is file-scope device memory shared by all launches, which therefore must not overlap in time
// (the optimizer issues them on one stream); at most kSumsqBatch tensors x kSumsqBlocks blocks per launch.
constexpr int kSumsqBlocks = 256, kSumsqBatch = 1024;
static __device__ float g_sumsq_partial[kSumsqBatch * kSumsqBlocks];
static __device__ unsigned int g_sumsq_ticket[kSumsqBatch];

__global__ void __launch_bounds__(256)
sumsq_kernel(const void* __restrict__ x, int dt, int round_dt, long long n, float* __restrict__ accum) {
  // blockIdx.y selects one of gridDim.y stacked tensors of n elements each
  accum += blockIdx.y;
  const long long base = (long long)blockIdx.y * n;
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = load_as_float(x, base + i, dt);
    if (round_dt == kBF16) v = __bfloat162float(__float2bfloat16_rn(v));
    else if (round_dt == kF16) v = __half2float(__float2half_rn(v));
    s += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float red[8];
  __shared__ bool last;
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    g_sumsq_partial[blockIdx.y * kSumsqBlocks + blockIdx.x] = t;
    __threadfence();
    last = atomicAdd(&g_sumsq_ticket[blockIdx.y], 1u) == gridDim.x - 1;
    if (last) {
      g_sumsq_ticket[blockIdx.y] = 0u;
      __threadfence();
      float total = 0.f;
      for (int b = 0; b < (int)gridDim.x; ++b) total += __ldcg(&g_sumsq_partial[blockIdx.y * kSumsqBlocks + b]);
      *accum += total;
    }
  }
}

// out = x / (sqrt(sumsq) + eps), optionally also out_t = out^T (64x64 tiles through smem)
__global__ void __launch_bounds__(256)
ns_prescale_kernel(const void* __restrict__ x, int dt, int rows, int cols, const float* __restrict__ sumsq,
                   float eps, void* __restrict__ out, void* __restrict__ out_t, int odt) {
  __shared__ float tile[64][65];
  // blockIdx.z selects one of the stacked matrices
  const float inv = 1.f / (sqrtf(sumsq[blockIdx.z]) + eps);
  const long long plane = (long long)blockIdx.z * rows * cols;
  const int esize = dt == kF32 ? 4 : 2, osize = odt == kF32 ? 4 : 2;
  x = reinterpret_cast<const char*>(x) + plane * esize;
  if (out != nullptr) out = reinterpret_cast<char*>(out) + plane * osize;
  if (out_t != nullptr) out_t = reinterpret_cast<char*>(out_t) + plane * osize;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  // bf16 in, bf16 out, no transposed copy, rows of whole 16-byte pieces: eight elements per access
  if (out_t == nullptr && dt == kBF16 && odt == kBF16 && (cols & 7) == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    for (int i = threadIdx.x; i < 64 * 8; i += blockDim.x) {
      const int r = r0 + (i >> 3), c = c0 + (i & 7) * 8;
      if (r >= rows || c >= cols) continue;
      const long long at = (long long)r * cols + c;
      uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + at);
      uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
        const __nv_bfloat162 scaled = __halves2bfloat162(__float2bfloat16_rn(f.x * inv), __float2bfloat16_rn(f.y * inv));
        w[e] = *reinterpret_cast<const uint32_t*>(&scaled);
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + at) = raw;
    }
    return;
  }
  for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
    const int tr = i >> 6, tc = i & 63;
    const int r = r0 + tr, c = c0 + tc;
    float v = 0.f;
    if (r < rows && c < cols) {
      v = load_as_float(x, (long long)r * cols + c, dt);
      if (odt == kBF16) v = __bfloat162float(__float2bfloat16_rn(v));
      else if (odt == kF16) v = __half2float(__float2half_rn(v));
      v = v * inv;
      if (out != nullptr) store_from_float(out, (long long)r * cols + c, odt, v);
    }
    tile[tr][tc] = v;
  }
  if (out_t == nullptr) return;
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
    const int tc = i >> 6, tr = i & 63;  // output row = source column
    const int r = r0 + tr, c = c0 + tc;
    if (r < rows && c < cols) store_from_float(out_t, (long long)c * rows + r, odt, tile[tr][tc]);
  }
}

__global__ void __launch_bounds__(256)
ema_lerp_kernel(void* __restrict__ ema, int edt, const void* __restrict__ master, int mdt, long long n, float decay) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float e = load_as_float(ema, i, edt) * decay;
    store_from_float(ema, i, edt, fmaf(1.f - decay, load_as_float(master, i, mdt), e));
  }
}

__global__ void philox_kat_kernel(unsigned long long element, unsigned long long step, unsigned long long key,
                                  unsigned int* out, int count) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = philox(element + i, step, key);
}

// --------------------------------------------------------------------------------
// gated activation (unfused)
// --------------------------------------------------------------------------------
__device__ __forceinline__ float gate_act(float g, int act) {
  if (act == VB_ACT_SILU) return g / (1.f + __expf(-g));
  if (act == VB_ACT_RELU) return fmaxf(g, 0.f);
  float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
  return 0.5f * g * (1.f + t);
}
__device__ __forceinline__ float gate_act_grad(float g, int act) {
  if (act == VB_ACT_SILU) {
    float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  if (act == VB_ACT_RELU) return g > 0.f ? 1.f : 0.f;
  float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * g * g);
}
__global__ void __launch_bounds__(256)
gated_forward_kernel(const void* __restrict__ gu, int dt, long long rows, int hidden, int act, void* __restrict__ out) {
  const long long n = rows * hidden;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / hidden, c = i % hidden;
    const float g = load_as_float(gu, r * 2 * hidden + c, dt), u = load_as_float(gu, r * 2 * hidden + hidden + c, dt);
    store_from_float(out, i, dt, gate_act(g, act) * u);
  }
}
__global__ void __launch_bounds__(256)
gated_backward_kernel(const void* __restrict__ gu, const void* __restrict__ dh, int dt, long long rows, int hidden,
                      int act, void* __restrict__ dgu) {
  const long long n = rows * hidden;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / hidden, c = i % hidden;
    const float g = load_as_float(gu, r * 2 * hidden + c, dt), u = load_as_float(gu, r * 2 * hidden + hidden + c, dt);
    const float d = load_as_float(dh, i, dt);
    store_from_float(dgu, r * 2 * hidden + c, dt, d * u * gate_act_grad(g, act));
    store_from_float(dgu, r * 2 * hidden + hidden + c, dt, d * gate_act(g, act));
  }
}

// --------------------------------------------------------------------------------
// Hadamard-64: H64 = H4 (x) H4 (x) H4, H4 = (ones - 2 flip(eye)) / 2; self-inverse.
// One warp per (row, 64-column group); each lane owns 2 elements, stages go through smem.
// --------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
hadamard64_kernel(const void* __restrict__ x, int dt, long long rows, int cols, void* __restrict__ out) {
  __shared__ float buf[8][2][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = cols / 64;
  const long long total = rows * groups;
  for (long long w = (long long)blockIdx.x * 8 + warp; w < total; w += (long long)gridDim.x * 8) {
    const long long r = w / groups;
    const int c0 = (int)(w % groups) * 64;
    float* cur = buf[warp][0];
    float* nxt = buf[warp][1];
    cur[lane] = load_as_float(x, r * cols + c0 + lane, dt);
    cur[lane + 32] = load_as_float(x, r * cols + c0 + lane + 32, dt);
    __syncwarp();
#pragma unroll
    for (int stage = 0; stage < 3; ++stage) {
      const int stride = 1 << (2 * stage);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = lane + 32 * h;
        const int base = j / (4 * stride) * (4 * stride) + j % stride;
        const int digit = j / stride % 4;
        const float total4 = (cur[base] + cur[base + stride]) + (cur[base + 2 * stride] + cur[base + 3 * stride]);
        nxt[j] = total4 * 0.5f - cur[base + (3 - digit) * stride];
      }
      __syncwarp();
      float* t = cur; cur = nxt; nxt = t;
    }
    store_from_float(out, r * cols + c0 + lane, dt, cur[lane]);
    store_from_float(out, r * cols + c0 + lane + 32, dt, cur[lane + 32]);
    __syncwarp();
  }
}

static inline int grid_for(long long n, int per_block = 256) {
  long long b = (n + per_block - 1) / per_block;
  if (b < 1) b = 1;
  return (int)std::min<long long>(b, 148LL * 16);
}

}  // namespace vb

using namespace vb;

template <typename G>
static int launch_m1d(const void* grad, long long n, const uint8_t* oq, const float* os, uint8_t* nq, float* ns,
                      void* upd, int tile, float beta, float ils, int nesterov, int stochastic, long long step,
                      unsigned long long key, cudaStream_t stream) {
  const long long blocks = (n + tile - 1) / tile;
  const int grid = (int)std::min<long long>((blocks + 7) / 8, 148LL * 16);
#define VB_M1D(T)                                                                                        \
  momentum_1d_kernel<T, G><<<grid, 256, 0, stream>>>(reinterpret_cast<const G*>(grad), n, oq, os, nq, ns, \
                                                     reinterpret_cast<__nv_bfloat16*>(upd), beta, ils,    \
                                                     nesterov, stochastic, (unsigned long long)step, key)
  switch (tile) {
    case 64: VB_M1D(64); break;
    case 128: VB_M1D(128); break;
    case 256: VB_M1D(256); break;
    case 512: VB_M1D(512); break;
    case 1024: VB_M1D(1024); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef VB_M1D
  return (int)cudaGetLastError();
}

extern "C" int vb_momentum_1d(const void* grad, int grad_dtype, long long n, const uint8_t* old_q,
                              const float* old_scale, uint8_t* new_q, float* new_scale, void* update_bf16,
                              int tile_size, float beta, float inv_loss_scale, int nesterov, int stochastic,
                              long long step, unsigned long long key, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (grad_dtype == kF32) return launch_m1d<float>(grad, n, old_q, old_scale, new_q, new_scale, update_bf16, tile_size, beta, inv_loss_scale, nesterov, stochastic, step, key, stream);
  if (grad_dtype == kBF16) return launch_m1d<__nv_bfloat16>(grad, n, old_q, old_scale, new_q, new_scale, update_bf16, tile_size, beta, inv_loss_scale, nesterov, stochastic, step, key, stream);
  if (grad_dtype == kF16) return launch_m1d<__half>(grad, n, old_q, old_scale, new_q, new_scale, update_bf16, tile_size, beta, inv_loss_scale, nesterov, stochastic, step, key, stream);
  return (int)cudaErrorInvalidValue;
}

extern "C" int vb_momentum_2d(const void* grad, int grad_dtype, int planes, int rows, int cols,
                              const uint8_t* old_q, const float* old_scale, uint8_t* new_q, float* new_scale,
                              void* update_bf16, int tr, int tc, float beta, float inv_loss_scale, int nesterov,
                              int stochastic, long long step, unsigned long long key, cudaStream_t stream) {
  const long long tiles = (long long)planes * ((rows + tr - 1) / tr) * ((cols + tc - 1) / tc);
  if (tiles <= 0) return 0;
  const int grid = (int)std::min<long long>((tiles + 7) / 8, 148LL * 16);
  __nv_bfloat16* upd = reinterpret_cast<__nv_bfloat16*>(update_bf16);
  if (grad_dtype == kF32) momentum_2d_kernel<float><<<grid, 256, 0, stream>>>(reinterpret_cast<const float*>(grad), planes, rows, cols, old_q, old_scale, new_q, new_scale, upd, tr, tc, beta, inv_loss_scale, nesterov, stochastic, (unsigned long long)step, key);
  else if (grad_dtype == kBF16) momentum_2d_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(grad), planes, rows, cols, old_q, old_scale, new_q, new_scale, upd, tr, tc, beta, inv_loss_scale, nesterov, stochastic, (unsigned long long)step, key);
  else if (grad_dtype == kF16) momentum_2d_kernel<__half><<<grid, 256, 0, stream>>>(reinterpret_cast<const __half*>(grad), planes, rows, cols, old_q, old_scale, new_q, new_scale, upd, tr, tc, beta, inv_loss_scale, nesterov, stochastic, (unsigned long long)step, key);
  else return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

extern "C" int vb_weight_update(void* weight, int weight_dtype, const void* update, int update_dtype, long long n,
                                float lr, float decay, float update_scale, int stochastic, long long step,
                                unsigned long long key, long long offset, cudaStream_t stream) {
  if (n <= 0) return 0;
  weight_update_kernel<<<grid_for(n), 256, 0, stream>>>(weight, weight_dtype, update, update_dtype, n, lr, decay,
                                                        update_scale, stochastic, (unsigned long long)step, key, offset);
  return (int)cudaGetLastError();
}

extern "C" int vb_adam_update(void* weight, int weight_dtype, const void* grad, int grad_dtype, void* first,
                              void* second, int state_dtype, long long n, float lr, float decay, float b1, float b2,
                              float inv_c1, float inv_c2, float eps, int adamw, int maximize, int stochastic,
                              long long step, unsigned long long key, long long offset, cudaStream_t stream) {
  if (n <= 0) return 0;
  adam_kernel<<<grid_for(n), 256, 0, stream>>>(weight, weight_dtype, grad, grad_dtype, first, second, state_dtype, n,
                                               lr, decay, b1, b2, inv_c1, inv_c2, eps, adamw, maximize, stochastic,
                                               (unsigned long long)step, key, offset);
  return (int)cudaGetLastError();
}

extern "C" int vb_copy_scaled(const void* update, int dtype, void* out, int out_dtype, long long src, long long dst,
                              long long count, float scale, cudaStream_t stream) {
  if (count <= 0) return 0;
  copy_scaled_kernel<<<grid_for(count), 256, 0, stream>>>(update, dtype, out, out_dtype, src, dst, count, scale);
  return (int)cudaGetLastError();
}

extern "C" int vb_momentum16(const void* grad, int grad_dtype, void* momentum, int momentum_dtype, void* update_bf16,
                             long long n, float beta, int nesterov, cudaStream_t stream) {
  if (n <= 0) return 0;
  momentum16_kernel<<<grid_for(n), 256, 0, stream>>>(grad, grad_dtype, momentum, momentum_dtype,
                                                     reinterpret_cast<__nv_bfloat16*>(update_bf16), n, beta, nesterov);
  return (int)cudaGetLastError();
}

extern "C" int vb_sumsq(const void* x, int dtype, long long n, float* accum, int batch, cudaStream_t stream) {
  // `dtype` packs the storage dtype in the low byte and the rounding dtype in the next byte.
  if (n <= 0 || batch <= 0) return 0;
  const int esize = (dtype & 0xff) == kF32 ? 4 : 2;
  for (int first = 0; first < batch; first += kSumsqBatch) {       // the scratch holds kSumsqBatch tensors per launch
    const int count = std::min(batch - first, kSumsqBatch);
    dim3 grid(std::min(grid_for(n, 1024), kSumsqBlocks), count);
    sumsq_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const char*>(x) + (long long)first * n * esize, dtype & 0xff,
                                           (dtype >> 8) & 0xff, n, accum + first);
  }
  return (int)cudaGetLastError();
}

extern "C" int vb_ns_prescale(const void* x, int dtype, int rows, int cols, const float* sumsq, float eps, void* out,
                              void* out_t, int out_dtype, int batch, cudaStream_t stream) {
  dim3 grid((cols + 63) / 64, (rows + 63) / 64, batch);
  ns_prescale_kernel<<<grid, 256, 0, stream>>>(x, dtype, rows, cols, sumsq, eps, out, out_t, out_dtype);
  return (int)cudaGetLastError();
}

extern "C" int vb_ema_lerp(void* ema, int ema_dtype, const void* master, int master_dtype, long long n, float decay,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  ema_lerp_kernel<<<grid_for(n), 256, 0, stream>>>(ema, ema_dtype, master, master_dtype, n, decay);
  return (int)cudaGetLastError();
}

extern "C" int vb_philox_kat(unsigned long long element, unsigned long long step, unsigned long long key,
                             unsigned int* out, int count, cudaStream_t stream) {
  philox_kat_kernel<<<(count + 127) / 128, 128, 0, stream>>>(element, step, key, out, count);
  return (int)cudaGetLastError();
}

extern "C" int vb_gated_forward(const void* gu, int dtype, int rows, int hidden, int activation, void* out,
                                cudaStream_t stream) {
  const long long n = (long long)rows * hidden;
  if (n <= 0) return 0;
  gated_forward_kernel<<<grid_for(n), 256, 0, stream>>>(gu, dtype, rows, hidden, activation, out);
  return (int)cudaGetLastError();
}
extern "C" int vb_gated_backward(const void* gu, const void* dh, int dtype, int rows, int hidden, int activation,
                                 void* dgu, cudaStream_t stream) {
  const long long n = (long long)rows * hidden;
  if (n <= 0) return 0;
  gated_backward_kernel<<<grid_for(n), 256, 0, stream>>>(gu, dh, dtype, rows, hidden, activation, dgu);
  return (int)cudaGetLastError();
}

extern "C" int vb_hadamard64(const void* x, int dtype, int rows, int cols, void* out, cudaStream_t stream) {
  if (cols % 64 != 0) return (int)cudaErrorInvalidValue;
  const long long groups = (long long)rows * (cols / 64);
  if (groups <= 0) return 0;
  hadamard64_kernel<<<(int)std::min<long long>((groups + 7) / 8, 148LL * 16), 256, 0, stream>>>(x, dtype, rows, cols, out);
  return (int)cudaGetLastError();
}
