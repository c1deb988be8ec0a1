// Producer-fused quantisers for transformer blocks (sm_100a, bf16 activations).
//
// The reference quantises the output of LayerNorm/modulate and of GELU in separate passes
// (viola/nn/linear.py:38-53 is fed by PyTorch LayerNorm / mul / add / gelu kernels in
// experiments/dit.py:33-39).  Here the producing elementwise work is folded into the two passes a
// per-tensor "current" scale needs anyway:
//   pass 1  vb_ln_stats_amax : per-row mean / rstd of x, and the global amax of
//                              h = (x - mean) * rstd * (1 + scale[b]) + shift[b]   -> FP8 scale
//           vb_act_amax      : global amax of act(z)                               -> FP8 scale
//   pass 2  vb_fused_quantize: recompute h (or act(z)) from x and emit FP8 codes rowwise and
//                              transposed; h itself is never written to memory.
// and the matching backward of LayerNorm+modulate in one kernel (vb_ln_modulate_backward).
#include "api.h"
#include "common/numerics.cuh"

namespace vb {

enum FusedMode : int { kModeLnModulate = 1, kModeGelu = 2, kModeSilu = 3 };

__device__ __forceinline__ float gelu_tanh(float g) {
  const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
  return 0.5f * g * (1.f + t);
}
__device__ __forceinline__ float apply_act(float v, int mode) {
  if (mode == kModeGelu) return gelu_tanh(v);
  if (mode == kModeSilu) return v / (1.f + __expf(-v));
  return v;
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// amax -> scale with the delayed-scaling history, executed by the last block to finish.
__device__ __forceinline__ void finish_scale(float block_amax, unsigned int* scratch, float* history, int history_len,
                                             long long index, int delayed, float limit, float* scale_out) {
  __shared__ bool last;
  if (threadIdx.x == 0) {
    atomicMax(&scratch[0], __float_as_uint(block_amax));
    __threadfence();
    last = atomicAdd(&scratch[1], 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    const float amax = __uint_as_float(atomicExch(&scratch[0], 0u));
    scratch[1] = 0u;
    float chosen = amax;
    if (history != nullptr) {
      if (delayed && index != 0) {
        float old = 0.f;
        for (int i = 0; i < history_len; ++i) old = fmaxf(old, history[i]);
        chosen = old;
      }
      history[index % history_len] = amax;
    }
    scale_out[0] = fmaxf(chosen, 1e-30f) / limit;
  }
}

__device__ __forceinline__ float block_max(float m) {
  __shared__ float warp_m[8];
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) warp_m[threadIdx.x >> 5] = m;
  __syncthreads();
  float b = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) b = fmaxf(b, warp_m[i]);
  return b;
}

// One warp per row; the row (<= 64 elements per lane) stays in registers between the statistics and
// the modulated amax.  mod_shift / mod_scale are [samples, cols] in bf16; sample = row / tokens.
template <int EPL>
__global__ void __launch_bounds__(256)
ln_stats_amax_kernel(const __nv_bfloat16* __restrict__ x, int rows, int cols, float eps,
                     const __nv_bfloat16* __restrict__ mod_shift, const __nv_bfloat16* __restrict__ mod_scale,
                     int tokens, float* __restrict__ mean_out, float* __restrict__ rstd_out, float* history,
                     int history_len, long long index, int delayed, float limit, float* scale_out,
                     unsigned int* scratch) {
  const int lane = threadIdx.x & 31;
  float amax = 0.f;
  for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += gridDim.x * 8) {
    const __nv_bfloat16* xr = x + (long long)row * cols;
    float v[EPL];
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int c = e * 32 + lane;
      v[e] = c < cols ? __bfloat162float(xr[c]) : 0.f;
      sum += v[e];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / cols;
    float var = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int c = e * 32 + lane;
      const float d = c < cols ? v[e] - mean : 0.f;
      var += d * d;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
    const float rstd = rsqrtf(var / cols + eps);
    if (lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    const long long mod = (long long)(row / tokens) * cols;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int c = e * 32 + lane;
      if (c < cols) {
        const float normed = (v[e] - mean) * rstd;
        const float h = round_bf16(fmaf(normed, 1.f + __bfloat162float(mod_scale[mod + c]), __bfloat162float(mod_shift[mod + c])));
        amax = fmaxf(amax, fabsf(h));
      }
    }
  }
  finish_scale(block_max(amax), scratch, history, history_len, index, delayed, limit, scale_out);
}

__global__ void __launch_bounds__(256)
act_amax_kernel(const __nv_bfloat16* __restrict__ z, long long n, int mode, float* history, int history_len,
                long long index, int delayed, float limit, float* scale_out, unsigned int* scratch) {
  float m = 0.f;
  const long long nvec = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 t = reinterpret_cast<const uint4*>(z)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      m = fmaxf(m, fmaxf(fabsf(round_bf16(apply_act(f.x, mode))), fabsf(round_bf16(apply_act(f.y, mode)))));
    }
  }
  for (long long i = nvec * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(round_bf16(apply_act(__bfloat162float(z[i]), mode))));
  finish_scale(block_max(m), scratch, history, history_len, index, delayed, limit, scale_out);
}

struct FusedArgs {
  int mode;
  const float* mean;
  const float* rstd;
  const __nv_bfloat16* mod_shift;
  const __nv_bfloat16* mod_scale;
  int tokens;
};

__device__ __forceinline__ float fused_value(float v, int r, int c, int cols, const FusedArgs& a) {
  if (a.mode == kModeLnModulate) {
    const float normed = (v - a.mean[r]) * a.rstd[r];
    const long long mod = (long long)(r / a.tokens) * cols + c;
    return round_bf16(fmaf(normed, 1.f + __bfloat162float(a.mod_scale[mod]), __bfloat162float(a.mod_shift[mod])));
  }
  return round_bf16(apply_act(v, a.mode));
}

// 64x64 tiles: rowwise and/or transposed FP8 codes of the transformed input (bf16 source).
__global__ void __launch_bounds__(256)
fused_quantize_kernel(const __nv_bfloat16* __restrict__ x, int rows, int cols, FusedArgs fa,
                      const float* __restrict__ scale_ptr, float limit, int fmt, uint8_t* __restrict__ q,
                      uint8_t* __restrict__ qt) {
  __shared__ __align__(16) uint8_t tile[64][64 + 16];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const float scale = scale_ptr[0];
  const int tr = threadIdx.x >> 2, tc = (threadIdx.x & 3) * 16;
  const int r = r0 + tr, c = c0 + tc;
  uint8_t codes[16];
  if (r < rows && c + 15 < cols && cols % 8 == 0) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint4 t = *reinterpret_cast<const uint4*>(x + (long long)r * cols + c + j * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        codes[j * 8 + 2 * e] = fp8_encode(scaled_clamp(fused_value(f.x, r, c + j * 8 + 2 * e, cols, fa), scale, limit), fmt);
        codes[j * 8 + 2 * e + 1] = fp8_encode(scaled_clamp(fused_value(f.y, r, c + j * 8 + 2 * e + 1, cols, fa), scale, limit), fmt);
      }
    }
  } else {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const bool in = r < rows && c + e < cols;
      const float v = in ? fused_value(__bfloat162float(x[(long long)r * cols + c + e]), r, c + e, cols, fa) : 0.f;
      codes[e] = fp8_encode(scaled_clamp(v, scale, limit), fmt);
    }
  }
  if (q != nullptr && r < rows) {
    if (c + 15 < cols && cols % 16 == 0) {
      *reinterpret_cast<uint4*>(q + (long long)r * cols + c) = *reinterpret_cast<uint4*>(codes);
    } else {
      for (int e = 0; e < 16; ++e)
        if (c + e < cols) q[(long long)r * cols + c + e] = codes[e];
    }
  }
  if (qt != nullptr) {
    *reinterpret_cast<uint4*>(&tile[tr][tc]) = *reinterpret_cast<uint4*>(codes);
    __syncthreads();
    const int oc = threadIdx.x >> 2, orow = (threadIdx.x & 3) * 16;
    uint8_t out[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) out[e] = tile[orow + e][oc];
    const int gr = c0 + oc, gc = r0 + orow;
    if (gr < cols) {
      if (gc + 15 < rows && rows % 16 == 0) {
        *reinterpret_cast<uint4*>(qt + (long long)gr * rows + gc) = *reinterpret_cast<uint4*>(out);
      } else {
        for (int e = 0; e < 16; ++e)
          if (gc + e < rows) qt[(long long)gr * rows + gc + e] = out[e];
      }
    }
  }
}

// Backward of h = LN(x) * (1 + scale[b]) + shift[b] for one warp per row:
//   dx     = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dh * (1 + scale[b])
//   dshift[b] += dh,  dscale[b] += dh * xhat        (fp32 atomics into zero-initialised [samples, cols])
// A block walks `rows_per_block` consecutive rows of ONE sample and reduces dshift / dscale in shared
// memory first, so the global atomics are one per (block, column).
template <int EPL>
__global__ void __launch_bounds__(256)
ln_modulate_backward_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ x,
                            const float* __restrict__ mean, const float* __restrict__ rstd,
                            const __nv_bfloat16* __restrict__ mod_scale, int rows, int cols, int tokens,
                            int rows_per_block, __nv_bfloat16* __restrict__ dx, float* __restrict__ dshift,
                            float* __restrict__ dscale) {
  extern __shared__ float partial[];            // [2][cols]
  float* p_shift = partial;
  float* p_scale = partial + cols;
  for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) partial[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int blocks_per_sample = (tokens + rows_per_block - 1) / rows_per_block;
  const int sample = blockIdx.x / blocks_per_sample;
  const int first = sample * tokens + (blockIdx.x % blocks_per_sample) * rows_per_block;
  const int last = min(min(first + rows_per_block, (sample + 1) * tokens), rows);
  const long long mod = (long long)sample * cols;
  float acc_shift[EPL], acc_scale[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) acc_shift[e] = acc_scale[e] = 0.f;
  for (int row = first + warp; row < last; row += 8) {
    const long long base = (long long)row * cols;
    const float mu = mean[row], rs = rstd[row];
    float g[EPL], xh[EPL];
    float sum_g = 0.f, sum_gx = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int c = e * 32 + lane;
      if (c < cols) {
        const float d = __bfloat162float(dh[base + c]);
        xh[e] = (__bfloat162float(x[base + c]) - mu) * rs;
        g[e] = d * (1.f + __bfloat162float(mod_scale[mod + c]));
        acc_shift[e] += d;
        acc_scale[e] += d * xh[e];
        sum_g += g[e];
        sum_gx += g[e] * xh[e];
      } else {
        g[e] = xh[e] = 0.f;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sum_g += __shfl_xor_sync(0xffffffffu, sum_g, o);
      sum_gx += __shfl_xor_sync(0xffffffffu, sum_gx, o);
    }
    const float mean_g = sum_g / cols, mean_gx = sum_gx / cols;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int c = e * 32 + lane;
      if (c < cols) dx[base + c] = __float2bfloat16_rn(rs * (g[e] - mean_g - xh[e] * mean_gx));
    }
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int c = e * 32 + lane;
    if (c < cols) {
      atomicAdd(&p_shift[c], acc_shift[e]);
      atomicAdd(&p_scale[c], acc_scale[e]);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    atomicAdd(&dshift[mod + c], p_shift[c]);
    atomicAdd(&dscale[mod + c], p_scale[c]);
  }
}

}  // namespace vb

using namespace vb;

#define VB_EPL_SWITCH(cols, ...)                                \
  if ((cols) <= 512) { constexpr int EPL = 16; __VA_ARGS__; }   \
  else if ((cols) <= 1024) { constexpr int EPL = 32; __VA_ARGS__; } \
  else if ((cols) <= 1536) { constexpr int EPL = 48; __VA_ARGS__; } \
  else if ((cols) <= 2048) { constexpr int EPL = 64; __VA_ARGS__; } \
  else return (int)cudaErrorInvalidValue;

extern "C" int vb_ln_stats_amax(const void* x, int rows, int cols, float eps, const void* mod_shift, const void* mod_scale,
                                int tokens, float* mean, float* rstd, float* history, int history_len, long long index,
                                int delayed, float limit, float* scale_out, unsigned int* scratch, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || tokens <= 0) return (int)cudaErrorInvalidValue;
  const int grid = std::min((rows + 7) / 8, 148 * 8);
  VB_EPL_SWITCH(cols, (ln_stats_amax_kernel<EPL><<<grid, 256, 0, stream>>>(
                          (const __nv_bfloat16*)x, rows, cols, eps, (const __nv_bfloat16*)mod_shift,
                          (const __nv_bfloat16*)mod_scale, tokens, mean, rstd, history, history_len, index, delayed, limit,
                          scale_out, scratch)));
  return (int)cudaGetLastError();
}

extern "C" int vb_act_amax(const void* z, long long n, int mode, float* history, int history_len, long long index,
                           int delayed, float limit, float* scale_out, unsigned int* scratch, cudaStream_t stream) {
  if (n <= 0) return (int)cudaErrorInvalidValue;
  const int grid = (int)std::max<long long>(1, std::min<long long>((n / 8 + 255) / 256 / 4, 148 * 8));
  act_amax_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)z, n, mode, history, history_len, index, delayed, limit,
                                            scale_out, scratch);
  return (int)cudaGetLastError();
}

extern "C" int vb_fused_quantize(const void* x, int rows, int cols, int mode, const float* mean, const float* rstd,
                                 const void* mod_shift, const void* mod_scale, int tokens, const float* scale, float limit,
                                 int fmt, void* q, void* qt, cudaStream_t stream) {
  FusedArgs fa{mode, mean, rstd, (const __nv_bfloat16*)mod_shift, (const __nv_bfloat16*)mod_scale, tokens > 0 ? tokens : 1};
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  fused_quantize_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, rows, cols, fa, scale, limit, fmt, (uint8_t*)q,
                                                  (uint8_t*)qt);
  return (int)cudaGetLastError();
}

extern "C" int vb_ln_modulate_backward(const void* dh, const void* x, const float* mean, const float* rstd,
                                       const void* mod_scale, int rows, int cols, int tokens, void* dx, float* dshift,
                                       float* dscale, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || tokens <= 0 || rows % tokens != 0) return (int)cudaErrorInvalidValue;
  const int rows_per_block = 32;
  const int blocks_per_sample = (tokens + rows_per_block - 1) / rows_per_block;
  const int grid = (rows / tokens) * blocks_per_sample;
  const size_t smem = 2 * (size_t)cols * sizeof(float);
  VB_EPL_SWITCH(cols, (ln_modulate_backward_kernel<EPL><<<grid, 256, smem, stream>>>(
                          (const __nv_bfloat16*)dh, (const __nv_bfloat16*)x, mean, rstd, (const __nv_bfloat16*)mod_scale, rows,
                          cols, tokens, rows_per_block, (__nv_bfloat16*)dx, dshift, dscale)));
  return (int)cudaGetLastError();
}
