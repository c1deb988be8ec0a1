// Producer-fused quantisers for transformer blocks (sm_100a; bf16 or fp32 residual stream).
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
// and the matching backward of LayerNorm+modulate in one kernel (vb_ln_modulate_backward), plus the
// gated residual x + gate[b] * y with its backward (vb_gate_residual / vb_gate_residual_backward).
// Rows are walked in 16-byte vectors: a lane owns the 8-element chunks lane, lane + 32, ... of a row.
#include <mutex>
#include <set>

#include "api.h"
#include "common/numerics.cuh"

namespace vb {

enum FusedMode : int { kModeLnModulate = 1, kModeGelu = 2, kModeSilu = 3 };

// tanh-GELU as g * sigmoid(2u), u = sqrt(2/pi) (g + 0.044715 g^3): 0.5 (1 + tanh u) == 1 / (1 + exp(-2u)).
// One ex2 and one fast reciprocal per element; the ~1e-6 relative error is far below the bf16 rounding
// that follows.  Saturates cleanly: exp(-2u) -> inf gives 0, -> 0 gives g.
__device__ __forceinline__ float gelu_tanh(float g) {
  const float u2 = 1.5957691216057308f * (g + 0.044715f * g * g * g);
  return __fdividef(g, 1.f + __expf(-u2));
}
// act(v) and act'(v) from one exponential.  GELU: with s = sigmoid(2u), 1 - tanh^2 u = 4 s (1 - s).
__device__ __forceinline__ float apply_act_with_slope(float v, int mode, float& slope) {
  if (mode == kModeGelu) {
    const float v2 = v * v;
    const float s = __fdividef(1.f, 1.f + __expf(-1.5957691216057308f * v * fmaf(0.044715f, v2, 1.f)));
    slope = fmaf(1.5957691216057308f * v * s * (1.f - s), fmaf(0.134145f, v2, 1.f), s);
    return v * s;
  }
  const float s = __fdividef(1.f, 1.f + __expf(-v));
  slope = s * fmaf(v, 1.f - s, 1.f);
  return v * s;
}
__device__ __forceinline__ float apply_act(float v, int mode) {
  if (mode == kModeGelu) return gelu_tanh(v);
  if (mode == kModeSilu) return __fdividef(v, 1.f + __expf(-v));
  return v;
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// 8 consecutive elements <-> fp32 registers (bf16: one 16-byte access, fp32: two)
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    v[2 * e] = f.x;
    v[2 * e + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 t;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4*>(p) = t;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}

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

// One warp per row; the row (VPL chunks of 8 elements per lane) stays in registers between the statistics
// and the modulated amax.  mod_shift / mod_scale are bf16 rows of pitch mod_stride; sample = row / tokens.
template <typename T, int VPL>
__global__ void __launch_bounds__(256)
ln_stats_amax_kernel(const T* __restrict__ x, int rows, int cols, float eps,
                     const __nv_bfloat16* __restrict__ mod_shift, const __nv_bfloat16* __restrict__ mod_scale,
                     long long mod_stride, int tokens, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                     float* history, int history_len, long long index, int delayed, float limit, float* scale_out,
                     unsigned int* scratch) {
  const int lane = threadIdx.x & 31;
  const int chunks = cols >> 3;
  float amax = 0.f;
  for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += gridDim.x * 8) {
    const T* xr = x + (long long)row * cols;
    float v[VPL][8];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int chunk = lane + 32 * j;
      if (chunk < chunks) {
        load8(xr + chunk * 8, v[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += v[j][e];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / cols;
    float var = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      if (lane + 32 * j < chunks) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = v[j][e] - mean;
          var += d * d;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
    const float rstd = rsqrtf(var / cols + eps);
    if (lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    const long long mod = (long long)(row / tokens) * mod_stride;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int chunk = lane + 32 * j;
      if (chunk < chunks) {
        float sc[8], sh[8];
        load8(mod_scale + mod + chunk * 8, sc);
        load8(mod_shift + mod + chunk * 8, sh);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          amax = fmaxf(amax, fabsf(round_bf16(fmaf((v[j][e] - mean) * rstd, 1.f + sc[e], sh[e]))));
      }
    }
  }
  finish_scale(block_max(amax), scratch, history, history_len, index, delayed, limit, scale_out);
}

// amax of act(z) without evaluating act per element.  tanh-GELU and SiLU fall from 0 to one minimum at z0 and
// rise from there, so |act| over a set is largest at one of three points: the largest z, the smallest z >= z0, or
// the largest z < z0.  The pass therefore tracks two maxima and one minimum (no transcendental: the exact amax pass
// was bound by the exponential unit, not by memory), and the last block evaluates act at those three points with
// the very function the encode pass uses.  A NaN anywhere gives amax = +inf, as in the other amax kernels.
// Partials go through file-scope device scratch: launches of this kernel must not overlap (one stream).
constexpr int kActAmaxBlocks = 148 * 8;
static __device__ float g_act_partial[kActAmaxBlocks * 4];

__global__ void __launch_bounds__(256)
act_amax_kernel(const __nv_bfloat16* __restrict__ z, long long n, int mode, float* history, int history_len,
                long long index, int delayed, float limit, float* scale_out, unsigned int* scratch) {
  const float z0 = mode == kModeGelu ? -0.75179f : -1.27846f;
  float zmax = -INFINITY, zleft = -INFINITY, zright = INFINITY, bad = 0.f;
  auto see = [&](float v) {
    zmax = fmaxf(zmax, v);
    if (v < z0) zleft = fmaxf(zleft, v);
    else zright = fminf(zright, v);
    if (v != v) bad = 1.f;
  };
  const long long nvec = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float v[8];
    load8(z + i * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) see(v[e]);
  }
  for (long long i = nvec * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    see(__bfloat162float(z[i]));
  // block reduction of (zmax, zleft, zright, bad)
  __shared__ float part[8][4];
  __shared__ bool last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
    zleft = fmaxf(zleft, __shfl_xor_sync(0xffffffffu, zleft, o));
    zright = fminf(zright, __shfl_xor_sync(0xffffffffu, zright, o));
    bad = fmaxf(bad, __shfl_xor_sync(0xffffffffu, bad, o));
  }
  if ((threadIdx.x & 31) == 0) {
    float* p = part[threadIdx.x >> 5];
    p[0] = zmax; p[1] = zleft; p[2] = zright; p[3] = bad;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
      zmax = fmaxf(zmax, part[w][0]); zleft = fmaxf(zleft, part[w][1]);
      zright = fminf(zright, part[w][2]); bad = fmaxf(bad, part[w][3]);
    }
    float* mine = g_act_partial + blockIdx.x * 4;
    mine[0] = zmax; mine[1] = zleft; mine[2] = zright; mine[3] = bad;
    __threadfence();
    last = atomicAdd(&scratch[1], 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  // the last block folds every block's partial: strided over its threads, then the same block reduction again
  __threadfence();
  zmax = zleft = -INFINITY; zright = INFINITY; bad = 0.f;
  for (int b = threadIdx.x; b < (int)gridDim.x; b += blockDim.x) {
    const float* other = g_act_partial + b * 4;
    zmax = fmaxf(zmax, __ldcg(other)); zleft = fmaxf(zleft, __ldcg(other + 1));
    zright = fminf(zright, __ldcg(other + 2)); bad = fmaxf(bad, __ldcg(other + 3));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
    zleft = fmaxf(zleft, __shfl_xor_sync(0xffffffffu, zleft, o));
    zright = fminf(zright, __shfl_xor_sync(0xffffffffu, zright, o));
    bad = fmaxf(bad, __shfl_xor_sync(0xffffffffu, bad, o));
  }
  __syncthreads();                     // part[] is reused
  if ((threadIdx.x & 31) == 0) {
    float* p = part[threadIdx.x >> 5];
    p[0] = zmax; p[1] = zleft; p[2] = zright; p[3] = bad;
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
    zmax = fmaxf(zmax, part[w][0]); zleft = fmaxf(zleft, part[w][1]);
    zright = fminf(zright, part[w][2]); bad = fmaxf(bad, part[w][3]);
  }
  scratch[1] = 0u;
  float amax = 0.f;
  if (zmax > -INFINITY) amax = fmaxf(amax, fabsf(round_bf16(apply_act(zmax, mode))));
  if (zleft > -INFINITY) amax = fmaxf(amax, fabsf(round_bf16(apply_act(zleft, mode))));
  if (zright < INFINITY) amax = fmaxf(amax, fabsf(round_bf16(apply_act(zright, mode))));
  if (bad != 0.f) amax = INFINITY;
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

struct FusedArgs {
  int mode;
  const float* mean;
  const float* rstd;
  const __nv_bfloat16* mod_shift;
  const __nv_bfloat16* mod_scale;
  long long mod_stride;
  int tokens;
};

__device__ __forceinline__ float fused_value(float v, int r, int c, int cols, const FusedArgs& a) {
  if (a.mode == kModeLnModulate) {
    const float normed = (v - a.mean[r]) * a.rstd[r];
    const long long mod = (long long)(r / a.tokens) * a.mod_stride + c;
    return round_bf16(fmaf(normed, 1.f + __bfloat162float(a.mod_scale[mod]), __bfloat162float(a.mod_shift[mod])));
  }
  return round_bf16(apply_act(v, a.mode));
}

// Row-wise codes only: a thread turns 16 consecutive elements into one 16-byte store (cols % 16 == 0).
template <typename T>
__global__ void __launch_bounds__(256)
fused_quantize_rows_kernel(const T* __restrict__ x, int rows, int cols, FusedArgs fa,
                           const float* __restrict__ scale_ptr, float limit, int fmt, uint8_t* __restrict__ q,
                           __nv_bfloat16* __restrict__ slope_out) {
  const Divisor scale = make_divisor(scale_ptr[0]);
  const bool clamp = limit < fp8_max(fmt);
  const int per_row = cols >> 4;
  const long long total = (long long)rows * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / per_row);
    const int c = (int)(i - (long long)r * per_row) << 4;
    float v[2][8];
    load8(x + (long long)r * cols + c, v[0]);
    load8(x + (long long)r * cols + c + 8, v[1]);
    if (fa.mode == kModeLnModulate) {
      const float mu = fa.mean[r], rs = fa.rstd[r];
      const long long mod = (long long)(r / fa.tokens) * fa.mod_stride + c;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float sc[8], sh[8];
        load8(fa.mod_scale + mod + 8 * j, sc);
        load8(fa.mod_shift + mod + 8 * j, sh);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = round_bf16(fmaf((v[j][e] - mu) * rs, 1.f + sc[e], sh[e]));
      }
    } else if (slope_out != nullptr) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float slope[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = round_bf16(apply_act_with_slope(v[j][e], fa.mode, slope[e]));
        store8(slope_out + (long long)r * cols + c + 8 * j, slope);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = round_bf16(apply_act(v[j][e], fa.mode));
    }
    uint4 packed;
    uint16_t* codes = reinterpret_cast<uint16_t*>(&packed);
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        codes[j * 4 + e] = fp8_encode2(scaled_clamp(v[j][2 * e], scale, limit, clamp),
                                       scaled_clamp(v[j][2 * e + 1], scale, limit, clamp), fmt);
    *reinterpret_cast<uint4*>(q + (long long)r * cols + c) = packed;
  }
}

// 64x64 tiles: rowwise and/or transposed FP8 codes of the transformed input.
template <typename T>
__global__ void __launch_bounds__(256)
fused_quantize_kernel(const T* __restrict__ x, int rows, int cols, FusedArgs fa,
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
      float f[8];
      load8(x + (long long)r * cols + c + j * 8, f);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        codes[j * 8 + e] = fp8_encode(scaled_clamp(fused_value(f[e], r, c + j * 8 + e, cols, fa), scale, limit), fmt);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const bool in = r < rows && c + e < cols;
      const float v = in ? fused_value((float)x[(long long)r * cols + c + e], r, c + e, cols, fa) : 0.f;
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

// Reproducible per-sample column sums.  Every block of a sample stores its `width` column totals in `workspace`
// (block-major); the last block of the sample to get here (ticket in `tickets[sample]`, left at zero) adds the
// blocks in ascending order and writes the result, so the sums do not depend on scheduling and the outputs
// need no zero-initialisation.  `partial` = [8 warps][width] shared-memory slices with element i of the totals
// at `slot(i)`; `emit(i, total)` stores one finished column sum.
template <typename Slot, typename Emit>
__device__ __forceinline__ void ordered_sample_sums(const float* partial, int width, int sample, int blocks_per_sample,
                                                    float* __restrict__ workspace, unsigned int* __restrict__ tickets,
                                                    Slot slot, Emit emit) {
  __shared__ bool last_block;
  float* mine = workspace + (long long)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += partial[(size_t)w * width + slot(i)];
    mine[i] = total;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    last_block = atomicAdd(&tickets[sample], 1u) == (unsigned)blocks_per_sample - 1;
    if (last_block) tickets[sample] = 0u;
  }
  __syncthreads();
  if (!last_block) return;
  __threadfence();
  const float* first = workspace + (long long)sample * blocks_per_sample * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    // four independent chains keep the loads in flight; the order of additions is still fixed
    float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
    int b = 0;
    for (; b + 4 <= blocks_per_sample; b += 4) {
      t0 += __ldcg(first + (long long)b * width + i);
      t1 += __ldcg(first + (long long)(b + 1) * width + i);
      t2 += __ldcg(first + (long long)(b + 2) * width + i);
      t3 += __ldcg(first + (long long)(b + 3) * width + i);
    }
    for (; b < blocks_per_sample; ++b) t0 += __ldcg(first + (long long)b * width + i);
    emit(i, (t0 + t1) + (t2 + t3));
  }
}

// Backward of h = LN(x) * (1 + scale[b]) + shift[b] for one warp per row:
//   dx     = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dh * (1 + scale[b])
//   dshift[b] = sum dh,  dscale[b] = sum dh * xhat     (fp32 [samples, cols], reproducible, see above)
// A block walks `rows_per_block` consecutive rows of ONE sample.  Each warp keeps its running column sums in
// its own shared-memory slice (element e of chunk c at e * chunks + c, so a warp's accesses are conflict
// free) rather than in registers: that halves the register count and lets two blocks share an SM, which is
// what a latency-bound streaming kernel needs.  dx has the dtype of x.
template <typename T, int VPL>
__global__ void __launch_bounds__(256, 2)
ln_modulate_backward_kernel(const __nv_bfloat16* __restrict__ dh, const T* __restrict__ x,
                            const float* __restrict__ mean, const float* __restrict__ rstd,
                            const __nv_bfloat16* __restrict__ mod_scale, long long mod_stride, int rows, int cols,
                            int tokens, int rows_per_block, const T* __restrict__ grad_in, T* __restrict__ dx,
                            void* __restrict__ dshift, void* __restrict__ dscale, int sums_bf16,
                            float* __restrict__ workspace, unsigned int* __restrict__ tickets) {
  extern __shared__ float partial[];            // [8 warps][2][cols]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunks = cols >> 3;
  const int blocks_per_sample = (tokens + rows_per_block - 1) / rows_per_block;
  const int sample = blockIdx.x / blocks_per_sample;
  const int first = sample * tokens + (blockIdx.x % blocks_per_sample) * rows_per_block;
  const int last = min(min(first + rows_per_block, (sample + 1) * tokens), rows);
  float* my_shift = partial + (size_t)warp * 2 * cols;
  float* my_scale = my_shift + cols;
  for (int i = lane; i < 2 * cols; i += 32) my_shift[i] = 0.f;
  __syncwarp();
  const __nv_bfloat16* gain_row = mod_scale + (long long)sample * mod_stride;
  for (int row = first + warp; row < last; row += 8) {
    const long long base = (long long)row * cols;
    const float mu = mean[row], rs = rstd[row];
    float g[VPL][8], xh[VPL][8];
    float sum_g = 0.f, sum_gx = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int chunk = lane + 32 * j;
      if (chunk < chunks) {
        float d[8], gain[8];
        load8(dh + base + chunk * 8, d);
        load8(x + base + chunk * 8, xh[j]);
        load8(gain_row + chunk * 8, gain);      // L1 resident
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[j][e] = (xh[j][e] - mu) * rs;
          g[j][e] = d[e] * (1.f + gain[e]);
          my_shift[e * chunks + chunk] += d[e];
          my_scale[e * chunks + chunk] += d[e] * xh[j][e];
          sum_g += g[j][e];
          sum_gx += g[j][e] * xh[j][e];
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sum_g += __shfl_xor_sync(0xffffffffu, sum_g, o);
      sum_gx += __shfl_xor_sync(0xffffffffu, sum_gx, o);
    }
    const float mean_g = sum_g / cols, mean_gx = sum_gx / cols;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int chunk = lane + 32 * j;
      if (chunk < chunks) {
        float o[8];
        if (grad_in != nullptr) load8(grad_in + base + chunk * 8, o);     // gradient arriving on the residual path
        else {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += rs * (g[j][e] - mean_g - xh[j][e] * mean_gx);
        store8(dx + base + chunk * 8, o);
      }
    }
  }
  __syncthreads();
  const long long mod = (long long)sample * cols;
  // totals are indexed [shift columns | scale columns]; column c lives at slice position (c % 8) * chunks + c / 8
  ordered_sample_sums(
      partial, 2 * cols, sample, blocks_per_sample, workspace, tickets,
      [=](int i) { const int which = i >= cols, c = i - which * cols; return which * cols + (c & 7) * chunks + (c >> 3); },
      [=](int i, float total) {
        void* base = i >= cols ? dscale : dshift;
        const long long at = mod + (i >= cols ? i - cols : i);
        if (sums_bf16) reinterpret_cast<__nv_bfloat16*>(base)[at] = __float2bfloat16_rn(total);
        else reinterpret_cast<float*>(base)[at] = total;
      });
}

// out = x + gate[b] * y: x / out in T (the residual stream), y and gate in bf16; 8 elements per thread.
template <typename T>
__global__ void __launch_bounds__(256)
gate_residual_kernel(const T* __restrict__ x, const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                     const __nv_bfloat16* __restrict__ y, int rows, int cols, int tokens, T* __restrict__ out) {
  const int per_row = cols >> 3;
  const long long total = (long long)rows * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / per_row);
    const int c = (int)(i - (long long)r * per_row) << 3;
    float xv[8], yv[8], gv[8];
    load8(x + (long long)r * cols + c, xv);
    load8(y + (long long)r * cols + c, yv);
    load8(gate + (long long)(r / tokens) * gate_stride + c, gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) xv[e] = fmaf(gv[e], yv[e], xv[e]);
    store8(out + (long long)r * cols + c, xv);
  }
}

// Backward of the gated residual for the branch: dy = dout * gate[b] (bf16), dgate[b] = sum over the sample's
// rows of dout * y (fp32 [samples, cols], reproducible).  Same block shape as the LayerNorm backward.
template <typename T, int VPL>
__global__ void __launch_bounds__(256)
gate_residual_backward_kernel(const T* __restrict__ dout, const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                              const __nv_bfloat16* __restrict__ y, int rows, int cols, int tokens, int rows_per_block,
                              __nv_bfloat16* __restrict__ dy, void* __restrict__ dgate, int sums_bf16,
                              float* __restrict__ workspace, unsigned int* __restrict__ tickets) {
  extern __shared__ float partial[];            // [8 warps][cols], element e of chunk c at e * chunks + c
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunks = cols >> 3;
  const int blocks_per_sample = (tokens + rows_per_block - 1) / rows_per_block;
  const int sample = blockIdx.x / blocks_per_sample;
  const int first = sample * tokens + (blockIdx.x % blocks_per_sample) * rows_per_block;
  const int last = min(min(first + rows_per_block, (sample + 1) * tokens), rows);
  float gv[VPL][8], acc[VPL][8];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int chunk = lane + 32 * j;
    if (chunk < chunks) load8(gate + (long long)sample * gate_stride + chunk * 8, gv[j]);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  }
  for (int row = first + warp; row < last; row += 8) {
    const long long base = (long long)row * cols;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int chunk = lane + 32 * j;
      if (chunk < chunks) {
        float d[8], yv[8], o[8];
        load8(dout + base + chunk * 8, d);
        load8(y + base + chunk * 8, yv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          o[e] = d[e] * gv[j][e];
          acc[j][e] = fmaf(d[e], yv[e], acc[j][e]);
        }
        store8(dy + base + chunk * 8, o);
      }
    }
  }
  float* mine = partial + (size_t)warp * cols;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int chunk = lane + 32 * j;
    if (chunk < chunks) {
#pragma unroll
      for (int e = 0; e < 8; ++e) mine[e * chunks + chunk] = acc[j][e];
    }
  }
  __syncthreads();
  const long long out_row = (long long)sample * cols;
  ordered_sample_sums(
      partial, cols, sample, blocks_per_sample, workspace, tickets,
      [=](int c) { return (c & 7) * chunks + (c >> 3); },
      [=](int c, float total) {
        if (sums_bf16) reinterpret_cast<__nv_bfloat16*>(dgate)[out_row + c] = __float2bfloat16_rn(total);
        else reinterpret_cast<float*>(dgate)[out_row + c] = total;
      });
}

}  // namespace vb

using namespace vb;

// chunks of 8 elements per lane for one warp per row; rows up to 2048 elements
#define VB_VPL_SWITCH(cols, ...)                                       \
  if ((cols) <= 256) { constexpr int VPL = 1; __VA_ARGS__; }           \
  else if ((cols) <= 512) { constexpr int VPL = 2; __VA_ARGS__; }      \
  else if ((cols) <= 768) { constexpr int VPL = 3; __VA_ARGS__; }      \
  else if ((cols) <= 1024) { constexpr int VPL = 4; __VA_ARGS__; }     \
  else if ((cols) <= 1280) { constexpr int VPL = 5; __VA_ARGS__; }     \
  else if ((cols) <= 1536) { constexpr int VPL = 6; __VA_ARGS__; }     \
  else if ((cols) <= 2048) { constexpr int VPL = 8; __VA_ARGS__; }     \
  else return (int)cudaErrorInvalidValue;

// Rows of one sample a block walks before it reduces its column sums: as many as still leave about two
// blocks per SM's worth of work in the grid (the per-block reduction is a fixed cost), at least 8.
static int pick_rows_per_block(int rows, int tokens) {
  int rpb = 128;
  while (rpb > 8 && (long long)(rows / tokens) * ((tokens + rpb - 1) / rpb) < 148LL * 2) rpb >>= 1;
  // ... but no more than 32 blocks per sample: the last block of a sample adds all of them up (small batches need
  // the blocks: at 16 samples eight blocks per sample leave a fifth of the SMs idle and one block per SM)
  while (rpb < 128 && (tokens + rpb - 1) / rpb > 32) rpb <<= 1;
  return rpb;
}

// Opt a kernel in, once, to the dynamic shared memory its widest supported row needs (8 warps x 2 x 2048 floats).
template <typename Kernel>
static void allow_smem(Kernel kernel) {
  static std::mutex lock;
  static std::set<const void*> configured;
  std::lock_guard<std::mutex> guard(lock);
  if (configured.insert(reinterpret_cast<const void*>(kernel)).second)
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 2 * 2048 * (int)sizeof(float));
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// x_dtype: 0 fp32, 1 bf16 (the dtype codes of numerics.cuh)
extern "C" int vb_ln_stats_amax(const void* x, int x_dtype, int rows, int cols, float eps, const void* mod_shift,
                                const void* mod_scale, long long mod_stride, int tokens, float* mean, float* rstd,
                                float* history, int history_len, long long index, int delayed, float limit,
                                float* scale_out, unsigned int* scratch, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || tokens <= 0 || cols % 8 != 0 || mod_stride % 8 != 0 || x_dtype > kBF16 ||
      !aligned16(x) || !aligned16(mod_shift) || !aligned16(mod_scale))
    return (int)cudaErrorInvalidValue;
  const int grid = std::min((rows + 7) / 8, 148 * 8);
  const __nv_bfloat16* sh = (const __nv_bfloat16*)mod_shift;
  const __nv_bfloat16* sc = (const __nv_bfloat16*)mod_scale;
  if (x_dtype == kBF16) {
    VB_VPL_SWITCH(cols, (ln_stats_amax_kernel<__nv_bfloat16, VPL><<<grid, 256, 0, stream>>>(
                            (const __nv_bfloat16*)x, rows, cols, eps, sh, sc, mod_stride, tokens, mean, rstd, history,
                            history_len, index, delayed, limit, scale_out, scratch)));
  } else {
    VB_VPL_SWITCH(cols, (ln_stats_amax_kernel<float, VPL><<<grid, 256, 0, stream>>>(
                            (const float*)x, rows, cols, eps, sh, sc, mod_stride, tokens, mean, rstd, history, history_len,
                            index, delayed, limit, scale_out, scratch)));
  }
  return (int)cudaGetLastError();
}

extern "C" int vb_act_amax(const void* z, long long n, int mode, float* history, int history_len, long long index,
                           int delayed, float limit, float* scale_out, unsigned int* scratch, cudaStream_t stream) {
  if (n <= 0) return (int)cudaErrorInvalidValue;
  const int grid = (int)std::max<long long>(1, std::min<long long>((n / 8 + 255) / 256 / 4, kActAmaxBlocks));
  act_amax_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)z, n, mode, history, history_len, index, delayed, limit,
                                            scale_out, scratch);
  return (int)cudaGetLastError();
}

template <typename T>
static int launch_fused_quantize(const T* x, int rows, int cols, const FusedArgs& fa, const float* scale, float limit,
                                 int fmt, void* q, void* qt, void* slope, cudaStream_t stream) {
  const bool vector_ok = cols % 16 == 0 && aligned16(x) && aligned16(q) &&
                         (fa.mode != kModeLnModulate ||
                          (fa.mod_stride % 8 == 0 && aligned16(fa.mod_shift) && aligned16(fa.mod_scale)));
  if (qt == nullptr && q != nullptr && vector_ok) {
    const long long total = (long long)rows * (cols / 16);
    const int grid = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256, 148LL * 16));
    if (slope != nullptr && (fa.mode == kModeLnModulate || !aligned16(slope))) return (int)cudaErrorInvalidValue;
    fused_quantize_rows_kernel<T><<<grid, 256, 0, stream>>>(x, rows, cols, fa, scale, limit, fmt, (uint8_t*)q,
                                                            (__nv_bfloat16*)slope);
  } else {
    if (slope != nullptr) return (int)cudaErrorInvalidValue;
    if (cols % 8 != 0 || !aligned16(x)) return (int)cudaErrorInvalidValue;
    dim3 grid((cols + 63) / 64, (rows + 63) / 64);
    fused_quantize_kernel<T><<<grid, 256, 0, stream>>>(x, rows, cols, fa, scale, limit, fmt, (uint8_t*)q, (uint8_t*)qt);
  }
  return (int)cudaGetLastError();
}

extern "C" int vb_fused_quantize(const void* x, int x_dtype, int rows, int cols, int mode, const float* mean,
                                 const float* rstd, const void* mod_shift, const void* mod_scale, long long mod_stride,
                                 int tokens, const float* scale, float limit, int fmt, void* q, void* qt, void* slope,
                                 cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || x_dtype > kBF16) return (int)cudaErrorInvalidValue;
  FusedArgs fa{mode, mean, rstd, (const __nv_bfloat16*)mod_shift, (const __nv_bfloat16*)mod_scale, mod_stride,
               tokens > 0 ? tokens : 1};
  if (x_dtype == kBF16)
    return launch_fused_quantize((const __nv_bfloat16*)x, rows, cols, fa, scale, limit, fmt, q, qt, slope, stream);
  return launch_fused_quantize((const float*)x, rows, cols, fa, scale, limit, fmt, q, qt, slope, stream);
}

extern "C" int vb_ln_modulate_backward(const void* dh, const void* x, int x_dtype, const float* mean, const float* rstd,
                                       const void* mod_scale, long long mod_stride, int rows, int cols, int tokens,
                                       const void* grad_in, void* dx, void* dshift, void* dscale, int sums_bf16, float* workspace,
                                       long long workspace_floats, unsigned int* tickets, int ticket_count,
                                       cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || tokens <= 0 || rows % tokens != 0 || cols % 8 != 0 || mod_stride % 8 != 0 ||
      x_dtype > kBF16 || !aligned16(dh) || !aligned16(x) || !aligned16(dx) || !aligned16(mod_scale) || !aligned16(grad_in))
    return (int)cudaErrorInvalidValue;
  const int rows_per_block = pick_rows_per_block(rows, tokens);
  const int blocks_per_sample = (tokens + rows_per_block - 1) / rows_per_block;
  const int grid = (rows / tokens) * blocks_per_sample;
  const size_t smem = 8 * 2 * (size_t)cols * sizeof(float);
  if (workspace == nullptr || tickets == nullptr || workspace_floats < (long long)grid * 2 * cols || ticket_count < rows / tokens)
    return (int)cudaErrorInvalidValue;
  const __nv_bfloat16* sc = (const __nv_bfloat16*)mod_scale;
  if (x_dtype == kBF16) {
    VB_VPL_SWITCH(cols, (allow_smem(ln_modulate_backward_kernel<__nv_bfloat16, VPL>), ln_modulate_backward_kernel<__nv_bfloat16, VPL><<<grid, 256, smem, stream>>>(
                            (const __nv_bfloat16*)dh, (const __nv_bfloat16*)x, mean, rstd, sc, mod_stride, rows, cols,
                            tokens, rows_per_block, (const __nv_bfloat16*)grad_in, (__nv_bfloat16*)dx, dshift, dscale,
                            sums_bf16, workspace, tickets)));
  } else {
    VB_VPL_SWITCH(cols, (allow_smem(ln_modulate_backward_kernel<float, VPL>), ln_modulate_backward_kernel<float, VPL><<<grid, 256, smem, stream>>>(
                            (const __nv_bfloat16*)dh, (const float*)x, mean, rstd, sc, mod_stride, rows, cols, tokens,
                            rows_per_block, (const float*)grad_in, (float*)dx, dshift, dscale, sums_bf16, workspace, tickets)));
  }
  return (int)cudaGetLastError();
}

// number of blocks the two row-block backward kernels launch (the reduction workspace holds one row of column
// totals per block)
extern "C" int vb_row_block_count(int rows, int tokens) {
  if (rows <= 0 || tokens <= 0 || rows % tokens != 0) return 0;
  const int rows_per_block = pick_rows_per_block(rows, tokens);
  return (rows / tokens) * ((tokens + rows_per_block - 1) / rows_per_block);
}

extern "C" int vb_gate_residual(const void* x, int x_dtype, const void* gate, long long gate_stride, const void* y,
                                int rows, int cols, int tokens, void* out, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || tokens <= 0 || cols % 8 != 0 || gate_stride % 8 != 0 || x_dtype > kBF16 ||
      !aligned16(x) || !aligned16(gate) || !aligned16(y) || !aligned16(out))
    return (int)cudaErrorInvalidValue;
  const long long total = (long long)rows * (cols / 8);
  const int grid = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256, 148LL * 16));
  if (x_dtype == kBF16)
    gate_residual_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate,
                                                                  gate_stride, (const __nv_bfloat16*)y, rows, cols, tokens,
                                                                  (__nv_bfloat16*)out);
  else
    gate_residual_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (const __nv_bfloat16*)gate, gate_stride,
                                                          (const __nv_bfloat16*)y, rows, cols, tokens, (float*)out);
  return (int)cudaGetLastError();
}

extern "C" int vb_gate_residual_backward(const void* dout, int dout_dtype, const void* gate, long long gate_stride,
                                         const void* y, int rows, int cols, int tokens, void* dy, void* dgate, int sums_bf16,
                                         float* workspace, long long workspace_floats, unsigned int* tickets,
                                         int ticket_count, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || tokens <= 0 || rows % tokens != 0 || cols % 8 != 0 || gate_stride % 8 != 0 ||
      dout_dtype > kBF16 || !aligned16(dout) || !aligned16(gate) || !aligned16(y) || !aligned16(dy))
    return (int)cudaErrorInvalidValue;
  const int rows_per_block = pick_rows_per_block(rows, tokens);
  const int blocks_per_sample = (tokens + rows_per_block - 1) / rows_per_block;
  const int grid = (rows / tokens) * blocks_per_sample;
  const size_t smem = 8 * (size_t)cols * sizeof(float);
  if (workspace == nullptr || tickets == nullptr || workspace_floats < (long long)grid * cols || ticket_count < rows / tokens)
    return (int)cudaErrorInvalidValue;
  const __nv_bfloat16* g = (const __nv_bfloat16*)gate;
  if (dout_dtype == kBF16) {
    VB_VPL_SWITCH(cols, (allow_smem(gate_residual_backward_kernel<__nv_bfloat16, VPL>), gate_residual_backward_kernel<__nv_bfloat16, VPL><<<grid, 256, smem, stream>>>(
                            (const __nv_bfloat16*)dout, g, gate_stride, (const __nv_bfloat16*)y, rows, cols, tokens,
                            rows_per_block, (__nv_bfloat16*)dy, dgate, sums_bf16, workspace, tickets)));
  } else {
    VB_VPL_SWITCH(cols, (allow_smem(gate_residual_backward_kernel<float, VPL>), gate_residual_backward_kernel<float, VPL><<<grid, 256, smem, stream>>>(
                            (const float*)dout, g, gate_stride, (const __nv_bfloat16*)y, rows, cols, tokens, rows_per_block,
                            (__nv_bfloat16*)dy, dgate, sums_bf16, workspace, tickets)));
  }
  return (int)cudaGetLastError();
}
