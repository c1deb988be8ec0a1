// Multi-tensor ("one launch for many parameters") optimizer kernels, driven by descriptor tables in
// device memory that the host builds once per parameter set.
//
// An optimizer step over a transformer touches hundreds of small tensors; launching one kernel per
// tensor per operation (as the reference does: viola/optim/muon.py:111-141 calls momentum_update,
// weight_update and adam_update per parameter, viola/distributed/ema.py:100-113 loops lerps) makes the
// step launch-bound.  Here every operation is one launch: block b looks its tensor up in a prefix
// table of 4096-element chunks and processes one chunk.  Arithmetic is the single-tensor kernels'.
#include "api.h"
#include "common/numerics.cuh"

namespace vb {

constexpr int kChunk = 4096;

// 8 x int64 per tensor; meaning of the slots depends on the operation (see the launchers).
struct Desc {
  long long p0, p1, p2, p3;   // pointers
  long long n;                // elements
  long long i0;               // integer payload (Philox key, ...)
  float f0, f1;               // float payload
  int d0, d1;                 // dtype codes
};
static_assert(sizeof(Desc) == 64, "descriptor is 8 x 8 bytes");

// block -> (tensor, first element of this block's chunk)
__device__ __forceinline__ int find_tensor(const int* __restrict__ chunk_prefix, int tensors, int block) {
  int lo = 0, hi = tensors;             // prefix[lo] <= block < prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (chunk_prefix[mid] <= block) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(256)
multi_ema_kernel(const Desc* __restrict__ table, const int* __restrict__ prefix, int tensors, float decay) {
  const int t = find_tensor(prefix, tensors, blockIdx.x);
  const Desc d = table[t];
  const long long begin = (long long)(blockIdx.x - prefix[t]) * kChunk;
  const long long end = min(begin + kChunk, d.n);
  void* ema = reinterpret_cast<void*>(d.p0);
  const void* master = reinterpret_cast<const void*>(d.p1);
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float e = load_as_float(ema, i, d.d0) * decay;
    store_from_float(ema, i, d.d0, fmaf(1.f - decay, load_as_float(master, i, d.d1), e));
  }
}

// p0 weight, p1 grad, p2 first, p3 second; d0 weight dtype, d1 = grad dtype | state dtype << 8; i0 key
__global__ void __launch_bounds__(256)
multi_adam_kernel(const Desc* __restrict__ table, const int* __restrict__ prefix, int tensors, float lr, float decay,
                  float b1, float b2, float inv_c1, float inv_c2, float eps, int adamw, int maximize, int stochastic,
                  unsigned long long step) {
  const int t = find_tensor(prefix, tensors, blockIdx.x);
  const Desc d = table[t];
  const long long begin = (long long)(blockIdx.x - prefix[t]) * kChunk;
  const long long end = min(begin + kChunk, d.n);
  void* weight = reinterpret_cast<void*>(d.p0);
  const void* grad = reinterpret_cast<const void*>(d.p1);
  void* first = reinterpret_cast<void*>(d.p2);
  void* second = reinterpret_cast<void*>(d.p3);
  const int gdt = d.d1 & 0xff, sdt = (d.d1 >> 8) & 0xff;
  for (long long j = begin + threadIdx.x; j < end; j += blockDim.x) {
    float w = load_as_float(weight, j, d.d0);
    float g = load_as_float(grad, j, gdt);
    if (maximize) g = -g;
    if (!adamw) g = g + decay * w;
    const float m = b1 * load_as_float(first, j, sdt) + (1.f - b1) * g;
    const float v = b2 * load_as_float(second, j, sdt) + (1.f - b2) * g * g;
    store_from_float(first, j, sdt, m);
    store_from_float(second, j, sdt, v);
    if (adamw) w = w * (1.f - lr * decay);
    const float value = w - lr * (m * inv_c1) / (sqrtf(v * inv_c2) + eps);
    store_rounded(weight, j, d.d0, value, stochastic != 0, (unsigned long long)j, step, (unsigned long long)d.i0);
  }
}

// p0 weight, p1 update; d0 weight dtype, d1 update dtype; f0 update scale; i0 key
__global__ void __launch_bounds__(256)
multi_weight_update_kernel(const Desc* __restrict__ table, const int* __restrict__ prefix, int tensors, float lr,
                           float decay, int stochastic, unsigned long long step) {
  const int t = find_tensor(prefix, tensors, blockIdx.x);
  const Desc d = table[t];
  const long long begin = (long long)(blockIdx.x - prefix[t]) * kChunk;
  const long long end = min(begin + kChunk, d.n);
  void* weight = reinterpret_cast<void*>(d.p0);
  const void* update = reinterpret_cast<const void*>(d.p1);
  const float keep = 1.f - lr * decay, rate = lr * d.f0;
  // fp32 master, bf16 update, 16-byte aligned: eight elements per thread and iteration (32-byte and 16-byte accesses);
  // the arithmetic per element is the scalar loop's
  if (d.d0 == kF32 && d.d1 == kBF16 && ((d.p0 | d.p1) & 15) == 0) {
    float* w = reinterpret_cast<float*>(d.p0);
    const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(d.p1);
    long long j = begin + (long long)threadIdx.x * 8;
    for (; j + 8 <= end; j += (long long)blockDim.x * 8) {
      float4 a = *reinterpret_cast<const float4*>(w + j), b = *reinterpret_cast<const float4*>(w + j + 4);
      const uint4 raw = *reinterpret_cast<const uint4*>(u + j);
      const float2 u0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      const float2 u1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      const float2 u2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.z));
      const float2 u3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.w));
      a.x = a.x * keep - rate * u0.x; a.y = a.y * keep - rate * u0.y;
      a.z = a.z * keep - rate * u1.x; a.w = a.w * keep - rate * u1.y;
      b.x = b.x * keep - rate * u2.x; b.y = b.y * keep - rate * u2.y;
      b.z = b.z * keep - rate * u3.x; b.w = b.w * keep - rate * u3.y;
      *reinterpret_cast<float4*>(w + j) = a;
      *reinterpret_cast<float4*>(w + j + 4) = b;
    }
    if (j < end && j + 8 > end)                     // the ragged end of the last chunk, by the same thread
      for (; j < end; ++j) w[j] = w[j] * keep - rate * __bfloat162float(u[j]);
    return;
  }
  for (long long j = begin + threadIdx.x; j < end; j += blockDim.x) {
    const float v = load_as_float(weight, j, d.d0) * keep - rate * load_as_float(update, j, d.d1);
    store_rounded(weight, j, d.d0, v, stochastic != 0, (unsigned long long)j, step, (unsigned long long)d.i0);
  }
}

// FP8 momentum with 1-D tiles: p0 grad, p1 codes (in place), p2 scales (in place), p3 bf16 update out;
// d0 grad dtype; i0 Philox key.  One warp per tile, kChunk / TILE tiles per block.
template <int TILE>
__global__ void __launch_bounds__(256)
multi_momentum_kernel(const Desc* __restrict__ table, const int* __restrict__ prefix, int tensors, float beta,
                      float inv_loss_scale, int nesterov, int stochastic, unsigned long long step) {
  constexpr int EPL = TILE / 32;
  const int t = find_tensor(prefix, tensors, blockIdx.x);
  const Desc d = table[t];
  const long long first_tile = (long long)(blockIdx.x - prefix[t]) * (kChunk / TILE);
  const long long tiles = (d.n + TILE - 1) / TILE;
  const void* grad = reinterpret_cast<const void*>(d.p0);
  uint8_t* codes = reinterpret_cast<uint8_t*>(d.p1);
  float* scales = reinterpret_cast<float*>(d.p2);
  __nv_bfloat16* update = reinterpret_cast<__nv_bfloat16*>(d.p3);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // fp32 gradient, 16-byte aligned buffers, whole tiles: every lane owns EPL consecutive elements and moves them with
  // vector accesses; which lane holds which element does not enter the arithmetic, so the results are the scalar path's
  const bool vector_ok = EPL % 4 == 0 && d.d0 == kF32 && ((d.p0 | d.p1 | d.p3) & 15) == 0;
  for (long long tile = first_tile + warp; tile < min(first_tile + kChunk / TILE, tiles); tile += 8) {
    const long long base = tile * TILE;
    const float old_scale = scales[tile];
    float g[EPL], m[EPL];
    float amax = 0.f;
    if constexpr (EPL % 4 == 0) {
      if (vector_ok && base + TILE <= d.n) {
        const long long i0 = base + (long long)lane * EPL;
        const float* gp = reinterpret_cast<const float*>(grad) + i0;
        uint32_t words[EPL / 4];
#pragma unroll
        for (int v = 0; v < EPL / 4; ++v) {
          const float4 q = *reinterpret_cast<const float4*>(gp + 4 * v);
          g[4 * v] = q.x * inv_loss_scale; g[4 * v + 1] = q.y * inv_loss_scale;
          g[4 * v + 2] = q.z * inv_loss_scale; g[4 * v + 3] = q.w * inv_loss_scale;
        }
        if constexpr (EPL == 4) {
          words[0] = *reinterpret_cast<const uint32_t*>(codes + i0);
        } else if constexpr (EPL == 8) {
          const uint2 q = *reinterpret_cast<const uint2*>(codes + i0);
          words[0] = q.x; words[1] = q.y;
        } else {
#pragma unroll
          for (int v = 0; v < EPL / 16; ++v) {
            const uint4 q = *reinterpret_cast<const uint4*>(codes + i0 + 16 * v);
            words[4 * v] = q.x; words[4 * v + 1] = q.y; words[4 * v + 2] = q.z; words[4 * v + 3] = q.w;
          }
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          const float old = fp8_decode((uint8_t)(words[e >> 2] >> (8 * (e & 3))), kE4M3) * old_scale;
          m[e] = beta * old + (1.f - beta) * g[e];
          amax = fmaxf(amax, fabsf(m[e]));
        }
        amax = warp_max(amax);
        const float scale = fmaxf(amax, 1e-30f) / 448.f;
        if (lane == 0) scales[tile] = scale;
        uint32_t out_words[EPL / 4];
        uint32_t up[EPL / 2];
#pragma unroll
        for (int v = 0; v < EPL / 4; ++v) out_words[v] = 0u;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          float c = fminf(fmaxf(m[e] / scale, -448.f), 448.f);
          if (m[e] != m[e]) c = m[e];
          if (stochastic) c = stochastic_e4m3(c, (unsigned long long)(i0 + e), step, (unsigned long long)d.i0);
          out_words[e >> 2] |= (uint32_t)fp8_encode(c, kE4M3) << (8 * (e & 3));
        }
#pragma unroll
        for (int e = 0; e < EPL; e += 2) {
          const float a = nesterov ? (1.f - beta) * g[e] + beta * m[e] : m[e];
          const float b = nesterov ? (1.f - beta) * g[e + 1] + beta * m[e + 1] : m[e + 1];
          const __nv_bfloat162 pair = __halves2bfloat162(__float2bfloat16_rn(a), __float2bfloat16_rn(b));
          up[e >> 1] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        if constexpr (EPL == 4) {
          *reinterpret_cast<uint32_t*>(codes + i0) = out_words[0];
          *reinterpret_cast<uint2*>(update + i0) = make_uint2(up[0], up[1]);
        } else if constexpr (EPL == 8) {
          *reinterpret_cast<uint2*>(codes + i0) = make_uint2(out_words[0], out_words[1]);
          *reinterpret_cast<uint4*>(update + i0) = make_uint4(up[0], up[1], up[2], up[3]);
        } else {
#pragma unroll
          for (int v = 0; v < EPL / 16; ++v)
            *reinterpret_cast<uint4*>(codes + i0 + 16 * v) =
                make_uint4(out_words[4 * v], out_words[4 * v + 1], out_words[4 * v + 2], out_words[4 * v + 3]);
#pragma unroll
          for (int v = 0; v < EPL / 8; ++v)
            *reinterpret_cast<uint4*>(update + i0 + 8 * v) = make_uint4(up[4 * v], up[4 * v + 1], up[4 * v + 2], up[4 * v + 3]);
        }
        continue;
      }
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const long long i = base + e * 32 + lane;
      const bool in = i < d.n;
      g[e] = in ? load_as_float(grad, i, d.d0) * inv_loss_scale : 0.f;
      const float old = in ? fp8_decode(codes[i], kE4M3) * old_scale : 0.f;
      m[e] = beta * old + (1.f - beta) * g[e];
      amax = fmaxf(amax, fabsf(m[e]));
    }
    amax = warp_max(amax);
    const float scale = fmaxf(amax, 1e-30f) / 448.f;
    if (lane == 0) scales[tile] = scale;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const long long i = base + e * 32 + lane;
      float c = fminf(fmaxf(m[e] / scale, -448.f), 448.f);
      if (m[e] != m[e]) c = m[e];
      if (stochastic) c = stochastic_e4m3(c, (unsigned long long)i, step, (unsigned long long)d.i0);
      codes[i] = fp8_encode(c, kE4M3);                      // the padded tail belongs to the state buffer
      if (i < d.n) update[i] = __float2bfloat16_rn(nesterov ? (1.f - beta) * g[e] + beta * m[e] : m[e]);
    }
  }
}

}  // namespace vb

using namespace vb;

extern "C" int vb_multi_ema(const void* table, const int* prefix, int tensors, int blocks, float decay, cudaStream_t stream) {
  if (blocks <= 0) return 0;
  multi_ema_kernel<<<blocks, 256, 0, stream>>>((const Desc*)table, prefix, tensors, decay);
  return (int)cudaGetLastError();
}

extern "C" int vb_multi_adam(const void* table, const int* prefix, int tensors, int blocks, float lr, float decay, float b1,
                             float b2, float inv_c1, float inv_c2, float eps, int adamw, int maximize, int stochastic,
                             long long step, cudaStream_t stream) {
  if (blocks <= 0) return 0;
  multi_adam_kernel<<<blocks, 256, 0, stream>>>((const Desc*)table, prefix, tensors, lr, decay, b1, b2, inv_c1, inv_c2, eps,
                                                adamw, maximize, stochastic, (unsigned long long)step);
  return (int)cudaGetLastError();
}

extern "C" int vb_multi_weight_update(const void* table, const int* prefix, int tensors, int blocks, float lr, float decay,
                                      int stochastic, long long step, cudaStream_t stream) {
  if (blocks <= 0) return 0;
  multi_weight_update_kernel<<<blocks, 256, 0, stream>>>((const Desc*)table, prefix, tensors, lr, decay, stochastic,
                                                         (unsigned long long)step);
  return (int)cudaGetLastError();
}

extern "C" int vb_multi_momentum(const void* table, const int* prefix, int tensors, int blocks, int tile, float beta,
                                 float inv_loss_scale, int nesterov, int stochastic, long long step, cudaStream_t stream) {
  if (blocks <= 0) return 0;
#define VB_MM(T)                                                                                                  \
  multi_momentum_kernel<T><<<blocks, 256, 0, stream>>>((const Desc*)table, prefix, tensors, beta, inv_loss_scale, \
                                                       nesterov, stochastic, (unsigned long long)step)
  switch (tile) {
    case 64: VB_MM(64); break;
    case 128: VB_MM(128); break;
    case 256: VB_MM(256); break;
    case 512: VB_MM(512); break;
    case 1024: VB_MM(1024); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef VB_MM
  return (int)cudaGetLastError();
}
