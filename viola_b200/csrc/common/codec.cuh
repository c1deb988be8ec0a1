// Warp-level tile codec shared by the standalone wire kernels and the fused
// communication kernels: one warp encodes / decodes one tile of TILE fp32 values.
// Element e of lane l inside a tile is index (e / V) * 32 * V + l * V + e % V with
// V = min(4, TILE / 32), so global accesses are 16-byte (fp32) / 4-byte (codes) vectors.
#pragma once
#include "numerics.cuh"

namespace vb {

template <int TILE>
struct TileShape {
  static constexpr int EPL = TILE / 32;
  static constexpr int V = EPL >= 4 ? 4 : EPL;
  static constexpr int IT = EPL / V;
  static_assert(TILE >= 32 && (TILE & (TILE - 1)) == 0, "tile must be a power of two >= 32");
};

// Load this lane's share of the tile starting at element src0 (zeros beyond n).
template <int TILE>
__device__ __forceinline__ void load_tile(const float* __restrict__ x, long long src0, long long n, int lane,
                                          float (&v)[TILE / 32]) {
  using S = TileShape<TILE>;
  const bool vec = S::V == 4 && src0 + TILE <= n && ((reinterpret_cast<uintptr_t>(x + src0) & 15) == 0);
#pragma unroll
  for (int it = 0; it < S::IT; ++it) {
    const long long i0 = src0 + it * 32 * S::V + lane * S::V;
    if constexpr (S::V == 4) {
      if (vec) {
        float4 t = *reinterpret_cast<const float4*>(x + i0);
        v[it * 4 + 0] = t.x; v[it * 4 + 1] = t.y; v[it * 4 + 2] = t.z; v[it * 4 + 3] = t.w;
        continue;
      }
    }
    {
#pragma unroll
      for (int e = 0; e < S::V; ++e) v[it * S::V + e] = (i0 + e < n) ? x[i0 + e] : 0.f;
    }
  }
}

// amax (NaN -> +inf) -> scale -> codes.  `codes` may point into another GPU's memory.
template <int TILE>
__device__ __forceinline__ float encode_tile(const float (&v)[TILE / 32], int fmt, uint8_t* codes, int lane) {
  using S = TileShape<TILE>;
  float m = 0.f;
#pragma unroll
  for (int e = 0; e < S::EPL; ++e) m = fmaxf(m, abs_nan_to_inf(v[e]));
  m = warp_max(m);
  const float scale = fmaxf(m, 1e-30f) / fp8_max(fmt);
#pragma unroll
  for (int it = 0; it < S::IT; ++it) {
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < S::V; ++e) word |= (uint32_t)fp8_encode(v[it * S::V + e] / scale, fmt) << (8 * e);
    uint8_t* dst = codes + it * 32 * S::V + lane * S::V;
    if constexpr (S::V == 4) *reinterpret_cast<uint32_t*>(dst) = word;
    else if constexpr (S::V == 2) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)word;
    else *dst = (uint8_t)word;
  }
  return scale;
}

template <int TILE>
__device__ __forceinline__ void pack_tile(const float* __restrict__ x, long long src0, long long n, int fmt,
                                          uint8_t* codes, float* scale_out, int lane) {
  float v[TILE / 32];
  load_tile<TILE>(x, src0, n, lane, v);
  const float s = encode_tile<TILE>(v, fmt, codes, lane);
  if (lane == 0) *scale_out = s;
}

// result += decode(codes) * scale
template <int TILE>
__device__ __forceinline__ void accumulate_tile(const uint8_t* codes, float scale, int fmt, int lane,
                                                float (&result)[TILE / 32]) {
  using S = TileShape<TILE>;
#pragma unroll
  for (int it = 0; it < S::IT; ++it) {
    const uint8_t* src = codes + it * 32 * S::V + lane * S::V;
    uint32_t word;
    if constexpr (S::V == 4) word = *reinterpret_cast<const uint32_t*>(src);
    else if constexpr (S::V == 2) word = *reinterpret_cast<const uint16_t*>(src);
    else word = *src;
#pragma unroll
    for (int e = 0; e < S::V; ++e) result[it * S::V + e] += fp8_decode((uint8_t)(word >> (8 * e)), fmt) * scale;
  }
}

template <int TILE>
__device__ __forceinline__ void store_tile(float* __restrict__ out, long long dst0, long long n, int lane,
                                           const float (&result)[TILE / 32], bool accumulate) {
  using S = TileShape<TILE>;
  const bool vec = S::V == 4 && dst0 + TILE <= n && ((reinterpret_cast<uintptr_t>(out + dst0) & 15) == 0);
#pragma unroll
  for (int it = 0; it < S::IT; ++it) {
    const long long i0 = dst0 + it * 32 * S::V + lane * S::V;
    if constexpr (S::V == 4) {
      if (vec) {
        float4 t = make_float4(result[it * 4], result[it * 4 + 1], result[it * 4 + 2], result[it * 4 + 3]);
        if (accumulate) {
          float4 o = *reinterpret_cast<float4*>(out + i0);
          t.x += o.x; t.y += o.y; t.z += o.z; t.w += o.w;
        }
        *reinterpret_cast<float4*>(out + i0) = t;
        continue;
      }
    }
    {
#pragma unroll
      for (int e = 0; e < S::V; ++e)
        if (i0 + e < n) out[i0 + e] = accumulate ? out[i0 + e] + result[it * S::V + e] : result[it * S::V + e];
    }
  }
}

}  // namespace vb
