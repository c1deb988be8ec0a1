// Scalar numerics shared by every elementwise kernel: FP8 encode/decode, the
// counter-based Philox4x32-10 generator and the three stochastic-rounding grids.
//
// The formulas restate the reference's device helpers (viola/optim/_kernels.py:12-58:
// Philox counter = (element lo/hi, step lo/hi), 64-bit key; E4M3 grid spacing
// 2^max(e-3,-9); BF16 "add 16 random bits, truncate"; FP16 spacing 2^max(e-10,-24)).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace vb {

enum Fp8Format : int { kE4M3 = 0, kE5M2 = 1 };

__host__ __device__ __forceinline__ float fp8_max(int fmt) { return fmt == kE4M3 ? 448.0f : 57344.0f; }

// Saturating round-to-nearest-even encode; NaN stays NaN (callers clamp finite
// values themselves so the saturation mode only matters for +-inf).
__device__ __forceinline__ uint8_t fp8_encode(float v, int fmt) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, fmt == kE4M3 ? __NV_E4M3 : __NV_E5M2);
}
__device__ __forceinline__ float fp8_decode(uint8_t c, int fmt) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, fmt == kE4M3 ? __NV_E4M3 : __NV_E5M2);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// Two values -> two codes in one cvt (low 8 bits = first value).
__device__ __forceinline__ uint16_t fp8_encode2(float a, float b, int fmt) {
  return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE,
                                            fmt == kE4M3 ? __NV_E4M3 : __NV_E5M2);
}

// Smallest power of two >= s for a positive finite s (exactly: exponent bumped when the mantissa is non-zero);
// the MXFP8 recipe stores scales as UE8M0 exponents.  Inf / NaN pass through.
__device__ __forceinline__ float ceil_pow2(float s) {
  const uint32_t bits = __float_as_uint(s);
  const uint32_t exponent = (bits >> 23) & 0xffu;
  if (exponent == 0xffu) return s;
  return __uint_as_float((exponent + ((bits & 0x7fffffu) != 0u ? 1u : 0u)) << 23);
}

// clamp(v / scale, +-limit) with NaN preserved (fminf/fmaxf would drop it).
__device__ __forceinline__ float scaled_clamp(float v, float inv_or_scale_div, float limit) {
  float q = v / inv_or_scale_div;
  return (q != q) ? q : fminf(fmaxf(q, -limit), limit);
}

// v / scale for many v and one scale: a reciprocal computed once, then per element one multiply and one
// Newton correction whose residual is exact under FMA; the quotient is the correctly rounded one (what the
// division instruction sequence computes), at three instructions instead of a dozen.  +-inf and NaN pass through.
struct Divisor {
  float scale, inv;
};
__device__ __forceinline__ Divisor make_divisor(float scale) { return Divisor{scale, __frcp_rn(scale)}; }
__device__ __forceinline__ float divide(float v, const Divisor& d) {
  const float q = v * d.inv;
  const float r = fmaf(-q, d.scale, v);
  return fabsf(q) <= 3.0e38f ? fmaf(r, d.inv, q) : q;
}
// clamp(v / scale, +-limit) with NaN preserved; `clamp` is false when the limit is the format's largest finite
// value, which the saturating conversion enforces by itself.
__device__ __forceinline__ float scaled_clamp(float v, const Divisor& d, float limit, bool clamp) {
  const float q = divide(v, d);
  return (!clamp || q != q) ? q : fminf(fmaxf(q, -limit), limit);
}

__host__ __device__ __forceinline__ uint32_t mulhi32(uint32_t a, uint32_t b) {
#ifdef __CUDA_ARCH__
  return __umulhi(a, b);
#else
  return (uint32_t)(((uint64_t)a * (uint64_t)b) >> 32);
#endif
}

// Philox4x32-10, first output word.
__host__ __device__ __forceinline__ uint32_t philox(uint64_t element, uint64_t step, uint64_t key) {
  uint32_t a = (uint32_t)element, b = (uint32_t)(element >> 32);
  uint32_t c = (uint32_t)step, d = (uint32_t)(step >> 32);
  uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    uint32_t lo0 = 0xD2511F53u * a, hi0 = mulhi32(0xD2511F53u, a);
    uint32_t lo1 = 0xCD9E8D57u * c, hi1 = mulhi32(0xCD9E8D57u, c);
    a = hi1 ^ b ^ k0;
    b = lo1;
    c = hi0 ^ d ^ k1;
    d = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return a;
}

__device__ __forceinline__ float bits_to_float(uint32_t u) { return __uint_as_float(u); }

// Stochastic rounding of an already scaled/clamped value onto the E4M3 grid.  The
// result is exactly representable, so the following RN encode is the identity.
__device__ __forceinline__ float stochastic_e4m3(float x, uint64_t element, uint64_t step,
                                                 uint64_t key) {
  if (!isfinite(x)) return x;
  float a = fabsf(x);
  int exponent = int((__float_as_uint(a) >> 23) & 255) - 127;
  float spacing = bits_to_float((uint32_t)(max(exponent - 3, -9) + 127) << 23);
  float lower = floorf(a / spacing) * spacing;
  float probability = (a - lower) / spacing;
  float uniform = float(philox(element, step, key) >> 8) * 0x1p-24f;
  return copysignf(lower + (uniform < probability ? spacing : 0.0f), x);
}
__device__ __forceinline__ float stochastic_bf16(float x, uint64_t element, uint64_t step,
                                                 uint64_t key) {
  if (!isfinite(x)) return x;
  uint32_t bits = __float_as_uint(x);
  bits = (bits + (philox(element, step, key) >> 16)) & 0xffff0000u;
  return bits_to_float(bits);
}
__device__ __forceinline__ float stochastic_fp16(float x, uint64_t element, uint64_t step,
                                                 uint64_t key) {
  if (!isfinite(x) || fabsf(x) > 65504.0f) return x;
  float a = fabsf(x);
  int exponent = int((__float_as_uint(a) >> 23) & 255) - 127;
  float spacing = bits_to_float((uint32_t)(max(exponent - 10, -24) + 127) << 23);
  float lower = floorf(a / spacing) * spacing;
  float uniform = float(philox(element, step, key) >> 8) * 0x1p-24f;
  return copysignf(lower + (uniform < (a - lower) / spacing ? spacing : 0.0f), x);
}

// dtype codes shared with the bindings
enum DType : int { kF32 = 0, kBF16 = 1, kF16 = 2 };

__device__ __forceinline__ float load_as_float(const void* p, long long i, int dt) {
  if (dt == kF32) return reinterpret_cast<const float*>(p)[i];
  if (dt == kBF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void store_from_float(void* p, long long i, int dt, float v) {
  if (dt == kF32) reinterpret_cast<float*>(p)[i] = v;
  else if (dt == kBF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}
// Store with optional stochastic rounding onto the bf16 / fp16 grid.
__device__ __forceinline__ void store_rounded(void* p, long long i, int dt, float v, bool stochastic,
                                              uint64_t element, uint64_t step, uint64_t key) {
  if (stochastic && dt == kBF16) v = stochastic_bf16(v, element, step, key);
  else if (stochastic && dt == kF16) v = stochastic_fp16(v, element, step, key);
  store_from_float(p, i, dt, v);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// abs that maps NaN to +inf so that an amax reduction propagates non-finites.
__device__ __forceinline__ float abs_nan_to_inf(float v) { return (v != v) ? INFINITY : fabsf(v); }

}  // namespace vb
