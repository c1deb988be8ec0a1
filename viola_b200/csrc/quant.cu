// Quantisation kernels (sm_100a): per-tensor amax/scale with delayed-scaling history,
// per-tensor quantise (+transpose), FP8 byte transpose, and group-scaled encode /
// decode (1-D K-groups for activations, 2-D blocks for weights, rowwise and
// transposed from ONE read of the source).
//
// Numerics restate viola/nn/_linear_kernels.py:33-121 and _grouped_kernels.py:24-124:
// scale = max(amax, 1e-30) / limit; codes = clamp(x / scale, +-limit) with NaN kept.
#include "api.h"
#include "common/numerics.cuh"

namespace vb {

// ------------------------------------------------------------------------------
// 16-byte vector load of 8 (16-bit) or 4 (fp32) source elements, as floats
// ------------------------------------------------------------------------------
template <int DT>
struct Src;
template <>
struct Src<kF32> {
  using T = float;
  static constexpr int kVec = 4;
  static __device__ __forceinline__ void load(const T* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ float one(const T* p) { return *p; }
};
template <>
struct Src<kBF16> {
  using T = __nv_bfloat16;
  static constexpr int kVec = 8;
  static __device__ __forceinline__ void load(const T* p, float (&v)[8]) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ float one(const T* p) { return __bfloat162float(*p); }
};
template <>
struct Src<kF16> {
  using T = __half;
  static constexpr int kVec = 8;
  static __device__ __forceinline__ void load(const T* p, float (&v)[8]) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ float one(const T* p) { return __half2float(*p); }
};

// ------------------------------------------------------------------------------
// amax -> scale (+ delayed history).  scratch[0] = running amax bits, scratch[1] =
// ticket counter; the last block to finish computes the scale and re-zeroes both.
// ------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256) amax_scale_kernel(const typename Src<DT>::T* __restrict__ x,
                                                         long long n, float* __restrict__ history,
                                                         int history_len, long long index, int delayed,
                                                         float limit, float* __restrict__ scale_out,
                                                         unsigned int* __restrict__ scratch) {
  constexpr int V = Src<DT>::kVec;
  float m = 0.f;
  const long long nvec = n / V;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  if (aligned) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
      float v[V];
      Src<DT>::load(x + i * V, v);
#pragma unroll
      for (int j = 0; j < V; ++j) m = fmaxf(m, fabsf(v[j]));
    }
    for (long long i = nvec * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
      m = fmaxf(m, fabsf(Src<DT>::one(x + i)));
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
      m = fmaxf(m, fabsf(Src<DT>::one(x + i)));
  }
  m = warp_max(m);
  __shared__ float warp_m[8];
  __shared__ bool last;
  if ((threadIdx.x & 31) == 0) warp_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) b = fmaxf(b, warp_m[i]);
    atomicMax(&scratch[0], __float_as_uint(b));  // non-negative floats order like uints
    __threadfence();
    unsigned int ticket = atomicAdd(&scratch[1], 1u);
    last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    float amax = __uint_as_float(atomicExch(&scratch[0], 0u));
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

// ------------------------------------------------------------------------------
// per-tensor quantise: 64x64 tiles, rowwise and/or transposed output
// ------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256) quantize_kernel(const typename Src<DT>::T* __restrict__ x,
                                                       int rows, int cols,
                                                       const float* __restrict__ scale_ptr, float limit,
                                                       int fmt, uint8_t* __restrict__ q,
                                                       uint8_t* __restrict__ qt) {
  __shared__ __align__(16) uint8_t tile[64][64 + 16];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const float scale = scale_ptr[0];
  const int tr = threadIdx.x >> 2;          // 0..63 row in tile
  const int tc = (threadIdx.x & 3) * 16;    // 16 columns per thread
  const int r = r0 + tr, c = c0 + tc;
  uint8_t codes[16];
  const bool vec_ok = (cols % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (r < rows && c + 15 < cols && vec_ok) {
    constexpr int V = Src<DT>::kVec;
#pragma unroll
    for (int j = 0; j < 16 / V; ++j) {
      float v[V];
      Src<DT>::load(x + (long long)r * cols + c + j * V, v);
#pragma unroll
      for (int e = 0; e < V; ++e) codes[j * V + e] = fp8_encode(scaled_clamp(v[e], scale, limit), fmt);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      float v = (r < rows && c + e < cols) ? Src<DT>::one(x + (long long)r * cols + c + e) : 0.f;
      codes[e] = fp8_encode(scaled_clamp(v, scale, limit), fmt);
    }
  }
  if (q != nullptr && r < rows) {
    if (c + 15 < cols && cols % 16 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
      *reinterpret_cast<uint4*>(q + (long long)r * cols + c) = *reinterpret_cast<uint4*>(codes);
    } else {
      for (int e = 0; e < 16; ++e)
        if (c + e < cols) q[(long long)r * cols + c + e] = codes[e];
    }
  }
  if (qt != nullptr) {
    *reinterpret_cast<uint4*>(&tile[tr][tc]) = *reinterpret_cast<uint4*>(codes);
    __syncthreads();
    // thread -> one source column (output row), 16 source rows (output columns)
    const int oc = threadIdx.x >> 2;        // source column in tile
    const int orow = (threadIdx.x & 3) * 16;  // first source row
    uint8_t out[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) out[e] = tile[orow + e][oc];
    const int gr = c0 + oc;   // row of qt
    const int gc = r0 + orow; // column of qt
    if (gr < cols) {
      if (gc + 15 < rows && rows % 16 == 0 && (reinterpret_cast<uintptr_t>(qt) & 15) == 0) {
        *reinterpret_cast<uint4*>(qt + (long long)gr * rows + gc) = *reinterpret_cast<uint4*>(out);
      } else {
        for (int e = 0; e < 16; ++e)
          if (gc + e < rows) qt[(long long)gr * rows + gc + e] = out[e];
      }
    }
  }
}

// Row-wise codes only, optionally with the fp32 column sums of the source (the bias gradient when the source
// is an output gradient).  A block walks a panel of `panel_rows` rows x 128 columns: thread t owns the 16
// columns (t & 7) * 16 of rows (t >> 3) + 32 i and keeps 16 running sums.  Column sums are reproducible: every
// block stores its panel's sums in `workspace`, and the last block to finish a 128-column strip (ticket in
// the first 1024 words of the workspace, self-resetting) adds the panels in ascending order into
// `colsum`.  Needs cols % 16 == 0 and 16-byte aligned x / q.
template <int DT>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const typename Src<DT>::T* __restrict__ x, int rows,
                                                            int cols, const float* __restrict__ scale_ptr,
                                                            float limit, int fmt, uint8_t* __restrict__ q,
                                                            float* __restrict__ colsum, int panel_rows,
                                                            float* __restrict__ workspace) {
  constexpr int V = Src<DT>::kVec;
  __shared__ float red[32][128 + 8];   // row pitch 136 floats: a warp's 4 rows x 8 groups land in 32 banks
  const Divisor scale = make_divisor(scale_ptr[0]);
  const bool clamp = limit < fp8_max(fmt);
  const int group = threadIdx.x & 7, lane_row = threadIdx.x >> 3;
  const int c = blockIdx.x * 128 + group * 16;
  const int r_begin = blockIdx.y * panel_rows, r_end = min(rows, r_begin + panel_rows);
  float sums[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) sums[e] = 0.f;
  if (c < cols) {
    for (int r = r_begin + lane_row; r < r_end; r += 32) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16 / V; ++j) Src<DT>::load(x + (long long)r * cols + c + j * V, *reinterpret_cast<float(*)[V]>(&v[j * V]));
      uint4 packed;
      uint16_t* codes = reinterpret_cast<uint16_t*>(&packed);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sums[2 * e] += v[2 * e];
        sums[2 * e + 1] += v[2 * e + 1];
        codes[e] = fp8_encode2(scaled_clamp(v[2 * e], scale, limit, clamp), scaled_clamp(v[2 * e + 1], scale, limit, clamp), fmt);
      }
      *reinterpret_cast<uint4*>(q + (long long)r * cols + c) = packed;
    }
  }
  if (colsum == nullptr) return;
#pragma unroll
  for (int e = 0; e < 16; ++e) red[lane_row][e * 8 + group] = sums[e];
  __syncthreads();
  const int strip_cols = gridDim.x * 128;
  unsigned int* tickets = reinterpret_cast<unsigned int*>(workspace);
  float* partial = workspace + 1024;                            // [panels][strip_cols]
  const int col = blockIdx.x * 128 + (threadIdx.x & 7) * 16 + (threadIdx.x >> 3);
  if (threadIdx.x < 128) {
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) total += red[i][threadIdx.x];
    partial[(long long)blockIdx.y * strip_cols + col] = total;
  }
  __shared__ bool last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    last = atomicAdd(&tickets[blockIdx.x], 1u) == gridDim.y - 1;
    if (last) tickets[blockIdx.x] = 0u;
  }
  __syncthreads();
  if (last && threadIdx.x < 128 && col < cols) {
    __threadfence();
    float total = 0.f;
    for (int p = 0; p < (int)gridDim.y; ++p) total += __ldcg(&partial[(long long)p * strip_cols + col]);   // other blocks' stores: read at L2
    colsum[col] += total;
  }
}

__global__ void __launch_bounds__(256) transpose_u8_kernel(const uint8_t* __restrict__ x, int rows,
                                                           int cols, uint8_t* __restrict__ out) {
  __shared__ __align__(16) uint8_t tile[64][64 + 16];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tr = threadIdx.x >> 2, tc = (threadIdx.x & 3) * 16;
  const int r = r0 + tr, c = c0 + tc;
  uint8_t codes[16];
  if (r < rows && c + 15 < cols && cols % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    *reinterpret_cast<uint4*>(codes) = *reinterpret_cast<const uint4*>(x + (long long)r * cols + c);
  } else {
    for (int e = 0; e < 16; ++e) codes[e] = (r < rows && c + e < cols) ? x[(long long)r * cols + c + e] : 0;
  }
  *reinterpret_cast<uint4*>(&tile[tr][tc]) = *reinterpret_cast<uint4*>(codes);
  __syncthreads();
  const int oc = threadIdx.x >> 2, orow = (threadIdx.x & 3) * 16;
  uint8_t o[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) o[e] = tile[orow + e][oc];
  const int gr = c0 + oc, gc = r0 + orow;
  if (gr < cols) {
    if (gc + 15 < rows && rows % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
      *reinterpret_cast<uint4*>(out + (long long)gr * rows + gc) = *reinterpret_cast<uint4*>(o);
    } else {
      for (int e = 0; e < 16; ++e)
        if (gc + e < rows) out[(long long)gr * rows + gc + e] = o[e];
    }
  }
}

// ------------------------------------------------------------------------------
// Group-scaled encode.  One CTA handles a 128 x 128 source tile held in shared
// memory as floats-rounded-to-source precision (we keep the raw 16-bit/32-bit
// values), then emits any of:
//   * rowwise codes  q [rows, cols]  with groups (gr x gc) in source coordinates
//   * transposed codes qt[cols, rows] with groups (tgr x tgc) in TRANSPOSED coordinates
// from that single read.  Group shapes must divide 128 or be multiples of it along
// each axis only through the tile-local part: we require gr, gc in {1,2,...,128}
// powers of two (larger groups fall back to the generic kernel below).
// scale layout: scale[(r / gr) * s_row + (c / gc) * s_col] so callers choose
// row-major [R/gr, C/gc] (s_row = ceil(C/gc), s_col = 1) or K-block-major.
// ------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256)
group_encode_kernel(const typename Src<DT>::T* __restrict__ x, int rows, int cols, int fmt, float limit,
                    uint8_t* __restrict__ q, float* __restrict__ s, int gr, int gc, long long s_row,
                    long long s_col, uint8_t* __restrict__ qt, float* __restrict__ st, int tgr, int tgc,
                    long long st_row, long long st_col, int pow2) {
  constexpr int TS = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float (*tile)[TS + 1] = reinterpret_cast<float (*)[TS + 1]>(smem_raw);  // 128 x 129 floats
  __shared__ float gscale[TS * 4];  // up to 512 group scales per tile per pass
  const int r0 = blockIdx.y * TS, c0 = blockIdx.x * TS;
  // load tile (zero padded)
  for (int i = threadIdx.x; i < TS * TS; i += blockDim.x) {
    int tr = i / TS, tc = i % TS;
    int r = r0 + tr, c = c0 + tc;
    tile[tr][tc] = (r < rows && c < cols) ? Src<DT>::one(x + (long long)r * cols + c) : 0.f;
  }
  __syncthreads();
  // pass 0: rowwise (source coordinates); pass 1: transposed coordinates
  for (int pass = 0; pass < 2; ++pass) {
    uint8_t* out = pass == 0 ? q : qt;
    if (out == nullptr) continue;
    float* sc = pass == 0 ? s : st;
    const int g_r = pass == 0 ? gr : tgr;   // group extent along output rows
    const int g_c = pass == 0 ? gc : tgc;   // group extent along output cols
    const int er = g_r < TS ? g_r : TS, ec = g_c < TS ? g_c : TS;  // tile-local extents
    const int ngr = TS / er, ngc = TS / ec;
    const int ngroups = ngr * ngc;
    // amax per group: one warp per group round-robin
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = warp; g < ngroups; g += (blockDim.x >> 5)) {
      int gy = g / ngc, gx = g % ngc;
      float m = 0.f;
      for (int e = lane; e < er * ec; e += 32) {
        int y = gy * er + e / ec, xx = gx * ec + e % ec;  // output-tile coordinates
        float v = pass == 0 ? tile[y][xx] : tile[xx][y];
        m = fmaxf(m, abs_nan_to_inf(v));
      }
      m = warp_max(m);
      if (lane == 0) gscale[g] = m;
    }
    __syncthreads();
    // Groups wider than the tile need a cross-CTA amax; those shapes use the generic kernel.
    for (int g = threadIdx.x; g < ngroups; g += blockDim.x) {
      float sc_v = fmaxf(gscale[g], 1e-30f) / limit;
      if (pow2) sc_v = ceil_pow2(sc_v);
      gscale[g] = sc_v;
      int gy = g / ngc, gx = g % ngc;
      int orow0 = (pass == 0 ? r0 : c0) + gy * er, ocol0 = (pass == 0 ? c0 : r0) + gx * ec;
      int orows = pass == 0 ? rows : cols, ocols = pass == 0 ? cols : rows;
      if (orow0 < orows && ocol0 < ocols)
        sc[(long long)(orow0 / g_r) * (pass == 0 ? s_row : st_row) +
           (long long)(ocol0 / g_c) * (pass == 0 ? s_col : st_col)] = sc_v;
    }
    __syncthreads();
    // encode: thread -> 16 consecutive output columns of one output row
    const int orows = pass == 0 ? rows : cols, ocols = pass == 0 ? cols : rows;
    const int obase_r = pass == 0 ? r0 : c0, obase_c = pass == 0 ? c0 : r0;
    for (int i = threadIdx.x; i < TS * (TS / 16); i += blockDim.x) {
      int y = i / (TS / 16), x16 = (i % (TS / 16)) * 16;
      uint8_t codes[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        int xx = x16 + e;
        float v = pass == 0 ? tile[y][xx] : tile[xx][y];
        float scv = gscale[(y / er) * ngc + xx / ec];
        codes[e] = fp8_encode(scaled_clamp(v, scv, limit), fmt);
      }
      int orow = obase_r + y, ocol = obase_c + x16;
      if (orow < orows) {
        uint8_t* dst = out + (long long)orow * ocols + ocol;
        if (ocol + 15 < ocols && ocols % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(codes);
        } else {
          for (int e = 0; e < 16; ++e)
            if (ocol + e < ocols) dst[e] = codes[e];
        }
      }
    }
    __syncthreads();
  }
}

// Fast path for the hot activation case: 1 x 128 groups rowwise, bf16/fp16/fp32 in,
// one warp per (row, 128-column group) -> 16 B loads, 4 B code stores per lane.
template <int DT>
__global__ void __launch_bounds__(256)
row128_encode_kernel(const typename Src<DT>::T* __restrict__ x, int rows, int cols, int fmt, float limit,
                     uint8_t* __restrict__ q, float* __restrict__ s, long long s_row, long long s_col, int pow2) {
  const int groups_per_row = cols / 128;
  const long long total = (long long)rows * groups_per_row;
  const int lane = threadIdx.x & 31;
  for (long long g = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); g < total;
       g += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int r = (int)(g / groups_per_row), kb = (int)(g % groups_per_row);
    const typename Src<DT>::T* src = x + (long long)r * cols + kb * 128 + lane * 4;
    float v[4];
    if constexpr (DT == kF32) {
      float4 t = *reinterpret_cast<const float4*>(src);
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
      uint2 t = *reinterpret_cast<const uint2*>(src);
      if constexpr (DT == kBF16) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
        float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
      } else {
        const __half2* h = reinterpret_cast<const __half2*>(&t);
        float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
      }
    }
    float m = fmaxf(fmaxf(abs_nan_to_inf(v[0]), abs_nan_to_inf(v[1])),
                    fmaxf(abs_nan_to_inf(v[2]), abs_nan_to_inf(v[3])));
    m = warp_max(m);
    float sc = fmaxf(m, 1e-30f) / limit;
    if (pow2) sc = ceil_pow2(sc);
    uint32_t packed = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) packed |= (uint32_t)fp8_encode(scaled_clamp(v[e], sc, limit), fmt) << (8 * e);
    *reinterpret_cast<uint32_t*>(q + (long long)r * cols + kb * 128 + lane * 4) = packed;
    if (lane == 0) s[(long long)r * s_row + (long long)kb * s_col] = sc;
  }
}

// Generic (slow, any group shape incl. groups larger than 128) encode: one CTA per group.
template <int DT>
__global__ void __launch_bounds__(128)
group_encode_generic_kernel(const typename Src<DT>::T* __restrict__ x, int rows, int cols, int fmt,
                            float limit, int transposed, uint8_t* __restrict__ q, float* __restrict__ s,
                            int gr, int gc, long long s_row, long long s_col, int pow2) {
  // output coordinates: (orows, ocols) = transposed ? (cols, rows) : (rows, cols)
  const int orows = transposed ? cols : rows, ocols = transposed ? rows : cols;
  const int ngc = (ocols + gc - 1) / gc;
  const int gy = blockIdx.x / ngc, gx = blockIdx.x % ngc;
  __shared__ float red[4];
  float m = 0.f;
  const int count = gr * gc;
  for (int e = threadIdx.x; e < count; e += blockDim.x) {
    int y = gy * gr + e / gc, xx = gx * gc + e % gc;
    if (y < orows && xx < ocols) {
      float v = transposed ? Src<DT>::one(x + (long long)xx * cols + y) : Src<DT>::one(x + (long long)y * cols + xx);
      m = fmaxf(m, abs_nan_to_inf(v));
    }
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  float sc = fmaxf(m, 1e-30f) / limit;
  if (pow2) sc = ceil_pow2(sc);
  if (threadIdx.x == 0) s[(long long)gy * s_row + (long long)gx * s_col] = sc;
  for (int e = threadIdx.x; e < count; e += blockDim.x) {
    int y = gy * gr + e / gc, xx = gx * gc + e % gc;
    if (y < orows && xx < ocols) {
      float v = transposed ? Src<DT>::one(x + (long long)xx * cols + y) : Src<DT>::one(x + (long long)y * cols + xx);
      q[(long long)y * ocols + xx] = fp8_encode(scaled_clamp(v, sc, limit), fmt);
    }
  }
}

__global__ void __launch_bounds__(256)
group_decode_kernel(const uint8_t* __restrict__ q, const float* __restrict__ s, int rows, int cols, int fmt,
                    int gr, int gc, long long s_row, long long s_col, float* __restrict__ out) {
  const long long n = (long long)rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    int r = (int)(i / cols), c = (int)(i % cols);
    out[i] = fp8_decode(q[i], fmt) * s[(long long)(r / gr) * s_row + (long long)(c / gc) * s_col];
  }
}

}  // namespace vb

using namespace vb;

#define VB_DISPATCH_DT(dt, ...)                                   \
  switch (dt) {                                                   \
    case kF32: { constexpr int DT = kF32; __VA_ARGS__; } break;   \
    case kBF16: { constexpr int DT = kBF16; __VA_ARGS__; } break; \
    case kF16: { constexpr int DT = kF16; __VA_ARGS__; } break;   \
    default: return (int)cudaErrorInvalidValue;                   \
  }

extern "C" int vb_amax_scale(const void* x, long long n, int dtype, float* history, int history_len,
                             long long index, int delayed, float limit, float* scale_out,
                             unsigned int* scratch, cudaStream_t stream) {
  if (n <= 0) return (int)cudaErrorInvalidValue;
  int blocks = (int)std::min<long long>((n + 256 * 32 - 1) / (256 * 32), 148 * 8);
  if (blocks < 1) blocks = 1;
  VB_DISPATCH_DT(dtype, (amax_scale_kernel<DT><<<blocks, 256, 0, stream>>>(
                            reinterpret_cast<const Src<DT>::T*>(x), n, history, history_len, index,
                            delayed, limit, scale_out, scratch)));
  return (int)cudaGetLastError();
}

// amax (float bits gathered by a producer's epilogue with atomicMax) -> scale, with the delayed-scaling
// history; re-zeroes the gather word for the next producer.
__global__ void scale_from_amax_kernel(unsigned int* __restrict__ amax_bits, float* __restrict__ history,
                                       int history_len, long long index, int delayed, float limit,
                                       float* __restrict__ scale_out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const float amax = __uint_as_float(amax_bits[0]);
  amax_bits[0] = 0u;
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

extern "C" int vb_scale_from_amax(unsigned int* amax_bits, float* history, int history_len, long long index,
                                  int delayed, float limit, float* scale_out, cudaStream_t stream) {
  scale_from_amax_kernel<<<1, 32, 0, stream>>>(amax_bits, history, history_len, index, delayed, limit, scale_out);
  return (int)cudaGetLastError();
}

extern "C" int vb_quantize(const void* x, int rows, int cols, int dtype, const float* scale, float limit,
                           int fmt, void* q, void* qt, float* colsum, float* workspace, long long workspace_floats,
                           cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const bool vector_ok = cols % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(q) & 15) == 0;
  if (qt == nullptr && q != nullptr && vector_ok) {
    // panels tall enough to amortise the column reduction, short enough to fill the machine
    const int col_blocks = (cols + 127) / 128;
    int panel_rows = 512;
    while (panel_rows > 32 && (long long)col_blocks * ((rows + panel_rows - 1) / panel_rows) < 148LL * 8) panel_rows >>= 1;
    if (colsum != nullptr) {
      panel_rows = 256;   // fixed, so the caller can size the workspace: 1024 + panels * strips * 128 floats
      const long long need = 1024 + (long long)((rows + 255) / 256) * col_blocks * 128;
      if (workspace == nullptr || workspace_floats < need || col_blocks > 1024) return (int)cudaErrorInvalidValue;
    }
    dim3 grid(col_blocks, (rows + panel_rows - 1) / panel_rows);
    VB_DISPATCH_DT(dtype, (quantize_rows_kernel<DT><<<grid, 256, 0, stream>>>(
                              reinterpret_cast<const Src<DT>::T*>(x), rows, cols, scale, limit, fmt,
                              reinterpret_cast<uint8_t*>(q), colsum, panel_rows, workspace)));
    return (int)cudaGetLastError();
  }
  if (colsum != nullptr) return (int)cudaErrorInvalidValue;   // column sums ride on the row-wise path only
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  VB_DISPATCH_DT(dtype, (quantize_kernel<DT><<<grid, 256, 0, stream>>>(
                            reinterpret_cast<const Src<DT>::T*>(x), rows, cols, scale, limit, fmt,
                            reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(qt))));
  return (int)cudaGetLastError();
}

extern "C" int vb_transpose_u8(const void* x, int rows, int cols, void* out, cudaStream_t stream) {
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  transpose_u8_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(x), rows, cols,
                                                reinterpret_cast<uint8_t*>(out));
  return (int)cudaGetLastError();
}

extern "C" int vb_group_encode(const void* x, int rows, int cols, int dtype, int fmt, float limit, void* q,
                               float* s, int gr, int gc, long long s_row, long long s_col, void* qt,
                               float* st, int tgr, int tgc, long long st_row, long long st_col, int pow2,
                               cudaStream_t stream) {
  auto is_pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
  if (!is_pow2(gr) || !is_pow2(gc) || (qt != nullptr && (!is_pow2(tgr) || !is_pow2(tgc))))
    return (int)cudaErrorInvalidValue;
  const bool tile_ok = gr <= 128 && gc <= 128 && (qt == nullptr || (tgr <= 128 && tgc <= 128));
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0;
  if (qt == nullptr && q != nullptr && gr == 1 && gc == 128 && cols % 128 == 0 && aligned) {
    long long groups = (long long)rows * (cols / 128);
    int blocks = (int)std::min<long long>((groups + 7) / 8, 148 * 16);
    VB_DISPATCH_DT(dtype, (row128_encode_kernel<DT><<<blocks, 256, 0, stream>>>(
                              reinterpret_cast<const Src<DT>::T*>(x), rows, cols, fmt, limit,
                              reinterpret_cast<uint8_t*>(q), s, s_row, s_col, pow2)));
    return (int)cudaGetLastError();
  }
  if (tile_ok) {
    dim3 grid((cols + 127) / 128, (rows + 127) / 128);
    size_t smem = 128 * 129 * sizeof(float);
    VB_DISPATCH_DT(dtype, {
      auto kernel = group_encode_kernel<DT>;
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      kernel<<<grid, 256, smem, stream>>>(reinterpret_cast<const Src<DT>::T*>(x), rows, cols, fmt, limit,
                                          reinterpret_cast<uint8_t*>(q), s, gr, gc, s_row, s_col,
                                          reinterpret_cast<uint8_t*>(qt), st, tgr, tgc, st_row, st_col, pow2);
    });
    return (int)cudaGetLastError();
  }
  if (q != nullptr) {
    int groups = ((rows + gr - 1) / gr) * ((cols + gc - 1) / gc);
    VB_DISPATCH_DT(dtype, (group_encode_generic_kernel<DT><<<groups, 128, 0, stream>>>(
                              reinterpret_cast<const Src<DT>::T*>(x), rows, cols, fmt, limit, 0,
                              reinterpret_cast<uint8_t*>(q), s, gr, gc, s_row, s_col, pow2)));
  }
  if (qt != nullptr) {
    int groups = ((cols + tgr - 1) / tgr) * ((rows + tgc - 1) / tgc);
    VB_DISPATCH_DT(dtype, (group_encode_generic_kernel<DT><<<groups, 128, 0, stream>>>(
                              reinterpret_cast<const Src<DT>::T*>(x), rows, cols, fmt, limit, 1,
                              reinterpret_cast<uint8_t*>(qt), st, tgr, tgc, st_row, st_col, pow2)));
  }
  return (int)cudaGetLastError();
}

extern "C" int vb_group_decode(const void* q, const float* s, int rows, int cols, int fmt, int gr, int gc,
                               long long s_row, long long s_col, float* out, cudaStream_t stream) {
  long long n = (long long)rows * cols;
  int blocks = (int)std::min<long long>((n + 255) / 256, 148 * 16);
  if (blocks < 1) blocks = 1;
  group_decode_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(q), s, rows, cols, fmt,
                                                  gr, gc, s_row, s_col, out);
  return (int)cudaGetLastError();
}
