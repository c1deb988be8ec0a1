// tcgen05 / TMEM / TMA GEMM family for sm_100a.
//
//   D[M, N] = A[M, K] . B[N, K]^T
//
// Either operand may be K-major (as written) or MN-major (the tensor holds the transpose, [K, M] / [K, N]); the
// producer then loads 128-byte-of-MN x K-row boxes and the UMMA descriptors use the MN-major SWIZZLE_128B form.
//
// One persistent, warp-specialised kernel template covers every GEMM-shaped op in
// the library:
//   * FP8 Linear forward / dgrad / wgrad with per-tensor scales (any e4m3 / e5m2 mix
//     through the instruction descriptor)             [replaces the reference's
//     T.gemm / mma.sync kernels, viola/nn/_linear_kernels.py:124-228]
//   * group-scaled FP8 GEMM, one fp32 scale per 128 K-elements on each operand
//     (two-level accumulation: UMMA over one K-block into a TMEM stage, promotion
//     with sa*sb into fp32 registers while the next K-block's MMA runs)
//                                                     [viola/nn/_grouped_kernels.py:195-293]
//   * fused gated-MLP forward (gate and up share the A tile, act(g)*u epilogue, aux
//     save) and backward (dgrad + gated derivative)   [viola/nn/_mlp_kernels.py:16-231]
//   * expert (ragged-M) GEMM through a tile -> expert map
//   * Newton-Schulz GEMMs in bf16 / fp16 with the two polynomial epilogues, an
//     optional transposed second output and a symmetric-output mode
//                                                     [viola/optim/_orthogonalize_kernels.py:16-50]
//   * dgrad through an activation: D = round(A . B^T) * slope with the amax of D gathered on the fly
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane)
// and TMEM owner, warps 2-5 = epilogue (TMEM lane quadrant = warp % 4); the AXPBY and ACT_BWD
// epilogues add warp 6, which TMA-loads their second operand into a ring of 128x32 slabs that the
// epilogue warps rewrite in place and TMA-store (LINEAR stages and TMA-stores its tile per warp).
// Pipeline: smem ring (full/empty mbarriers, TMA complete_tx / tcgen05.commit) and a
// TMEM accumulator ring (tmem_full via tcgen05.commit, tmem_empty via epilogue arrive).
// TMA loads are never cluster-multicast.  Every wait is bounded (common/ptx.cuh).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <atomic>
#include <mutex>
#include <type_traits>
#include "api.h"
#include "common/ptx.cuh"

namespace vb {

constexpr int BM = 128;
constexpr int BK_BYTES = 128;  // one 128-byte swizzle span along K per stage
// Roles: warp 0 TMA producer, warp 1 MMA issuer, then Config::kEpiWarps epilogue warps (four, or eight for the LINEAR,
// AXPBY and ACT_BWD kernels), then, where an epilogue reads an operand through the slab ring, one loader warp.

struct GemmArgs {
  int M, N, K;
  int num_m_tiles, num_n_tiles, num_k_blocks, num_tiles;
  uint32_t idesc;
  int b_gate_up_offset;  // gated forward: row offset of the "up" half inside B (= N)
  const float* sa;
  const float* sb;
  long long sa_row, sa_k, sb_row, sb_k;
  int sb_shift, k_shift;
  void* out;
  int out_dtype;
  long long ldo;
  const void* bias;
  int bias_dtype;
  float alpha, beta;
  const void* resid;
  long long ldr;
  void* out_t;
  long long ldot;
  int symmetric;
  int activation;
  void* aux;
  long long ldaux;
  const int* tile_map;  // expert mode: [3 * num_m_tiles] = (row0, row_end, expert), row0 < 0 = unused
  int expert_rows;      // rows of B per expert (= N)
  // batched mode: `batch` independent problems stacked along the rows of A, B and the outputs
  int batch, tiles_per_batch;
  long long b_rows_per_batch, out_bs, resid_bs, out_t_bs;
  unsigned int* amax_out;
  int tma_store;        // LINEAR epilogue: stage in shared memory and write with TMA
  int epi_sets;         // slab epilogues: 2 = two sets of four warps alternate over the chunks (needs N % 64 == 0), else 1
  int epi_stage;        // AXPBY residual / ACT_BWD slope arrives through the TMA slab ring
  int epi_store;        // AXPBY / ACT_BWD result leaves through the slab ring (TMA store)
  int a_mn, b_mn;       // operand stored MN-major: A as [K, M] / B as [K, N] (row-major, MN contiguous)
  // split-K (LINEAR epilogue, fp32 output through TMA): every output tile is computed by `split_k` work units, each
  // over `kb_per_split` K-blocks; unit 0 stores its partial tile, unit s adds its own with a TMA reduce once unit
  // s - 1 has finished (split_flags[tile * 8 + epilogue warp] counts finished units; the last one clears it)
  int split_k, kb_per_split;
  int* split_flags;
  int accumulate;       // LINEAR through TMA, fp32: every unit ADDS its tile to the output (out += A.B^T)
  int* status;
};

__device__ __forceinline__ void* advance(void* p, long long elems, int dt) {
  return p == nullptr ? nullptr : (void*)(reinterpret_cast<char*>(p) + elems * (dt == 0 ? 4 : 2));
}
__device__ __forceinline__ const void* advance(const void* p, long long elems, int dt) {
  return p == nullptr ? nullptr : (const void*)(reinterpret_cast<const char*>(p) + elems * (dt == 0 ? 4 : 2));
}

// ---------------------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float round_to(float v, int dt) {
  if (dt == 1) return __bfloat162float(__float2bfloat16_rn(v));
  if (dt == 2) return __half2float(__float2half_rn(v));
  return v;
}
__device__ __forceinline__ float load_elem(const void* p, long long i, int dt) {
  if (dt == 0) return reinterpret_cast<const float*>(p)[i];
  if (dt == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void store_elem(void* p, long long i, int dt, float v) {
  if (dt == 0) reinterpret_cast<float*>(p)[i] = v;
  else if (dt == 1) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, int dt) {
  if (dt == 1) {
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
  }
  __half2 t = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

// Store 32 consecutive values of one row; vectorised when the whole chunk is in range and
// the destination is 16-byte aligned, scalar with bounds checks otherwise.
__device__ __forceinline__ void store_row32(void* base, long long ld, int dt, long long row, int col0,
                                            int ncols, const float (&v)[32]) {
  const long long off = row * ld + col0;
  if (dt == 0) {
    float* p = reinterpret_cast<float*>(base) + off;
    if (col0 + 32 <= ncols && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        reinterpret_cast<float4*>(p)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < ncols) p[j] = v[j];
    }
  } else {
    uint16_t* p = reinterpret_cast<uint16_t*>(base) + off;
    if (col0 + 32 <= ncols && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 t;
        t.x = pack2(v[8 * j + 0], v[8 * j + 1], dt);
        t.y = pack2(v[8 * j + 2], v[8 * j + 3], dt);
        t.z = pack2(v[8 * j + 4], v[8 * j + 5], dt);
        t.w = pack2(v[8 * j + 6], v[8 * j + 7], dt);
        reinterpret_cast<uint4*>(p)[j] = t;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < ncols) store_elem(base, off + j, dt, v[j]);
    }
  }
}
// Load 32 consecutive values of one row as floats (zeros out of range).
__device__ __forceinline__ void load_row32(const void* base, long long ld, int dt, long long row, int col0,
                                           int ncols, float (&v)[32]) {
  const long long off = row * ld + col0;
  if (dt != 0) {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + off;
    if (col0 + 32 <= ncols && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 t = reinterpret_cast<const uint4*>(p)[j];
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f;
          if (dt == 1) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
          else f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
          v[8 * j + 2 * e] = f.x;
          v[8 * j + 2 * e + 1] = f.y;
        }
      }
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = (col0 + j < ncols) ? load_elem(base, off + j, dt) : 0.f;
}

// One row (32 16-bit columns = 64 bytes) of an epilogue slab: rows are 64 bytes apart and the 16-byte pieces of
// a row sit at piece ^ ((row >> 1) & 3) (SWIZZLE_64B), which also spreads a warp's accesses over all banks.
__device__ __forceinline__ uint4* slab_piece(uint8_t* slab, int row_in_tile, int piece) {
  return reinterpret_cast<uint4*>(slab + row_in_tile * 64 + ((piece ^ ((row_in_tile >> 1) & 3)) << 4));
}
__device__ __forceinline__ void load_slab32(uint8_t* slab, int row_in_tile, int dt, float (&v)[32]) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint4 t = *slab_piece(slab, row_in_tile, p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f;
      if (dt == 1) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
      else f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
      v[8 * p + 2 * e] = f.x;
      v[8 * p + 2 * e + 1] = f.y;
    }
  }
}
__device__ __forceinline__ void store_slab32(uint8_t* slab, int row_in_tile, int dt, const float (&v)[32]) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint4 t;
    t.x = pack2(v[8 * p + 0], v[8 * p + 1], dt);
    t.y = pack2(v[8 * p + 2], v[8 * p + 3], dt);
    t.z = pack2(v[8 * p + 4], v[8 * p + 5], dt);
    t.w = pack2(v[8 * p + 6], v[8 * p + 7], dt);
    *slab_piece(slab, row_in_tile, p) = t;
  }
}

// Lean in-place epilogue for one slab row (32 columns), specialised on the 16-bit type so no per-element dtype
// branch survives: v = scaled accumulator; the slab holds the operand x (or nothing) and receives
//   AXPBY  : round(alpha * round(v) + beta * x)
//   ACT_BWD: round(round(v) * x), with max |result| tracked as float bits (NaN orders above +inf)
template <int DT>
__device__ __forceinline__ uint32_t pack_round2(float a, float b) {
  if constexpr (DT == 1) {
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}
template <int DT>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (DT == 1) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <int EPI, int DT>
__device__ __forceinline__ void slab_row_epilogue(const float (&v)[32], uint8_t* slab, int row_in_tile, bool has_operand,
                                                  float alpha, float beta, uint32_t& amax_bits) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint4* ptr = slab_piece(slab, row_in_tile, p);
    const uint4 in = has_operand ? *ptr : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t w[4] = {in.x, in.y, in.z, in.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 d = unpack2<DT>(pack_round2<DT>(v[8 * p + 2 * e], v[8 * p + 2 * e + 1]));
      const float2 x = unpack2<DT>(w[e]);
      if constexpr (EPI == VB_EPI_AXPBY) {
        o[e] = pack_round2<DT>(alpha * d.x + beta * x.x, alpha * d.y + beta * x.y);
      } else {
        o[e] = pack_round2<DT>(d.x * x.x, d.y * x.y);
        const float2 f = unpack2<DT>(o[e]);
        amax_bits = max(amax_bits, max(__float_as_uint(f.x) & 0x7fffffffu, __float_as_uint(f.y) & 0x7fffffffu));
      }
    }
    *ptr = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

__device__ __forceinline__ float act_fn(float g, int act) {
  if (act == VB_ACT_SILU) return g / (1.f + __expf(-g));
  if (act == VB_ACT_RELU) return fmaxf(g, 0.f);
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * g * (1.f + t);
}
__device__ __forceinline__ float act_grad(float g, int act) {
  if (act == VB_ACT_SILU) {
    float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  if (act == VB_ACT_RELU) return g > 0.f ? 1.f : 0.f;
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
}

// Gate activation and its slope for the staged gated epilogues, specialised on the activation.  SiLU and the
// tanh form of GELU are both g * sigmoid(z) (z = g, or z = 2 k0 (g + k1 g^3), since 0.5 (1 + tanh(z / 2)) =
// sigmoid(z)), so one exp2 and one reciprocal approximation serve the value and the slope.
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int ACT>
__device__ __forceinline__ void gate_terms(float g, float& act, float& slope) {
  if constexpr (ACT == VB_ACT_RELU) {
    act = fmaxf(g, 0.f);
    slope = g > 0.f ? 1.f : 0.f;
  } else {
    float z = g, dz = 1.f;
    if constexpr (ACT != VB_ACT_SILU) {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      z = 2.f * k0 * (g + k1 * g * g * g);
      dz = 2.f * k0 * (1.f + 3.f * k1 * g * g);
    }
    const float s = rcp_approx(1.f + __expf(-z));
    act = g * s;
    slope = s * (1.f + g * (1.f - s) * dz);
  }
}

// tile id -> (m_tile, n_tile).  Plain: groups of 8 M-tiles sweep N (L2 reuse of B across the
// wave, of A inside a group).  Symmetric: row-major walk over the upper triangle.
__device__ __forceinline__ void tile_coords(const GemmArgs& a, int t, int& mt, int& nt) {
  if (a.symmetric) {
    int m = 0, T = a.num_m_tiles;
    while (t >= T - m) { t -= T - m; ++m; }
    mt = m; nt = m + t;
    return;
  }
  const int group = 8 * a.num_n_tiles;
  const int g = t / group, first_m = g * 8;
  const int gm = min(8, a.num_m_tiles - first_m);
  const int in = t % group;
  mt = first_m + in % gm;
  nt = in / gm;
}

// PAIR: two CTAs of a cluster work on one 256 x BN output tile with tcgen05 cta_group::2.  Each CTA loads its own 128
// rows of A and HALF of the B tile (BN / 2 rows), the leader (cluster rank 0) issues 256-row MMAs that read both
// CTAs' shared memory and write both CTAs' tensor memory, and each CTA's epilogue drains its own 128 rows.  A stage
// is 32 KB instead of 48 KB per CTA, so six stages fit where four did, and a third less operand traffic reaches
// every SM: what a short-K tile needs to keep the tensor pipe fed across the L2 round trip.
template <int KIND, int BN, bool GROUP, int EPI, bool PAIR = false>
struct Config {
  static_assert(!PAIR || (BN == 256 && !GROUP && EPI == VB_EPI_LINEAR), "CTA pairs: per-tensor LINEAR, 256 columns");
  static constexpr bool kGatedFwd = EPI == VB_EPI_GATED_FWD;
  static constexpr int kBBoxRows = (kGatedFwd || PAIR) ? BN / 2 : BN;
  static constexpr int kABytes = BM * BK_BYTES;
  static constexpr int kBBytes = (PAIR ? BN / 2 : BN) * BK_BYTES;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr bool kTmaStore = EPI == VB_EPI_LINEAR;   // epilogue staged in smem and written by TMA
  // With K of about a thousand a 128 x 256 tile's MMAs take about as long as four warps need to drain it (one
  // warp per scheduler, so every TMEM load and shared-memory store latency is exposed): the per-tensor LINEAR
  // kernels use eight epilogue warps, two per TMEM lane quadrant, each draining half of the tile's columns.
  // Group-scaled LINEAR: the promotion of every K-block (one FMA per accumulator element) is the epilogue warps'
  // whole job, so halving the columns per warp halves the time a K-block's accumulator stays occupied.
  static constexpr int kEpiWarps =
      (EPI == VB_EPI_LINEAR || !GROUP) ? 8 : 4;     // every per-tensor kernel; of the group-scaled ones, LINEAR
  // LINEAR splits a tile's columns into contiguous parts, one per group of four warps; the slab epilogues
  // (AXPBY, ACT_BWD) interleave instead: warps 2-5 take the even chunks, warps 6-9 the odd ones, in the order the
  // loader warp fills the slab ring.
  static constexpr int kColumnParts = EPI == VB_EPI_LINEAR ? kEpiWarps / 4 : 1;
  static constexpr int kStoreBytes = kTmaStore ? kEpiWarps * 4096 : 0;   // per warp: 2 x (32 rows x 64 B) or 32 rows x 128 B
  // AXPBY and ACT_BWD epilogues (16-bit output, optional 16-bit [M, N] operand: the residual / the activation
  // slope) run through a ring of 128-row x 32-column slabs in shared memory, one per output chunk: the
  // producer warp TMA-loads the operand slab while the tile's MMAs run, each epilogue warp rewrites its 32
  // rows of the slab in place with the result and TMA-stores them.  Plain loads issued after the accumulator
  // wait would expose a memory round trip per chunk, and per-thread row stores write half sectors.
  static constexpr bool kEpiSlab = (EPI == VB_EPI_AXPBY || EPI == VB_EPI_ACT_BWD) && !GROUP;
  // The per-tensor gated epilogues use the same slabs.  Forward: every output chunk leaves as three slabs (the
  // activation product h and, when the caller keeps them, the rounded gate and up halves), written by TMA from a
  // four-slab ring.  Backward: the loader warp brings the saved gate and up slabs of a chunk in, the epilogue
  // rewrites them in place with dGate and dUp and TMA-stores both; eight slabs keep four chunks in flight, paid
  // for with one main-loop stage.
  static constexpr bool kGatedBwd = EPI == VB_EPI_GATED_BWD;
  static constexpr bool kGatedSlab = (kGatedFwd || kGatedBwd) && !GROUP;
  static constexpr bool kSlabRing = kEpiSlab || kGatedSlab;
  static constexpr bool kSlabLoader = kEpiSlab || (kGatedBwd && !GROUP);
  static constexpr int kEpiSlabs = ((kGatedBwd || EPI == VB_EPI_ACT_BWD) && !GROUP) ? 8 : 4;
  static constexpr int kLoaderWarp = 2 + kEpiWarps;                                    // feeds the slab ring
  static constexpr int kCtaThreads = 64 + 32 * kEpiWarps + (kSlabLoader ? 32 : 0);
  static constexpr int kEpiSlabBytes = BM * 64;
  static constexpr int kEpiBytes = kSlabRing ? kEpiSlabs * kEpiSlabBytes : 0;
  static constexpr int kStages =
      PAIR ? 6 : (BN == 256) ? ((EPI == VB_EPI_ACT_BWD && !GROUP) ? 3 : 4)
                             : (BN == 128 ? ((((kGatedBwd || EPI == VB_EPI_ACT_BWD) && !GROUP) || (GROUP && kTmaStore)) ? 5 : 6) : 8);
  static constexpr int kAcc = GROUP ? (512 / BN > 4 ? 4 : 512 / BN) : 2;
  static constexpr int kTmemCols = kAcc * BN;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kSbStage = GROUP ? 4 * 2 * BN * (int)sizeof(float) : 0;  // per-warp staged B scales (two buffers)
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + kSbStage + kStoreBytes + kEpiBytes + 1024;
  static_assert(kSmemBytes <= 232448, "dynamic shared memory limit of sm_100");
  static constexpr int kElemBytes = KIND == VB_KIND_F8 ? 1 : 2;
  static constexpr int kBK = BK_BYTES / kElemBytes;  // elements per K-block
  static constexpr int kUmmaKBytes = 32;
  static constexpr int kMmasPerStage = BK_BYTES / kUmmaKBytes;
  static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "TMEM columns");
  static_assert(kSmemBytes > 116 * 1024, "one CTA per SM so TMEM allocation never contends");
};

template <int KIND, int BN, bool GROUP, int EPI, bool PAIR = false>
__global__ void __launch_bounds__((Config<KIND, BN, GROUP, EPI, PAIR>::kCtaThreads), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD, const GemmArgs args) {
  using C = Config<KIND, BN, GROUP, EPI, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full_bar = bars;                         // [kStages]
  uint64_t* empty_bar = bars + C::kStages;           // [kStages]
  uint64_t* tmem_full = bars + 2 * C::kStages;       // [kAcc]
  uint64_t* tmem_empty = tmem_full + C::kAcc;        // [kAcc]
  uint64_t* epi_full = tmem_empty + C::kAcc;         // [kEpiSlabs]
  uint64_t* epi_empty = epi_full + C::kEpiSlabs;     // [kEpiSlabs]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_empty + C::kEpiSlabs);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* sb_stage = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes + C::kBarrierBytes);
  // epilogue staging for TMA stores: the stage ring is a multiple of 1024 bytes and the barrier and
  // scale areas are 1024 / 4096 bytes, so this region keeps the 1024-byte alignment the swizzle needs
  uint8_t* store_stage = smem + C::kStages * C::kStageBytes + C::kBarrierBytes + C::kSbStage;
  uint8_t* epi_stage = store_stage + C::kStoreBytes;   // epilogue slab ring (1024-byte aligned)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // CTA pairs: the persistent loop runs over clusters; `rank` selects this CTA's half of the pair tile
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int cta_first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int cta_stride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < C::kAcc; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], PAIR ? 2 * C::kEpiWarps : C::kEpiWarps);   // pairs: both CTAs' warps, on the leader
    }
    for (int i = 0; i < C::kEpiSlabs; ++i) {
      mbar_init(&epi_full[i], 1);
      mbar_init(&epi_empty[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, C::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, C::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int u = cta_first; u < args.num_tiles * args.split_k && ok; u += cta_stride) {
      int mt, nt;
      const int split = u / args.num_tiles, t = u - split * args.num_tiles;
      const int kb_begin = split * args.kb_per_split, kb_end = min(kb_begin + args.kb_per_split, args.num_k_blocks);
      const int bi = t / args.tiles_per_batch;
      tile_coords(args, t - bi * args.tiles_per_batch, mt, nt);
      if constexpr (PAIR) mt = mt * 2 + (int)rank;          // this CTA's 128 rows of the 256-row pair tile
      const int b_col0 = nt * BN + (PAIR ? (int)rank * (BN / 2) : 0);   // first B row (output column) this CTA loads
      int a_row = bi * args.M + mt * BM;
      int b_row = (int)(bi * args.b_rows_per_batch) + (PAIR ? b_col0 : nt * C::kBBoxRows);
      if (args.tile_map != nullptr) {
        const int row0 = args.tile_map[3 * mt];
        if (row0 < 0) continue;
        a_row = row0;
        b_row += args.tile_map[3 * mt + 2] * args.expert_rows;
      }
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, args.status, kTimeoutEmpty));
        if (!ok) break;
        if (lane == 0) {
          uint8_t* sa_ptr = stage_base + stage * C::kStageBytes;
          uint8_t* sb_ptr = sa_ptr + C::kABytes;
          constexpr int kBlockElems = 128 / C::kElemBytes;      // MN elements per 128-byte block
          constexpr int kBlockBytes = C::kBK * 128;             // one MN block: kBK K-rows x 128 bytes
          // pairs: both CTAs' copies count on the LEADER's barrier, which expects the bytes of both
          const uint32_t full_addr = PAIR ? mapa_shared(smem_u32(&full_bar[stage]), 0) : 0u;
          auto load = [&](uint8_t* dst, const CUtensorMap* map, int x, int y) {
            if constexpr (PAIR) tma_load_2d_pair(dst, map, full_addr, x, y);
            else tma_load_2d(dst, map, &full_bar[stage], x, y);
          };
          if (!PAIR || rank == 0) mbar_expect_tx(&full_bar[stage], (PAIR ? 2 : 1) * C::kStageBytes);
          if (!args.a_mn) {
            load(sa_ptr, &tmA, kb * C::kBK, a_row);
          } else {
#pragma unroll
            for (int blk = 0; blk < BM / kBlockElems; ++blk)
              load(sa_ptr + blk * kBlockBytes, &tmA, mt * BM + blk * kBlockElems, bi * args.K + kb * C::kBK);
          }
          if (!args.b_mn) {
            load(sb_ptr, &tmB, kb * C::kBK, b_row);
          } else {
#pragma unroll
            for (int blk = 0; blk < (PAIR ? BN / 2 : BN) / kBlockElems; ++blk)
              load(sb_ptr + blk * kBlockBytes, &tmB, b_col0 + blk * kBlockElems, bi * args.K + kb * C::kBK);
          }
          if constexpr (C::kGatedFwd)
            tma_load_2d(sb_ptr + C::kBBoxRows * BK_BYTES, &tmB, &full_bar[stage], kb * C::kBK,
                        b_row + args.b_gate_up_offset);
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    // pairs: only the leader issues; its MMAs and commits act on both CTAs
    for (int u = cta_first; u < args.num_tiles * args.split_k && ok && rank == 0; u += cta_stride) {
      const int split = u / args.num_tiles, t = u - split * args.num_tiles;
      const int kb_begin = split * args.kb_per_split, kb_end = min(kb_begin + args.kb_per_split, args.num_k_blocks);
      if (args.tile_map != nullptr) {
        int mt, nt;
        tile_coords(args, t, mt, nt);
        if (args.tile_map[3 * mt] < 0) continue;
      }
      if constexpr (!GROUP) {
        ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, args.status, kTimeoutTmemEmpty));
        if (!ok) break;
        tc_fence_after_sync();
      }
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if constexpr (GROUP) {
          ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, args.status, kTimeoutTmemEmpty));
          if (!ok) break;
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, args.status, kTimeoutFull));
        if (!ok) break;
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(stage_base + stage * C::kStageBytes);
          const uint32_t b_addr = a_addr + C::kABytes;
          constexpr uint32_t kBlockBytes = C::kBK * 128;
          constexpr uint32_t kMnStep = (32 / C::kElemBytes) * 128;   // K rows of one MMA x 128-byte row pitch
          const uint64_t adesc = args.a_mn ? make_mnmajor_sw128_desc(a_addr, kBlockBytes) : make_kmajor_sw128_desc(a_addr);
          const uint64_t bdesc = args.b_mn ? make_mnmajor_sw128_desc(b_addr, kBlockBytes) : make_kmajor_sw128_desc(b_addr);
          const uint32_t d_tmem = tmem_base + acc * BN;
#pragma unroll
          for (int k = 0; k < C::kMmasPerStage; ++k) {
            const uint32_t accumulate = GROUP ? (k > 0) : (kb > kb_begin || k > 0);
            const uint64_t koff_a = (uint64_t)((k * (args.a_mn ? kMnStep : (uint32_t)C::kUmmaKBytes)) >> 4);
            const uint64_t koff_b = (uint64_t)((k * (args.b_mn ? kMnStep : (uint32_t)C::kUmmaKBytes)) >> 4);
            if constexpr (PAIR) {
              if constexpr (KIND == VB_KIND_F8) mma_f8_ss_pair(d_tmem, adesc + koff_a, bdesc + koff_b, args.idesc, accumulate);
              else mma_f16_ss_pair(d_tmem, adesc + koff_a, bdesc + koff_b, args.idesc, accumulate);
            } else {
              if constexpr (KIND == VB_KIND_F8) mma_f8_ss(d_tmem, adesc + koff_a, bdesc + koff_b, args.idesc, accumulate);
              else mma_f16_ss(d_tmem, adesc + koff_a, bdesc + koff_b, args.idesc, accumulate);
            }
          }
          if constexpr (PAIR) {                 // the stage is free in both CTAs once these MMAs retire
            tc_commit_pair(smem_u32(&empty_bar[stage]));
            tc_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 1));
          } else {
            tc_commit(&empty_bar[stage]);
          }
          if constexpr (GROUP) tc_commit(&tmem_full[acc]);
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        if constexpr (GROUP) {
          if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1; }
        }
      }
      if (!ok) break;
      if constexpr (!GROUP) {
        if (lane == 0) {
          if constexpr (PAIR) {
            tc_commit_pair(smem_u32(&tmem_full[acc]));
            tc_commit_pair(mapa_shared(smem_u32(&tmem_full[acc]), 1));
          } else {
            tc_commit(&tmem_full[acc]);
          }
        }
        __syncwarp();
        if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (C::kSlabLoader && warp == C::kLoaderWarp) {
    // ------------------------------ slab loader --------------------------------
    // Feeds the epilogue's operand slabs (AXPBY residual, ACT_BWD slope) on its own, so a full slab ring never
    // holds back the main-loop producer; it runs up to kEpiSlabs chunks ahead of the epilogue.
    if constexpr (C::kSlabLoader) {
      if (args.epi_stage) {
        int eslot = 0;
        uint32_t ephase = 0;
        bool ok = true;
        constexpr int kHalves = C::kGatedBwd ? 2 : 1;     // gated backward: the gate slab, then the up slab
        for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
          int mt, nt;
          const int bi = t / args.tiles_per_batch;
          tile_coords(args, t - bi * args.tiles_per_batch, mt, nt);
          for (int c = 0; c < BN / 32 && nt * BN + c * 32 < args.N && ok; ++c) {
            for (int half = 0; half < kHalves; ++half) {
              ok = __all_sync(0xffffffffu, mbar_wait(&epi_empty[eslot], ephase ^ 1, abort_flag, args.status, kTimeoutEmpty));
              if (!ok) break;
              if (lane == 0) {
                mbar_expect_tx(&epi_full[eslot], C::kEpiSlabBytes);
                if constexpr (C::kGatedBwd)
                  tma_load_3d(epi_stage + eslot * C::kEpiSlabBytes, &tmC, &epi_full[eslot], nt * BN + c * 32, half,
                              mt * BM);
                else
                  tma_load_2d(epi_stage + eslot * C::kEpiSlabBytes, &tmC, &epi_full[eslot], nt * BN + c * 32,
                              bi * args.M + mt * BM);
              }
              __syncwarp();
              if (++eslot == C::kEpiSlabs) { eslot = 0; ephase ^= 1; }
            }
          }
        }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quad = warp & 3;            // TMEM lane quadrant this warp may read
    const int epi = warp - 2;             // 0 .. kEpiWarps - 1
    const int half = epi >> 2;            // which part of the tile's columns this warp drains (0 with four warps)
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    float out_amax = 0.f;                 // VB_EPI_ACT_BWD: running |out| maximum of this thread
    uint32_t amax_bits = 0;               // ... and the same gathered as float bits by the slab path
    int eslot = 0, prev_slot = -1;        // epilogue slab ring: position, phase, slot awaiting release
    uint32_t ephase = 0;
    constexpr int NCHUNK = BN / 32;
    constexpr int NOUT = (C::kGatedFwd ? NCHUNK / 2 : NCHUNK) / C::kColumnParts;  // output chunks per tile and warp
    const int chunk0 = C::kColumnParts > 1 ? half * NOUT : 0;       // first chunk of this warp
    // slab epilogues with eight warps: this warp's set (0 = warps 2-5, 1 = warps 6-9) takes every `sets`-th chunk
    constexpr bool kTwoSets = (C::kEpiSlab || C::kGatedSlab) && C::kEpiWarps == 8;
    const int sets = kTwoSets ? (args.epi_sets == 2 ? 2 : 1) : 1;
    const int set = kTwoSets ? half : 0;
    if constexpr (C::kEpiSlab) eslot = sets == 2 ? set : 0;
    // gated backward: a chunk owns two consecutive slabs (gate, up), so a set starts two slabs further on
    if constexpr (C::kGatedSlab && C::kGatedBwd) eslot = sets == 2 ? 2 * set : 0;
    for (int u = cta_first; u < args.num_tiles * args.split_k && ok; u += cta_stride) {
      int mt, nt;
      const int split = u / args.num_tiles, t = u - split * args.num_tiles;
      const int bi = t / args.tiles_per_batch;
      tile_coords(args, t - bi * args.tiles_per_batch, mt, nt);
      if constexpr (PAIR) mt = mt * 2 + (int)rank;
      long long grow = (long long)mt * BM + row_in_tile;
      long long row_end = args.M;
      void* const out_base = advance(args.out, bi * args.out_bs, args.out_dtype);
      const void* const resid_base = advance(args.resid, bi * args.resid_bs, args.out_dtype);
      void* const out_t_base = advance(args.out_t, bi * args.out_t_bs, args.out_dtype);
      int expert = 0;
      if (args.tile_map != nullptr) {
        const int row0 = args.tile_map[3 * mt];
        if (row0 < 0) continue;
        grow = (long long)row0 + row_in_tile;
        row_end = args.tile_map[3 * mt + 1];
        expert = args.tile_map[3 * mt + 2];
      }
      const bool row_ok = grow < row_end;
      const int n0 = nt * (C::kGatedFwd ? BN / 2 : BN);  // first logical output column
      const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;

      // Bias of this tile's columns, fetched before the accumulator wait: lane L keeps column c * 32 + L
      // of every chunk and the epilogue broadcasts it with a shuffle (zero past N, so no guard later).
      constexpr bool kHasBias = EPI == VB_EPI_LINEAR || EPI == VB_EPI_GATED_FWD;
      float bias_reg[kHasBias ? NOUT : 1], bias_reg2[C::kGatedFwd ? NOUT : 1];
      if constexpr (kHasBias) {
#pragma unroll
        for (int c = 0; c < NOUT; ++c) {
          const int col = n0 + (chunk0 + c) * 32 + lane;
          const bool in = args.bias != nullptr && col < args.N;
          bias_reg[c] = in ? load_elem(args.bias, col, args.bias_dtype) : 0.f;
          if constexpr (C::kGatedFwd) bias_reg2[c] = in ? load_elem(args.bias, args.N + col, args.bias_dtype) : 0.f;
        }
      }

      constexpr int NW = NCHUNK / (C::kEpiWarps / 4);   // accumulator chunks this warp promotes (from chunk0 on)
      float accr[GROUP ? NW * 32 : 1];
      if constexpr (GROUP) {
#pragma unroll
        for (int j = 0; j < NW * 32; ++j) accr[j] = 0.f;
        // Scales are fetched one K-block ahead (global loads whose latency would otherwise sit between the
        // accumulator wait and the first FMA of every K-block), and the TMEM load of chunk c + 1 is in flight
        // while chunk c is promoted.
        const bool per_col = args.sb_shift < 5;      // a B scale block spans fewer than 32 rows: one value per column
        const int limit_rows = C::kGatedFwd ? 2 * args.N : args.N;
        auto sb_column = [&](int j) -> long long {   // row of B (scale row before the shift) behind tile column j, or -1
          int brow = C::kGatedFwd ? (j < BN / 2 ? n0 + j : args.b_gate_up_offset + n0 + (j - BN / 2)) : n0 + j;
          const bool in = C::kGatedFwd ? (brow - (j < BN / 2 ? 0 : args.b_gate_up_offset) < args.N) : (brow < args.N);
          return in ? (long long)(brow + expert * args.expert_rows) : -1LL;
        };
        auto sb_chunk = [&](int c) -> long long {    // same for a whole 32-column chunk (clamped at the edge)
          int brow = C::kGatedFwd ? (c < NCHUNK / 2 ? n0 + c * 32 : args.b_gate_up_offset + n0 + (c - NCHUNK / 2) * 32)
                                  : n0 + c * 32;
          return (long long)(min(brow, limit_rows - 1) + expert * args.expert_rows);
        };
        float next_sa = 0.f, next_sb[NW];
        auto fetch_scales = [&](int kb) {
          const int ks = kb >> args.k_shift;
          next_sa = row_ok ? args.sa[grow * args.sa_row + (long long)ks * args.sa_k] : 0.f;
#pragma unroll
          for (int c = 0; c < NW; ++c) {
            const long long brow = per_col ? sb_column((chunk0 + c) * 32 + lane) : sb_chunk(chunk0 + c);
            next_sb[c] = brow >= 0 ? args.sb[(brow >> args.sb_shift) * args.sb_row + (long long)ks * args.sb_k] : 0.f;
          }
        };
        fetch_scales(0);
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          const float sa_v = next_sa;
          float sb_v[NW];
#pragma unroll
          for (int c = 0; c < NW; ++c) sb_v[c] = next_sb[c];
          float* sbs = sb_stage + (epi * 2 + (kb & 1)) * (NW * 32);  // private to this warp: no CTA barrier
          if (per_col) {
#pragma unroll
            for (int c = 0; c < NW; ++c) sbs[c * 32 + lane] = sb_v[c];
            __syncwarp();
          }
          ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_phase, abort_flag, args.status, kTimeoutTmemFull));
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t r[2][32];
          tmem_ld_32x32(tmem_base + lane_addr + acc * BN + chunk0 * 32, r[0]);
          if (kb + 1 < args.num_k_blocks) fetch_scales(kb + 1);       // in flight under the promotion below
#pragma unroll
          for (int c = 0; c < NW; ++c) {
            tmem_ld_wait();
            if (c + 1 < NW) tmem_ld_32x32(tmem_base + lane_addr + acc * BN + (chunk0 + c + 1) * 32, r[(c + 1) & 1]);
            if (per_col) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                accr[c * 32 + j] = fmaf(__uint_as_float(r[c & 1][j]), sa_v * sbs[c * 32 + j], accr[c * 32 + j]);
            } else {
              const float s = sa_v * sb_v[c];
#pragma unroll
              for (int j = 0; j < 32; ++j) accr[c * 32 + j] = fmaf(__uint_as_float(r[c & 1][j]), s, accr[c * 32 + j]);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
          if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1; }
        }
        if (!ok) break;
      } else {
        ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_phase, abort_flag, args.status, kTimeoutTmemFull));
        if (!ok) break;
        tc_fence_after_sync();
      }

      const float alpha_pt = GROUP ? 1.f
                                   : (args.sa != nullptr ? args.sa[0] : 1.f) * (args.sb != nullptr ? args.sb[0] : 1.f);
      if constexpr (EPI == VB_EPI_LINEAR && !GROUP) {
        if (split > 0) {
          // split-K: these 32 rows of the tile were last written by unit `split - 1`; its warp of the same
          // quadrant publishes the count once its stores have landed
          bool ready = true;
          if (lane == 0) {
            ready = wait_flag_eq_gpu(args.split_flags + t * 8 + epi, split, abort_flag, args.status, kTimeoutSplit);
            fence_proxy_async_global();
          }
          ok = __all_sync(0xffffffffu, ready);
          if (!ok) break;
        }
      }
      // ---- staged gated epilogues (per-tensor scales, 16-bit outputs): rolled over the chunks, specialised on
      // the 16-bit type and the activation, every result row leaves through a shared-memory slab and a TMA store
      bool staged_done = false;
      if constexpr (C::kGatedSlab) {
        if (args.epi_store) {
          staged_done = true;
          const int warp_row = mt * BM + quad * 32;
          const bool rows_in = warp_row < args.M;
          if constexpr (C::kGatedFwd) {
            // two sets: each set stages through its own two slabs (ring of two), one set: ring of four
            const int ring = sets == 2 ? C::kEpiSlabs / 2 : C::kEpiSlabs;
            auto emit = [&](const uint32_t (&w)[16], int half, int col0) {
              uint8_t* slab = epi_stage + ((sets == 2 ? set * ring : 0) + eslot) * C::kEpiSlabBytes;
              if (lane == 0) {                                          // the store that last read this slab
                if (sets == 2) tma_store_wait_read<C::kEpiSlabs / 2 - 1>();
                else tma_store_wait_read<C::kEpiSlabs - 1>();
              }
              __syncwarp();
#pragma unroll
              for (int p = 0; p < 4; ++p)
                *slab_piece(slab, row_in_tile, p) = make_uint4(w[4 * p], w[4 * p + 1], w[4 * p + 2], w[4 * p + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (rows_in) {
                  if (half < 0) tma_store_2d(&tmC, slab + quad * 32 * 64, col0, warp_row);
                  else tma_store_3d(&tmD, slab + quad * 32 * 64, col0, half, warp_row);
                }
                tma_store_commit();
              }
              if (++eslot == ring) eslot = 0;
            };
            auto fwd_tile = [&](auto dt_tag, auto act_tag) {
              constexpr int DT = decltype(dt_tag)::value;
              constexpr int ACT = decltype(act_tag)::value;
#pragma unroll 1
              for (int c = (set < sets ? set : NOUT); c < NOUT; c += sets) {
                const int col0 = n0 + c * 32;
                if (col0 >= args.N) break;
                uint32_t rg[32], ru[32];
                tmem_ld_32x32(tmem_base + lane_addr + acc * BN + c * 32, rg);
                tmem_ld_32x32(tmem_base + lane_addr + acc * BN + BN / 2 + c * 32, ru);
                float bg = 0.f, bu = 0.f;
#pragma unroll
                for (int i = 0; i < NOUT; ++i)
                  if (i == c) { bg = bias_reg[i]; bu = bias_reg2[i]; }
                tmem_ld_wait();
                uint32_t pg[16], pu[16], ph[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  float g0 = __uint_as_float(rg[2 * j]) * alpha_pt, g1 = __uint_as_float(rg[2 * j + 1]) * alpha_pt;
                  float u0 = __uint_as_float(ru[2 * j]) * alpha_pt, u1 = __uint_as_float(ru[2 * j + 1]) * alpha_pt;
                  if (args.bias != nullptr) {
                    g0 += __shfl_sync(0xffffffffu, bg, 2 * j);
                    g1 += __shfl_sync(0xffffffffu, bg, 2 * j + 1);
                    u0 += __shfl_sync(0xffffffffu, bu, 2 * j);
                    u1 += __shfl_sync(0xffffffffu, bu, 2 * j + 1);
                  }
                  pg[j] = pack_round2<DT>(g0, g1);
                  pu[j] = pack_round2<DT>(u0, u1);
                  const float2 gf = unpack2<DT>(pg[j]), uf = unpack2<DT>(pu[j]);
                  float a0, a1, unused;
                  gate_terms<ACT>(gf.x, a0, unused);
                  gate_terms<ACT>(gf.y, a1, unused);
                  ph[j] = pack_round2<DT>(a0 * uf.x, a1 * uf.y);
                }
                emit(ph, -1, col0);
                if (args.aux != nullptr) {
                  emit(pg, 0, col0);
                  emit(pu, 1, col0);
                }
              }
            };
            auto with_act = [&](auto dt_tag) {
              if (args.activation == VB_ACT_SILU) fwd_tile(dt_tag, std::integral_constant<int, VB_ACT_SILU>{});
              else if (args.activation == VB_ACT_RELU) fwd_tile(dt_tag, std::integral_constant<int, VB_ACT_RELU>{});
              else fwd_tile(dt_tag, std::integral_constant<int, VB_ACT_GELU>{});
            };
            if (args.out_dtype == 1) with_act(std::integral_constant<int, 1>{});
            else with_act(std::integral_constant<int, 2>{});
          } else {
            auto bwd_tile = [&](auto dt_tag, auto act_tag) {
              constexpr int DT = decltype(dt_tag)::value;
              constexpr int ACT = decltype(act_tag)::value;
#pragma unroll 1
              for (int c = (set < sets ? set : NCHUNK); c < NCHUNK; c += sets) {
                const int col0 = n0 + c * 32;
                if (col0 >= args.N) break;
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + lane_addr + acc * BN + c * 32, r);
                uint8_t* slab_g = epi_stage + eslot * C::kEpiSlabBytes;     // saved gate, becomes dGate
                uint8_t* slab_u = slab_g + C::kEpiSlabBytes;                // saved up, becomes dUp
                const bool got = mbar_wait(&epi_full[eslot], ephase, abort_flag, args.status, kTimeoutFull) &&
                                 mbar_wait(&epi_full[eslot + 1], ephase, abort_flag, args.status, kTimeoutFull);
                ok = __all_sync(0xffffffffu, got);
                tmem_ld_wait();
                if (!ok) break;
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                  uint4* gp = slab_piece(slab_g, row_in_tile, p);
                  uint4* up = slab_piece(slab_u, row_in_tile, p);
                  const uint4 gin = *gp, uin = *up;
                  const uint32_t gw[4] = {gin.x, gin.y, gin.z, gin.w}, uw[4] = {uin.x, uin.y, uin.z, uin.w};
                  uint32_t og[4], ou[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 d = unpack2<DT>(pack_round2<DT>(__uint_as_float(r[8 * p + 2 * e]) * alpha_pt,
                                                                 __uint_as_float(r[8 * p + 2 * e + 1]) * alpha_pt));
                    const float2 g = unpack2<DT>(gw[e]), u = unpack2<DT>(uw[e]);
                    float a0, s0, a1, s1;
                    gate_terms<ACT>(g.x, a0, s0);
                    gate_terms<ACT>(g.y, a1, s1);
                    og[e] = pack_round2<DT>(d.x * u.x * s0, d.y * u.y * s1);
                    ou[e] = pack_round2<DT>(d.x * a0, d.y * a1);
                  }
                  *gp = make_uint4(og[0], og[1], og[2], og[3]);
                  *up = make_uint4(ou[0], ou[1], ou[2], ou[3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                  if (rows_in) {
                    tma_store_3d(&tmD, slab_g + quad * 32 * 64, col0, 0, warp_row);
                    tma_store_3d(&tmD, slab_u + quad * 32 * 64, col0, 1, warp_row);
                  }
                  tma_store_commit();
                  if (prev_slot >= 0) {          // the previous chunk's stores have read their slabs by now
                    tma_store_wait_read<1>();
                    mbar_arrive(&epi_empty[prev_slot]);
                    mbar_arrive(&epi_empty[prev_slot + 1]);
                  }
                }
                prev_slot = eslot;
                eslot += 2 * sets;
                if (eslot >= C::kEpiSlabs) { eslot -= C::kEpiSlabs; ephase ^= 1; }
              }
            };
            auto with_act = [&](auto dt_tag) {
              if (args.activation == VB_ACT_SILU) bwd_tile(dt_tag, std::integral_constant<int, VB_ACT_SILU>{});
              else if (args.activation == VB_ACT_RELU) bwd_tile(dt_tag, std::integral_constant<int, VB_ACT_RELU>{});
              else bwd_tile(dt_tag, std::integral_constant<int, VB_ACT_GELU>{});
            };
            if (args.out_dtype == 1) with_act(std::integral_constant<int, 1>{});
            else with_act(std::integral_constant<int, 2>{});
          }
        }
      }
      if (!staged_done) {
#pragma unroll(C::kEpiSlab ? 1 : NOUT)
      for (int c = (kTwoSets ? (set < sets ? set : NOUT) : 0); c < NOUT; c += (kTwoSets ? sets : 1)) {
        float v[32];
        float v2[C::kGatedFwd ? 32 : 1];
        if constexpr (GROUP) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = accr[c * 32 + j];
          if constexpr (C::kGatedFwd) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v2[j] = accr[BN / 2 + c * 32 + j];
          }
        } else {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + lane_addr + acc * BN + (chunk0 + c) * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha_pt;
          if constexpr (C::kGatedFwd) {
            tmem_ld_32x32(tmem_base + lane_addr + acc * BN + BN / 2 + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v2[j] = __uint_as_float(r[j]) * alpha_pt;
          }
        }
        const int col0 = n0 + (chunk0 + c) * 32;
        const bool staged = C::kTmaStore && args.tma_store != 0;
        if (col0 >= args.N && !staged) continue;  // warp-uniform; the producer skips these chunks too
        // slab ring: this chunk's slot holds the operand (once epi_full fires) and then the result
        uint8_t* slab = nullptr;
        if constexpr (C::kEpiSlab) {
          if (args.epi_stage || args.epi_store) {
            slab = epi_stage + eslot * C::kEpiSlabBytes;
            if (args.epi_stage) {
              ok = __all_sync(0xffffffffu, mbar_wait(&epi_full[eslot], ephase, abort_flag, args.status, kTimeoutFull));
              if (!ok) break;
            } else {
              // result staging only: the slot was last used kEpiSlabs / sets of this warp's own chunks ago
              if (lane == 0) {
                if (sets == 2) tma_store_wait_read<C::kEpiSlabs / 2 - 1>();
                else tma_store_wait_read<C::kEpiSlabs - 1>();
              }
              __syncwarp();
            }
          }
        }
        // after the body: store the rewritten rows, then hand the PREVIOUS chunk's slot back to the producer
        // (its store has had this chunk's time to finish reading shared memory)
        auto finish_slab = [&]() {
          if constexpr (C::kEpiSlab) {
            if (slab == nullptr) return;
            if (args.epi_store) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (mt * BM + quad * 32 < args.M)   // rows past M are clipped by the map; a warp wholly past it stores nothing
                  tma_store_2d(&tmD, slab + quad * 32 * 64, col0, (int)(bi * args.M) + mt * BM + quad * 32);
                tma_store_commit();
              }
            }
            if (args.epi_stage) {
              if (args.epi_store) {
                if (prev_slot >= 0) {
                  if (lane == 0) {
                    tma_store_wait_read<1>();
                    mbar_arrive(&epi_empty[prev_slot]);
                  }
                }
                prev_slot = eslot;
              } else {
                __syncwarp();
                if (lane == 0) mbar_arrive(&epi_empty[eslot]);
              }
            }
            eslot += sets;
            if (eslot >= C::kEpiSlabs) { eslot -= C::kEpiSlabs; ephase ^= 1; }
          }
        };
        if constexpr (EPI == VB_EPI_LINEAR) {
          if (args.bias != nullptr && split == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, bias_reg[c], j);
          }
          if (!staged) {
            if (row_ok) store_row32(out_base, args.ldo, args.out_dtype, grow, col0, args.N, v);
          } else {
            // Each warp owns a 4 KB staging region: two 32-row x 64-byte buffers (16-bit results, 64B swizzle,
            // alternating per chunk) or one 32-row x 128-byte buffer (fp32, 128B swizzle).  A lane writes its row's
            // 16-byte pieces at the swizzled position; one lane then issues the TMA store (or, for the later units
            // of a split-K tile, the TMA reduce-add), which clips rows >= M and columns >= N by itself.
            uint8_t* region = store_stage + epi * 4096;
            uint8_t* buffer = region;
            if (args.out_dtype == 0) {
              if (lane == 0) tma_store_wait_read<0>();               // the store that last used this buffer
              __syncwarp();
              uint8_t* row_ptr = buffer + lane * 128;
#pragma unroll
              for (int p = 0; p < 8; ++p)
                *reinterpret_cast<float4*>(row_ptr + ((p ^ (lane & 7)) << 4)) =
                    make_float4(v[4 * p], v[4 * p + 1], v[4 * p + 2], v[4 * p + 3]);
            } else {
              buffer = region + (c & 1) * 2048;
              if (lane == 0) tma_store_wait_read<1>();               // the store of two chunks ago
              __syncwarp();
              uint8_t* row_ptr = buffer + lane * 64;
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                uint4 t;
                t.x = pack2(v[8 * p + 0], v[8 * p + 1], args.out_dtype);
                t.y = pack2(v[8 * p + 2], v[8 * p + 3], args.out_dtype);
                t.z = pack2(v[8 * p + 4], v[8 * p + 5], args.out_dtype);
                t.w = pack2(v[8 * p + 6], v[8 * p + 7], args.out_dtype);
                *reinterpret_cast<uint4*>(row_ptr + ((p ^ ((lane >> 1) & 3)) << 4)) = t;
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            const int warp_row = mt * BM + quad * 32;
            if (lane == 0) {
              if (col0 < args.N && warp_row < args.M) {
                if (split == 0 && !args.accumulate) tma_store_2d(&tmC, buffer, col0, warp_row);
                else tma_reduce_add_2d(&tmC, buffer, col0, warp_row);
              }
              tma_store_commit();
            }
          }
        } else if constexpr (EPI == VB_EPI_AXPBY) {
          if (slab != nullptr && args.epi_store && (args.epi_stage || resid_base == nullptr)) {
            uint32_t unused = 0;
            if (args.out_dtype == 1)
              slab_row_epilogue<EPI, 1>(v, slab, row_in_tile, args.epi_stage != 0, args.alpha, args.beta, unused);
            else
              slab_row_epilogue<EPI, 2>(v, slab, row_in_tile, args.epi_stage != 0, args.alpha, args.beta, unused);
            finish_slab();
            continue;
          }
          float res[32];
          if (slab != nullptr && args.epi_stage) load_slab32(slab, row_in_tile, args.out_dtype, res);
          else if (resid_base != nullptr && row_ok) load_row32(resid_base, args.ldr, args.out_dtype, grow, col0, args.N, res);
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) res[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = round_to(args.alpha * round_to(v[j], args.out_dtype) + args.beta * res[j], args.out_dtype);
          if (slab != nullptr && args.epi_store) store_slab32(slab, row_in_tile, args.out_dtype, v);   // TMA clips
          else if (row_ok) store_row32(out_base, args.ldo, args.out_dtype, grow, col0, args.N, v);
          void* tbase = out_t_base;
          long long tld = args.ldot;
          if (args.symmetric && mt != nt) { tbase = out_base; tld = args.ldo; }
          if (tbase != nullptr && row_ok) {
            // transposed copy: lanes hold consecutive rows -> consecutive addresses per column
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < args.N) store_elem(tbase, (long long)(col0 + j) * tld + grow, args.out_dtype, v[j]);
          }
        } else if constexpr (EPI == VB_EPI_GATED_FWD) {
          if (args.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] += __shfl_sync(0xffffffffu, bias_reg[c], j);
              v2[j] += __shfl_sync(0xffffffffu, bias_reg2[c], j);
            }
          }
          float h[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = round_to(v[j], args.out_dtype);
            v2[j] = round_to(v2[j], args.out_dtype);
            h[j] = act_fn(v[j], args.activation) * v2[j];
          }
          if (row_ok) {
            store_row32(args.out, args.ldo, args.out_dtype, grow, col0, args.N, h);
            if (args.aux != nullptr) {
              store_row32(args.aux, args.ldaux, args.out_dtype, grow, col0, args.N, v);
              // "up" half lives at column offset N; bound by 2N but chunk validity is the same
              float* dummy = nullptr; (void)dummy;
              const long long off_cols = args.N;
              // shift base pointer by N columns
              void* up_base = (args.out_dtype == 0)
                                  ? (void*)(reinterpret_cast<float*>(args.aux) + off_cols)
                                  : (void*)(reinterpret_cast<uint16_t*>(args.aux) + off_cols);
              store_row32(up_base, args.ldaux, args.out_dtype, grow, col0, args.N, v2);
            }
          }
        } else if constexpr (EPI == VB_EPI_ACT_BWD) {  // v = d; aux = act'(z) saved by the forward; out = d * aux, with its amax
          if (slab != nullptr && args.epi_store && args.epi_stage) {
            if (args.out_dtype == 1) slab_row_epilogue<EPI, 1>(v, slab, row_in_tile, true, 0.f, 0.f, amax_bits);
            else slab_row_epilogue<EPI, 2>(v, slab, row_in_tile, true, 0.f, 0.f, amax_bits);
            finish_slab();
            continue;
          }
          {
            float z[32], o[32];
            if (slab != nullptr && args.epi_stage) load_slab32(slab, row_in_tile, args.out_dtype, z);
            else if (row_ok) load_row32(args.aux, args.ldaux, args.out_dtype, grow, col0, args.N, z);
            else {
#pragma unroll
              for (int j = 0; j < 32; ++j) z[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              o[j] = round_to(round_to(v[j], args.out_dtype) * z[j], args.out_dtype);
              if (row_ok && col0 + j < args.N) out_amax = fmaxf(out_amax, (o[j] != o[j]) ? INFINITY : fabsf(o[j]));
            }
            if (slab != nullptr && args.epi_store) store_slab32(slab, row_in_tile, args.out_dtype, o);
            else if (row_ok) store_row32(args.out, args.ldo, args.out_dtype, grow, col0, args.N, o);
          }
        } else {  // VB_EPI_GATED_BWD: v = d; aux = [g | u]; out = [dG | dU]
          if (row_ok) {
            float g[32], u[32], dg[32], du[32];
            const void* up_base = (args.out_dtype == 0)
                                      ? (const void*)(reinterpret_cast<const float*>(args.aux) + args.N)
                                      : (const void*)(reinterpret_cast<const uint16_t*>(args.aux) + args.N);
            load_row32(args.aux, args.ldaux, args.out_dtype, grow, col0, args.N, g);
            load_row32(up_base, args.ldaux, args.out_dtype, grow, col0, args.N, u);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float d = round_to(v[j], args.out_dtype);
              dg[j] = d * u[j] * act_grad(g[j], args.activation);
              du[j] = d * act_fn(g[j], args.activation);
            }
            void* out_up = (args.out_dtype == 0) ? (void*)(reinterpret_cast<float*>(args.out) + args.N)
                                                 : (void*)(reinterpret_cast<uint16_t*>(args.out) + args.N);
            store_row32(args.out, args.ldo, args.out_dtype, grow, col0, args.N, dg);
            store_row32(out_up, args.ldo, args.out_dtype, grow, col0, args.N, du);
          }
        }
        finish_slab();
      }
      }
      if constexpr (!GROUP) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[acc]), 0));   // on the leader
          else mbar_arrive(&tmem_empty[acc]);
        }
        if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1; }
      }
      if constexpr (EPI == VB_EPI_LINEAR && !GROUP) {
        if (args.split_k > 1 && ok) {
          // hand the rows to the next unit of this tile once every store of this warp has landed; the last
          // unit leaves the counter at zero for the next launch
          if (lane == 0) {
            tma_store_wait_all();
            fence_proxy_async_global();
            st_release_gpu(args.split_flags + t * 8 + epi, split + 1 == args.split_k ? 0 : split + 1);
          }
          __syncwarp();
        }
      }
    }
    if constexpr (C::kSlabRing) {
      if (lane == 0) tma_store_wait_all();   // stores read this CTA's shared memory until they finish
    }
    if constexpr (EPI == VB_EPI_ACT_BWD) {
      // non-negative floats order like their bit patterns (+inf, the stand-in for NaN, included)
      uint32_t m = max(__float_as_uint(out_amax), min(amax_bits, 0x7f800000u));   // NaN counts as +inf
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
      if (lane == 0 && args.amax_out != nullptr) atomicMax(args.amax_out, m);
    }
  }

  if constexpr (C::kTmaStore) {
    if (warp >= 2 && lane == 0) tma_store_wait_all();   // stores read this CTA's shared memory until they finish
  }
  // ------------------------------ teardown ------------------------------------
  // On the error path TMA copies may still be in flight towards this CTA's shared memory:
  // give them a bounded grace period before the CTA (and its smem) goes away.
  if (*abort_flag) {
    const long long start = clock64();
    while (clock64() - start < 2000000LL) { __nanosleep(256); }
  }
  tc_fence_before_sync();
  // pairs: neither CTA may leave while the other can still read its shared memory or arrive on its barriers
  if constexpr (PAIR) cluster_sync_all();
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, C::kTmemCols);
    else tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// Builds the tile -> (row0, row_end, expert) map for the expert GEMM from device offsets.
__global__ void expert_tile_map_kernel(const int* __restrict__ offsets, int num_experts, int max_tiles,
                                       int* __restrict__ tile_map) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int t = 0;
  for (int e = 0; e < num_experts; ++e) {
    const int begin = offsets[e], end = offsets[e + 1];
    for (int r = begin; r < end && t < max_tiles; r += BM) {
      tile_map[3 * t] = r;
      tile_map[3 * t + 1] = end;
      tile_map[3 * t + 2] = e;
      ++t;
    }
  }
  for (; t < max_tiles; ++t) {
    tile_map[3 * t] = -1;
    tile_map[3 * t + 1] = 0;
    tile_map[3 * t + 2] = 0;
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D K-major tensor map: inner dim = K (contiguous), outer = rows; box = (128 bytes of K) x box_rows.
static int make_map(CUtensorMap* map, const void* base, int kind, int fmt, long long rows, long long k,
                    long long ld_elems, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  const int elem = kind == VB_KIND_F8 ? 1 : 2;
  CUtensorMapDataType dt = kind == VB_KIND_F8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                              : (fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld_elems * elem)};
  cuuint32_t box[2] = {(cuuint32_t)(BK_BYTES / elem), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (strides[0] & 15) != 0) return (int)cudaErrorMisalignedAddress;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Tensor map for an MN-major operand stored as [k_rows, mn] row-major: box = 128 bytes of MN x box_k rows.
static int make_map_mn(CUtensorMap* map, const void* base, int kind, int fmt, long long k_rows, long long mn,
                       long long ld_elems, int box_k) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  const int elem = kind == VB_KIND_F8 ? 1 : 2;
  CUtensorMapDataType dt = kind == VB_KIND_F8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                              : (fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {(cuuint64_t)mn, (cuuint64_t)k_rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld_elems * elem)};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem), (cuuint32_t)box_k};
  cuuint32_t estr[2] = {1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (strides[0] & 15) != 0) return (int)cudaErrorMisalignedAddress;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Tensor map of a 16-bit [rows, cols] matrix moved in epilogue slabs: box = 32 columns (64 bytes) x box_rows rows,
// 64B swizzle (128 rows for the operand load, 32 for one warp's result store).
static int make_slab_map(CUtensorMap* map, const void* base, int dtype, long long rows, long long cols, long long ld_elems,
                         int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  CUtensorMapDataType dt = dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld_elems * 2)};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Tensor map of a 16-bit [rows, 2 * cols] matrix holding two [rows, cols] halves side by side (the gate | up
// layout of the gated MLP), as a 3-D tensor (column, half, row): a slab is 32 columns x 1 half x box_rows rows, and
// columns past `cols` are clipped (stores) or zero (loads) instead of running into the other half.
static int make_half_map(CUtensorMap* map, const void* base, int dtype, long long rows, long long cols, long long ld_elems,
                         int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  CUtensorMapDataType dt = dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[3] = {(cuuint64_t)cols, 2, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)(cols * 2), (cuuint64_t)(ld_elems * 2)};
  cuuint32_t box[3] = {32, 1, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  if ((strides[0] & 15) != 0 || (strides[1] & 15) != 0 || ld_elems < 2 * cols) return (int)cudaErrorInvalidValue;
  CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Output tensor map for the TMA-store epilogue: box = 128 bytes of columns x 32 rows, 128B swizzle.
static int make_out_map(CUtensorMap* map, void* base, int out_dtype, long long rows, long long cols, long long ld_elems) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  const int elem = out_dtype == 0 ? 4 : 2;
  CUtensorMapDataType dt = out_dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                          : (out_dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld_elems * elem)};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem), 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

static int sm_count() {
  static int count = 0;
  if (count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    if (count <= 0) count = 148;
  }
  return count;
}

// Hand-over counters of split-K launches: one per output tile and epilogue warp, eight regions used in rotation so that launches
// in flight on different streams do not share counters.  Every launch leaves its region at zero.
constexpr int kSplitMaxTiles = 2048, kSplitRegions = 8;
__device__ int g_split_flags[kSplitRegions * kSplitMaxTiles * 8];

// Work units per output tile for a [tiles] x [k_blocks] problem on `sms` persistent CTAs: whole waves of equal units,
// each paying a fixed prologue / epilogue cost of about `overhead` K-blocks; 1 = no split.
static int choose_split(long long tiles, int k_blocks, int sms, double* cost_out = nullptr) {
  const double overhead = 6.0;
  int best = 1;
  double best_cost = (double)((tiles + sms - 1) / sms) * (k_blocks + overhead);
  if (tiles > 0 && tiles <= kSplitMaxTiles) {
    for (int s = 2; s <= 16 && s * 8 <= k_blocks; ++s) {
      const int per = (k_blocks + s - 1) / s;
      if ((s - 1) * per >= k_blocks) continue;                  // an empty last unit
      const long long waves = (tiles * s + sms - 1) / sms;
      const double cost = (double)waves * (per + overhead) * 1.03;   // a split must win clearly
      if (cost < best_cost) { best_cost = cost; best = s; }
    }
  }
  if (cost_out != nullptr) *cost_out = best_cost;
  return best;
}

static int* split_flag_base() {
  static int* base[64] = {};
  static std::mutex lock;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> guard(lock);
  if (base[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_split_flags) != cudaSuccess) return nullptr;
    base[dev] = static_cast<int*>(ptr);
  }
  return base[dev];
}

template <int KIND, int BN, bool GROUP, int EPI, bool PAIR = false>
static int launch(const VbGemmDesc& d, cudaStream_t stream, int split = 1) {
  using C = Config<KIND, BN, GROUP, EPI, PAIR>;
  GemmArgs a{};
  a.M = d.M; a.N = d.N; a.K = d.K;
  const bool expert = d.expert_offsets != nullptr;
  constexpr int kTileRows = PAIR ? 2 * BM : BM;       // rows of one scheduled tile (a CTA pair covers 256)
  if (PAIR && (expert || d.batch > 1 || d.symmetric)) return (int)cudaErrorInvalidValue;
  a.num_m_tiles = expert ? (d.M + BM - 1) / BM + d.num_experts : (d.M + kTileRows - 1) / kTileRows;
  constexpr int n_per_tile = C::kGatedFwd ? BN / 2 : BN;
  a.num_n_tiles = (d.N + n_per_tile - 1) / n_per_tile;
  a.num_k_blocks = (d.K + C::kBK - 1) / C::kBK;
  if (d.symmetric) {
    if (d.M != d.N || BN != BM || expert) return (int)cudaErrorInvalidValue;
    a.tiles_per_batch = a.num_m_tiles * (a.num_m_tiles + 1) / 2;
  } else {
    a.tiles_per_batch = a.num_m_tiles * a.num_n_tiles;
  }
  a.batch = d.batch > 1 ? d.batch : 1;
  if (a.batch > 1 && (expert || EPI == VB_EPI_GATED_FWD || EPI == VB_EPI_GATED_BWD)) return (int)cudaErrorInvalidValue;
  a.num_tiles = a.batch * a.tiles_per_batch;
  a.b_rows_per_batch = d.N;
  a.out_bs = d.out_batch_stride; a.resid_bs = d.resid_batch_stride; a.out_t_bs = d.out_t_batch_stride;
  a.a_mn = d.a_mn_major ? 1 : 0;
  a.b_mn = d.b_mn_major ? 1 : 0;
  if ((a.a_mn || a.b_mn) && (expert || C::kGatedFwd)) return (int)cudaErrorInvalidValue;
  if ((a.a_mn || a.b_mn) && d.batch > 1 && d.K % C::kBK != 0) return (int)cudaErrorInvalidValue;
  a.idesc = make_idesc(d.a_fmt, d.b_fmt, kTileRows, BN, a.a_mn, a.b_mn);
  a.b_gate_up_offset = d.N;
  a.sa = d.sa; a.sb = d.sb;
  a.sa_row = d.sa_row; a.sa_k = d.sa_k; a.sb_row = d.sb_row; a.sb_k = d.sb_k;
  a.sb_shift = d.sb_shift; a.k_shift = d.k_shift;
  a.out = d.out; a.out_dtype = d.out_dtype; a.ldo = d.ldo;
  a.bias = d.bias; a.bias_dtype = d.bias_dtype;
  a.amax_out = d.amax_out;
  a.alpha = d.alpha; a.beta = d.beta; a.resid = d.resid; a.ldr = d.ldr;
  a.out_t = d.out_t; a.ldot = d.ldot; a.symmetric = d.symmetric;
  a.activation = d.activation; a.aux = d.aux; a.ldaux = d.ldaux;
  a.tile_map = expert ? d.tile_map : nullptr;
  a.expert_rows = d.N;
  a.status = d.status;
  if (a.num_tiles <= 0 || a.num_k_blocks <= 0) return 0;

  const long long b_rows = (long long)(C::kGatedFwd ? 2 : 1) * d.N * (expert ? d.num_experts : 1) * a.batch;
  CUtensorMap tmA, tmB;
  int rc = a.a_mn ? make_map_mn(&tmA, d.A, KIND, d.a_fmt, (long long)(d.k_mn > 0 ? d.k_mn : d.K) * a.batch, d.M, d.lda, C::kBK)
                  : make_map(&tmA, d.A, KIND, d.a_fmt, (long long)d.M * a.batch, d.K, d.lda, BM);
  if (rc) return rc;
  rc = a.b_mn ? make_map_mn(&tmB, d.B, KIND, d.b_fmt, (long long)(d.k_mn > 0 ? d.k_mn : d.K) * a.batch, d.N, d.ldb, C::kBK)
              : make_map(&tmB, d.B, KIND, d.b_fmt, b_rows, d.K, d.ldb, C::kBBoxRows);
  if (rc) return rc;
  CUtensorMap tmC = tmA;
  a.tma_store = 0;
  if (C::kTmaStore && !expert && a.batch == 1 && !d.no_tma_store) {
    const int elem = d.out_dtype == 0 ? 4 : 2;
    // fp32: 32 columns = 128-byte rows (128B swizzle); 16-bit: 32 columns = 64-byte rows (64B swizzle)
    if ((reinterpret_cast<uintptr_t>(d.out) & 15) == 0 && (d.ldo * elem) % 16 == 0 &&
        (d.out_dtype == 0 ? make_out_map(&tmC, d.out, d.out_dtype, d.M, d.N, d.ldo)
                          : make_slab_map(&tmC, d.out, d.out_dtype, d.M, d.N, d.ldo, 32)) == 0)
      a.tma_store = 1;
  }
  CUtensorMap tmD = tmA;
  a.epi_sets = 1;
  if constexpr (C::kEpiSlab) {
    // an even number of chunks in every tile keeps "even chunks / odd chunks" aligned with the loader's global order
    // (the activation-slope epilogue, whose operand slabs come from DRAM, needs the deeper ring of eight slabs for
    // this: with four slabs shared by two sets it lost the loader's look-ahead and got slower)
    a.epi_sets = (C::kEpiWarps == 8 && d.N % 64 == 0) ? 2 : 1;
    auto usable = [](const void* p, long long ld) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld * 2) % 16 == 0; };
    const void* src = EPI == VB_EPI_AXPBY ? d.resid : d.aux;
    const long long ld = EPI == VB_EPI_AXPBY ? d.ldr : d.ldaux;
    const long long bs = EPI == VB_EPI_AXPBY ? d.resid_batch_stride : 0;
    // a stack is moved as one [batch * M, N] matrix: it must be dense, and whole tiles per matrix for the store
    if (d.out_dtype != 0 && usable(src, ld) && (a.batch == 1 || bs == (long long)d.M * ld) &&
        make_slab_map(&tmC, src, d.out_dtype, (long long)d.M * a.batch, d.N, ld, BM) == 0)
      a.epi_stage = 1;
    if (d.out_dtype != 0 && usable(d.out, d.ldo) && !d.symmetric && d.out_t == nullptr &&
        (a.batch == 1 || (d.M % BM == 0 && d.out_batch_stride == (long long)d.M * d.ldo)) &&
        make_slab_map(&tmD, d.out, d.out_dtype, (long long)d.M * a.batch, d.N, d.ldo, 32) == 0)
      a.epi_store = 1;
  }
  if constexpr (C::kGatedSlab) {
    // forward: two sets, each staging through its own two slabs (186 -> 164 us at 32768 x 2*1728 x 1152).  Backward:
    // one active set; with two, each chunk's pair of operand slabs shares the eight-slab ring's look-ahead and the
    // kernel got slower (159 -> 189 us), as the activation-slope epilogue did on four slabs.
    a.epi_sets = (C::kEpiWarps == 8 && C::kGatedFwd) ? 2 : 1;
    auto usable = [](const void* p, long long ld) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld * 2) % 16 == 0; };
    const bool shape_ok = !expert && a.batch == 1 && d.out_dtype != 0 && d.N % 8 == 0 && !d.no_tma_store;
    if constexpr (C::kGatedFwd) {
      if (shape_ok && usable(d.out, d.ldo) && (d.aux == nullptr || usable(d.aux, d.ldaux)) &&
          make_slab_map(&tmC, d.out, d.out_dtype, d.M, d.N, d.ldo, 32) == 0 &&
          (d.aux == nullptr || make_half_map(&tmD, d.aux, d.out_dtype, d.M, d.N, d.ldaux, 32) == 0))
        a.epi_store = 1;
    } else {
      if (shape_ok && usable(d.aux, d.ldaux) && usable(d.out, d.ldo) &&
          make_half_map(&tmC, d.aux, d.out_dtype, d.M, d.N, d.ldaux, BM) == 0 &&
          make_half_map(&tmD, d.out, d.out_dtype, d.M, d.N, d.ldo, 32) == 0)
        a.epi_stage = a.epi_store = 1;
    }
  }
  if (expert) {
    expert_tile_map_kernel<<<1, 32, 0, stream>>>(d.expert_offsets, d.num_experts, a.num_m_tiles, d.tile_map);
  }
  a.split_k = 1;
  a.kb_per_split = a.num_k_blocks;
  a.accumulate = 0;
  if (d.accumulate_out) {
    // adding into the output needs the TMA reduce path, which exists for fp32 LINEAR results only
    if (EPI != VB_EPI_LINEAR || !a.tma_store || d.out_dtype != 0 || d.bias != nullptr) return (int)cudaErrorInvalidValue;
    a.accumulate = 1;
  }
  if constexpr (EPI == VB_EPI_LINEAR && !GROUP) {
    // split-K needs the TMA path (reduce-add stores), an fp32 result and one problem per launch
    if (!PAIR && split > 1 && a.tma_store && d.out_dtype == 0 && a.batch == 1 && a.num_tiles <= kSplitMaxTiles) {
      const int per = (a.num_k_blocks + split - 1) / split;
      if ((split - 1) * per < a.num_k_blocks) {
        static std::atomic<unsigned> rotation{0};
        int* flags = split_flag_base();
        if (flags != nullptr) {
          a.split_k = split;
          a.kb_per_split = per;
          a.split_flags = flags + (rotation.fetch_add(1) % kSplitRegions) * kSplitMaxTiles * 8;
        }
      }
    }
  }
  auto kernel = gemm_kernel<KIND, BN, GROUP, EPI, PAIR>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if constexpr (PAIR) {
    if (!a.tma_store) return (int)cudaErrorInvalidValue;      // the pair kernel has no other way out
    // one cluster of two CTAs per scheduled tile, at most one cluster per pair of SMs
    const int clusters = (int)std::min<long long>(a.num_tiles, sm_count() / 2);
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(2 * clusters);
    config.blockDim = dim3(C::kCtaThreads);
    config.dynamicSmemBytes = C::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&config, kernel, tmA, tmB, tmC, tmD, a);
  }
  const int grid = (int)std::min<long long>((long long)a.num_tiles * a.split_k, sm_count());
  kernel<<<grid, C::kCtaThreads, C::kSmemBytes, stream>>>(tmA, tmB, tmC, tmD, a);
  return (int)cudaGetLastError();
}

}  // namespace vb

using namespace vb;

extern "C" int vb_gemm(const VbGemmDesc* desc, cudaStream_t stream) {
  const VbGemmDesc& d = *desc;
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return 0;
  const int elem = d.kind == VB_KIND_F8 ? 1 : 2;
  if ((d.K * elem) % 16 != 0 && !(d.a_mn_major && d.b_mn_major)) return (int)cudaErrorInvalidValue;
  const int sms = sm_count();
  int bn = d.force_bn;
  const bool group = d.group != 0;
  if (bn == 0) {
    if (group || d.symmetric) bn = 128;
    else {
      // whole waves of the persistent grid: a 128-wide tile costs about 0.73 of a 256-wide one (measured), so
      // the narrow tile wins when it saves a partially filled wave
      const long long rows = (long long)((d.M + 127) / 128) * (d.batch > 1 ? d.batch : 1);
      const long long waves256 = (rows * ((d.N + 255) / 256) + sms - 1) / sms;
      const long long waves128 = (rows * ((d.N + 127) / 128) + sms - 1) / sms;
      bn = (d.N > 128 && 100 * waves256 <= 73 * waves128) ? 256 : 128;
      if (d.epilogue == VB_EPI_GATED_FWD) bn = 256;
    }
  }
  // split-K for fp32 results (weight gradients: few output tiles, long K): width and unit count are chosen together
  int split = d.force_split > 0 ? d.force_split : 1;
  if (d.force_split == 0 && d.epilogue == VB_EPI_LINEAR && !group && !d.symmetric && d.out_dtype == 0 &&
      d.expert_offsets == nullptr && d.batch <= 1 && !d.no_tma_store) {
    const int k_blocks = (int)(((long long)d.K * elem + BK_BYTES - 1) / BK_BYTES);
    const long long rows = (d.M + 127) / 128;
    double cost128 = 0.0, cost256 = 0.0;
    const int split128 = choose_split(rows * ((d.N + 127) / 128), k_blocks, sms, &cost128);
    const int split256 = choose_split(rows * ((d.N + 255) / 256), k_blocks, sms, &cost256);
    cost128 *= 0.73;
    if (d.force_bn == 0 && d.N > 128 && (split128 > 1 || split256 > 1)) bn = cost256 <= cost128 ? 256 : 128;
    split = bn == 256 ? split256 : split128;
  }
  // CTA pairs (256 x 256 tiles): per-tensor LINEAR results leaving through TMA, enough tiles to fill the clusters
  // (measured equal to the single-CTA 128 x 256 kernel on DiT and 8192-cubed shapes, whose main loops are already
  // power-bound: chosen only on request, i.e. by the tile tuner when it wins on a shape)
  bool pair = d.force_bn == 512;
  const int out_elem = d.out_dtype == 0 ? 4 : 2;
  if (d.epilogue != VB_EPI_LINEAR || group || d.symmetric || d.expert_offsets != nullptr || d.batch > 1 || d.no_tma_store ||
      (reinterpret_cast<uintptr_t>(d.out) & 15) != 0 || (d.ldo * out_elem) % 16 != 0 || split != 1)
    pair = false;
  if (d.force_bn == 512 && !pair) bn = 256;
#define VB_LAUNCH(KIND, BNV, GROUPV, EPIV) return launch<KIND, BNV, GROUPV, EPIV>(d, stream, split)
  if (pair) {
    if (d.kind == VB_KIND_F8) return launch<VB_KIND_F8, 256, false, VB_EPI_LINEAR, true>(d, stream, 1);
    return launch<VB_KIND_F16, 256, false, VB_EPI_LINEAR, true>(d, stream, 1);
  }
  if (d.kind == VB_KIND_F8) {
    switch (d.epilogue) {
      case VB_EPI_LINEAR:
        if (group) { VB_LAUNCH(VB_KIND_F8, 128, true, VB_EPI_LINEAR); }
        if (bn == 256) { VB_LAUNCH(VB_KIND_F8, 256, false, VB_EPI_LINEAR); }
        VB_LAUNCH(VB_KIND_F8, 128, false, VB_EPI_LINEAR);
      case VB_EPI_GATED_FWD:
        if (group) { VB_LAUNCH(VB_KIND_F8, 128, true, VB_EPI_GATED_FWD); }
        VB_LAUNCH(VB_KIND_F8, 256, false, VB_EPI_GATED_FWD);
      case VB_EPI_GATED_BWD:
        if (group) { VB_LAUNCH(VB_KIND_F8, 128, true, VB_EPI_GATED_BWD); }
        VB_LAUNCH(VB_KIND_F8, 128, false, VB_EPI_GATED_BWD);
      case VB_EPI_ACT_BWD:
        if (group || d.aux == nullptr) return (int)cudaErrorInvalidValue;
        if (bn == 256) { VB_LAUNCH(VB_KIND_F8, 256, false, VB_EPI_ACT_BWD); }
        VB_LAUNCH(VB_KIND_F8, 128, false, VB_EPI_ACT_BWD);
      default:
        return (int)cudaErrorInvalidValue;
    }
  } else {
    if (group) return (int)cudaErrorInvalidValue;
    switch (d.epilogue) {
      case VB_EPI_LINEAR:
        if (bn == 256) { VB_LAUNCH(VB_KIND_F16, 256, false, VB_EPI_LINEAR); }
        VB_LAUNCH(VB_KIND_F16, 128, false, VB_EPI_LINEAR);
      case VB_EPI_AXPBY:
        if (bn == 256 && !d.symmetric) { VB_LAUNCH(VB_KIND_F16, 256, false, VB_EPI_AXPBY); }
        VB_LAUNCH(VB_KIND_F16, 128, false, VB_EPI_AXPBY);
      default:
        return (int)cudaErrorInvalidValue;
    }
  }
#undef VB_LAUNCH
}
