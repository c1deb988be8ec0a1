// MXFP8 GEMM on the hardware block-scaled tensor-core path of sm_100a.
//
//   out[m, n] = sum_k  (A[m, k] * 2^(sfa[m, k / 32] - 127)) * (B[n, k] * 2^(sfb[n, k / 32] - 127))  (+ bias[n])
//
// A [M, K] and B [N, K] hold e4m3 / e5m2 codes, K contiguous; sfa / sfb hold one UE8M0 scale byte per 32
// consecutive K elements of every row.  The scales are applied by the tensor core itself:
// `tcgen05.mma.kind::mxf8f6f4.block_scale` reads them from tensor memory, where `tcgen05.cp` has put them.
// The reference reaches the same arithmetic with `mma.sync ... kind::mxf8f6f4.block_scale` on consumer
// Blackwell only (viola/nn/_grouped_kernels.py:174-192, 250-266; it asserts compute capability 12).
//
// Layout of the scale bytes in global memory ("tiled"): one 512-byte chunk per (128-row tile, 128-element K
// block); inside a chunk the byte of (row r, K group g) sits at (r % 32) * 16 + (r / 32) * 4 + g.  A chunk is
// then exactly the 32 x 128-bit source pattern of `tcgen05.cp.32x128b.warpx4`, which leaves, in each of the
// four 32-lane quadrants of tensor memory, lane l / 32-bit column j / byte g = scale of row 32 j + l, group g:
// the placement the instruction expects for a 128-row operand (the byte within the column is selected by the
// scale-factor id field of the instruction descriptor).  vb_mx_pack_scales produces this layout.
//
// Kernel shape: persistent over 128 x 128 output tiles; 192 threads: warp 0 = TMA producer (A and B boxes with
// SWIZZLE_128B plus two 512-byte bulk copies of scale chunks per stage, never multicast), warp 1 = tensor
// memory owner and MMA issuer (two tcgen05.cp + four K = 32 MMAs per stage from one lane), warps 2-5 = epilogue
// (tcgen05.ld, bias, cast, row stores).  Two accumulators alternate so the epilogue of a tile overlaps the
// main loop of the next.  Every wait is bounded and reports through the status word.
#include <algorithm>
#include <mutex>

#include "api.h"
#include "common/numerics.cuh"
#include "common/ptx.cuh"

namespace vb {
namespace mx {

constexpr int kBM = 128, kBN = 128, kBK = 128;          // kBK in elements = bytes
constexpr int kStages = 6;
constexpr int kTileBytes = kBM * kBK;                    // 16 KiB per operand
constexpr int kSfBytes = 512;
constexpr int kStageBytes = 2 * kTileBytes + 2 * kSfBytes;   // 33792 = 33 * 1024: stages stay 1024-byte aligned
constexpr int kAcc = 2;
constexpr int kSfColumn0 = kAcc * kBN;                   // scale columns follow the accumulators
constexpr int kTmemColumns = 512;
constexpr int kThreads = 192;
constexpr int kBarrierBytes = 1024;
constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;   // + slack for the 1024-byte round-up

struct Args {
  int M, N, K;
  int num_k_blocks, m_tiles, n_tiles, num_tiles;
  const uint8_t* sfa;      // tiled: [m_tiles][num_k_blocks][512]
  const uint8_t* sfb;      // tiled: [n_tiles][num_k_blocks][512]
  void* out; int out_dtype; long long ldo;
  const void* bias; int bias_dtype;
  uint32_t idesc;
  int* status;
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Shared-memory descriptor of one scale chunk for tcgen05.cp: 32 rows of 16 bytes, no swizzle; groups of eight
// rows (one 8 x 16-byte core matrix) are 128 bytes apart.
__device__ __forceinline__ uint64_t make_scale_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                 // leading byte offset (no second chunk along K: not used)
  d |= (uint64_t)(128 >> 4) << 32;        // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                 // descriptor version of this architecture
  return d;                               // layout type 0: no swizzle
}

__device__ __forceinline__ void copy_scales_to_tmem(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void mma_block_scaled(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate, uint32_t tsfa, uint32_t tsfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      :
      : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;                    // [kStages]
  uint64_t* empty_bar = bars + kStages;         // [kStages]
  uint64_t* tmem_full = bars + 2 * kStages;     // [kAcc]
  uint64_t* tmem_empty = tmem_full + kAcc;      // [kAcc]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + kAcc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < kAcc; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemColumns);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
      const int mt = t / args.n_tiles, nt = t - mt * args.n_tiles;
      for (int kb = 0; kb < args.num_k_blocks; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, args.status, kTimeoutEmpty));
        if (!ok) break;
        if (lane == 0) {
          uint8_t* a_ptr = smem + stage * kStageBytes;
          uint8_t* b_ptr = a_ptr + kTileBytes;
          uint8_t* sfa_ptr = b_ptr + kTileBytes;
          uint8_t* sfb_ptr = sfa_ptr + kSfBytes;
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_2d(a_ptr, &tmA, &full_bar[stage], kb * kBK, mt * kBM);
          tma_load_2d(b_ptr, &tmB, &full_bar[stage], kb * kBK, nt * kBN);
          bulk_load(sfa_ptr, args.sfa + ((long long)mt * args.num_k_blocks + kb) * kSfBytes, kSfBytes, &full_bar[stage]);
          bulk_load(sfb_ptr, args.sfb + ((long long)nt * args.num_k_blocks + kb) * kSfBytes, kSfBytes, &full_bar[stage]);
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
      ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, args.status, kTimeoutTmemEmpty));
      if (!ok) break;
      tc_fence_after_sync();
      for (int kb = 0; kb < args.num_k_blocks; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, args.status, kTimeoutFull));
        if (!ok) break;
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(smem + stage * kStageBytes);
          const uint32_t b_addr = a_addr + kTileBytes;
          const uint32_t sfa_addr = b_addr + kTileBytes;
          const uint32_t sfb_addr = sfa_addr + kSfBytes;
          const uint32_t tsfa = tmem_base + kSfColumn0 + stage * 8;
          const uint32_t tsfb = tsfa + 4;
          copy_scales_to_tmem(tsfa, make_scale_desc(sfa_addr));
          copy_scales_to_tmem(tsfb, make_scale_desc(sfb_addr));
          const uint64_t adesc = make_kmajor_sw128_desc(a_addr);
          const uint64_t bdesc = make_kmajor_sw128_desc(b_addr);
          const uint32_t d_tmem = tmem_base + acc * kBN;
#pragma unroll
          for (int k = 0; k < 4; ++k) {                       // K = 32 per instruction, scale byte k of the column
            const uint32_t idesc = args.idesc | ((uint32_t)k << 4) | ((uint32_t)k << 29);
            mma_block_scaled(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                             (kb > 0 || k > 0) ? 1u : 0u, tsfa, tsfb);
          }
          tc_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (lane == 0) tc_commit(&tmem_full[acc]);
      __syncwarp();
      if (++acc == kAcc) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quadrant = warp & 3;                            // the TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < args.num_tiles && ok; t += gridDim.x) {
      const int mt = t / args.n_tiles, nt = t - mt * args.n_tiles;
      ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_phase, abort_flag, args.status, kTimeoutTmemFull));
      if (!ok) break;
      tc_fence_after_sync();
      const long long row = (long long)mt * kBM + quadrant * 32 + lane;
#pragma unroll 1
      for (int chunk = 0; chunk < kBN / 32; ++chunk) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quadrant * 32) << 16) + acc * kBN + chunk * 32, v);
        tmem_ld_wait();
        const int col0 = nt * kBN + chunk * 32;
        if (row < args.M && col0 < args.N) {
          const int valid = min(32, args.N - col0);
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            f[j] = __uint_as_float(v[j]);
            if (args.bias != nullptr && j < valid) f[j] += load_as_float(args.bias, col0 + j, args.bias_dtype);
          }
          if (args.out_dtype == kF32) {
            float* dst = reinterpret_cast<float*>(args.out) + row * args.ldo + col0;
            const bool vec = valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
            if (vec) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
              for (int j = 0; j < valid; ++j) dst[j] = f[j];
            }
          } else {
            uint16_t* dst = reinterpret_cast<uint16_t*>(args.out) + row * args.ldo + col0;
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (args.out_dtype == kBF16) {
                __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                packed[j] = *reinterpret_cast<uint32_t*>(&h);
              } else {
                __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                packed[j] = *reinterpret_cast<uint32_t*>(&h);
              }
            }
            const bool vec = valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
            if (vec) {
#pragma unroll
              for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<uint4*>(dst + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
            } else {
              for (int j = 0; j < valid; ++j) dst[j] = (uint16_t)(packed[j >> 1] >> (16 * (j & 1)));
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == kAcc) { acc = 0; acc_phase ^= 1; }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
}

// scales: fp32 powers of two (or uint8 UE8M0 when `is_bytes`), one per (row >> row_shift, K group of 32);
// element (r, g) at scales[(r >> row_shift) * row_stride + g * group_stride].  Writes the tiled layout; rows and
// groups beyond the operand get 127 (= 1.0), their codes are zero.
__global__ void __launch_bounds__(256)
pack_scales_kernel(const void* __restrict__ scales, int is_bytes, long long row_stride, long long group_stride,
                   int rows, int groups, int row_shift, uint8_t* __restrict__ out, int row_tiles, int k_blocks) {
  const long long total = (long long)row_tiles * k_blocks * kSfBytes;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long chunk = i / kSfBytes;
    const int within = (int)(i - chunk * kSfBytes);
    const int rt = (int)(chunk / k_blocks), kb = (int)(chunk - (long long)rt * k_blocks);
    const int r = rt * 128 + ((within >> 2) & 3) * 32 + (within >> 4);
    const int g = kb * 4 + (within & 3);
    uint8_t byte = 127;
    if (r < rows && g < groups) {
      const long long at = (long long)(r >> row_shift) * row_stride + (long long)g * group_stride;
      byte = is_bytes ? reinterpret_cast<const uint8_t*>(scales)[at]
                      : (uint8_t)((__float_as_uint(reinterpret_cast<const float*>(scales)[at]) >> 23) & 0xffu);
    }
    out[i] = byte;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// [rows, K] bytes, K contiguous, row pitch ld bytes; box = 128 bytes of K x 128 rows, 128-byte swizzle, zero fill.
static int make_operand_map(CUtensorMap* map, const void* base, long long rows, long long k, long long ld) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld & 15) != 0) return (int)cudaErrorMisalignedAddress;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
  cuuint32_t element_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace mx
}  // namespace vb

using namespace vb;

extern "C" long long vb_mx_scale_bytes(long long rows, long long k) {
  return ((rows + 127) / 128) * ((k + 127) / 128) * mx::kSfBytes;
}

extern "C" int vb_mx_pack_scales(const void* scales, int is_bytes, long long row_stride, long long group_stride, int rows,
                                 int k, int row_shift, uint8_t* out, cudaStream_t stream) {
  if (rows <= 0 || k <= 0) return (int)cudaErrorInvalidValue;
  const int row_tiles = (rows + 127) / 128, k_blocks = (k + 127) / 128, groups = (k + 31) / 32;
  const long long total = (long long)row_tiles * k_blocks * mx::kSfBytes;
  const int grid = (int)std::min<long long>((total + 255) / 256, 1184);
  mx::pack_scales_kernel<<<grid, 256, 0, stream>>>(scales, is_bytes, row_stride, group_stride, rows, groups, row_shift, out,
                                                   row_tiles, k_blocks);
  return (int)cudaGetLastError();
}

extern "C" int vb_mx_gemm(const void* a, long long lda, int a_fmt, const void* b, long long ldb, int b_fmt,
                          const uint8_t* sfa_tiled, const uint8_t* sfb_tiled, int M, int N, int K, void* out, int out_dtype,
                          long long ldo, const void* bias, int bias_dtype, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || out_dtype < 0 || out_dtype > 2) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(sfa_tiled) & 15) != 0 || (reinterpret_cast<uintptr_t>(sfb_tiled) & 15) != 0)
    return (int)cudaErrorMisalignedAddress;
  CUtensorMap tmA, tmB;
  int rc = mx::make_operand_map(&tmA, a, M, K, lda);
  if (rc != 0) return rc;
  rc = mx::make_operand_map(&tmB, b, N, K, ldb);
  if (rc != 0) return rc;
  mx::Args args{};
  args.M = M; args.N = N; args.K = K;
  args.num_k_blocks = (K + mx::kBK - 1) / mx::kBK;
  args.m_tiles = (M + mx::kBM - 1) / mx::kBM;
  args.n_tiles = (N + mx::kBN - 1) / mx::kBN;
  args.num_tiles = args.m_tiles * args.n_tiles;
  args.sfa = sfa_tiled; args.sfb = sfb_tiled;
  args.out = out; args.out_dtype = out_dtype; args.ldo = ldo;
  args.bias = bias; args.bias_dtype = bias_dtype;
  // block-scaled instruction descriptor: formats, N >> 3, UE8M0 scales, M >> 4 (scale ids are added per instruction)
  args.idesc = ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(mx::kBN >> 3) << 17) | (1u << 23) |
               ((uint32_t)(mx::kBM >> 4) << 24);
  args.status = status;
  static std::once_flag once;
  static cudaError_t attr_rc = cudaSuccess;
  std::call_once(once, [] {
    attr_rc = cudaFuncSetAttribute(mx::mx_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mx::kSmemBytes);
  });
  if (attr_rc != cudaSuccess) return (int)attr_rc;
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int grid = std::min(args.num_tiles, sms > 0 ? sms : 148);
  mx::mx_gemm_kernel<<<grid, mx::kThreads, mx::kSmemBytes, stream>>>(tmA, tmB, args);
  return (int)cudaGetLastError();
}
