// Self-attention forward on tcgen05 for short sequences: one CTA per (sample, head), the whole 256 x 256 score
// matrix of a head lives in tensor memory, so the softmax needs no running maximum and no rescaling.
//
//   O[b, t, h, :] = softmax_over_keys(Q[b, t, h, :] . K[b, :, h, :]^T * scale) . V[b, :, h, :],    T = 256 tokens
//
// Input is the packed projection qkv [B, T, 3, H, D] (bf16 or fp16) exactly as the qkv GEMM writes it; output is
// [B, T, H, D] plus the log-sum-exp per row [B, H, T] (fp32, natural log of sum exp(score * scale)), the quantity a
// flash-attention backward needs.  The reference leaves attention to PyTorch SDPA (experiments/dit.py:36); this
// kernel is the Blackwell-native replacement for the DiT shapes (256 tokens, head size 72).
//
// Shared memory (1024-byte aligned): Q, K, V as [2 blocks of 64 columns][256 rows][128 B], written by TMA with
// SWIZZLE_128B from a 4-D tensor map (column, head, q/k/v, token) whose innermost extent is D, so columns D .. 127 of
// the second block arrive as zeros.  S_i = Q_i K^T (i = 0, 1: 128 queries each) are two 128 x 256 fp32 accumulators
// in tensor memory (512 columns).  Eight softmax warps (two per TMEM lane quadrant, each on 128 key columns) take the
// row maximum, exponentiate, write P_i as a bf16 K-major operand over the dead Q (P_0) and K (P_1) regions, and
// exchange row maxima and sums through shared memory.  O_i = P_i V reads V MN-major in place (16 MMAs of
// 128 x D' x 16, D' = D rounded up to 16) into the columns S_i occupied; the warps then scale by 1 / row sum and store.
// One thread issues every TMA load and MMA.  Every wait is bounded and reports through the status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "api.h"
#include "common/ptx.cuh"

namespace vb {
namespace attn {

constexpr int kTokens = 256;                       // sequence length this kernel is built for
constexpr int kOperandBytes = 2 * kTokens * 128;   // one of Q / K / V: two 64-column blocks of 256 rows x 128 B
constexpr int kBlockBytes = kTokens * 128;         // one 64-column block
constexpr int kThreads = 320;                      // warp 0 control, warp 1 TMEM owner, warps 2-9 softmax
constexpr int kTailBytes = 4096;                   // barriers, flags, row exchange
constexpr int kSmemBytes = 3 * kOperandBytes + kTailBytes + 1024;

struct Args {
  int batch, heads, head_dim;
  float scale_log2;          // softmax scale * log2(e)
  float scale;
  void* out;                 // [B, T, H, D]
  float* lse;                // [B, H, T]
  int dtype;                 // 1 bf16, 2 fp16
  uint32_t idesc_s, idesc_o;
  int* status;
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack16(float a, float b, int dtype) {
  if (dtype == 1) {
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
  }
  __half2 t = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ void softmax_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1)
attention_forward_kernel(const __grid_constant__ CUtensorMap tm_qkv, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* k_smem = smem + kOperandBytes;
  uint8_t* v_smem = smem + 2 * kOperandBytes;
  uint8_t* tail = smem + 3 * kOperandBytes;
  uint64_t* bar_qk = reinterpret_cast<uint64_t*>(tail);           // Q and K landed
  uint64_t* bar_v = bar_qk + 1;                                   // V landed
  uint64_t* s_full = bar_qk + 2;                                  // [2] S_i complete in tensor memory
  uint64_t* p_ready = bar_qk + 4;                                 // [2] P_i written to shared memory
  uint64_t* o_full = bar_qk + 6;                                  // [2] O_i complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_qk + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* row_max = reinterpret_cast<float*>(tail + 1024);         // [2 halves][128 rows]
  float* row_sum = row_max + 256;                                 // [2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / args.heads, h = blockIdx.x - b * args.heads;
  const int blocks = (args.head_dim + 63) / 64;                   // 64-column blocks per operand that hold data
  const int k_steps = (args.head_dim + 15) / 16;                  // MMA K steps of the score product

  if (threadIdx.x == 0) {
    mbar_init(bar_qk, 1);
    mbar_init(bar_v, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 8);
      mbar_init(&o_full[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // -------------------------- control: loads and MMAs from one thread --------------------------
    if (lane == 0) {
      const int row0 = b * kTokens;
      mbar_expect_tx(bar_qk, 2 * blocks * kBlockBytes);
      for (int blk = 0; blk < blocks; ++blk) {
        tma_load_4d(q_smem + blk * kBlockBytes, &tm_qkv, bar_qk, blk * 64, h, 0, row0);
        tma_load_4d(k_smem + blk * kBlockBytes, &tm_qkv, bar_qk, blk * 64, h, 1, row0);
      }
      mbar_expect_tx(bar_v, blocks * kBlockBytes);
      for (int blk = 0; blk < blocks; ++blk)
        tma_load_4d(v_smem + blk * kBlockBytes, &tm_qkv, bar_v, blk * 64, h, 2, row0);
      bool ok = mbar_wait(bar_qk, 0, abort_flag, args.status, kTimeoutFull);
      if (ok) {
        tc_fence_after_sync();
        for (int i = 0; i < 2; ++i) {
          for (int ks = 0; ks < k_steps; ++ks) {
            const uint32_t offset = (uint32_t)(ks >> 2) * kBlockBytes + (uint32_t)(ks & 3) * 32;
            const uint64_t adesc = make_kmajor_sw128_desc(smem_u32(q_smem) + i * 128 * 128 + offset);
            const uint64_t bdesc = make_kmajor_sw128_desc(smem_u32(k_smem) + offset);
            mma_f16_ss(tmem_base + i * 256, adesc, bdesc, args.idesc_s, ks > 0);
          }
          tc_commit(&s_full[i]);
        }
        ok = mbar_wait(bar_v, 0, abort_flag, args.status, kTimeoutFull);
      }
      for (int i = 0; i < 2 && ok; ++i) {
        ok = mbar_wait(&p_ready[i], 0, abort_flag, args.status, kTimeoutEmpty);
        if (!ok) break;
        tc_fence_after_sync();
        uint8_t* p_smem = i == 0 ? q_smem : k_smem;                // P_i lies over the dead operand
        for (int kk = 0; kk < kTokens / 16; ++kk) {
          // A = P_i: K-major, four 64-key blocks of 128 rows; B = V: MN-major, 16 key rows per step
          const uint64_t adesc = make_kmajor_sw128_desc(smem_u32(p_smem) + (uint32_t)(kk >> 2) * (128 * 128) +
                                                        (uint32_t)(kk & 3) * 32);
          const uint64_t bdesc = make_mnmajor_sw128_desc(smem_u32(v_smem) + (uint32_t)kk * 16 * 128, kBlockBytes);
          mma_f16_ss(tmem_base + i * 256, adesc, bdesc, args.idesc_o, kk > 0);
        }
        tc_commit(&o_full[i]);
      }
    }
    __syncwarp();
  } else if (warp >= 2) {
    // -------------------------- softmax and output --------------------------
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;                               // row of the 128-query tile
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    float tile_max[2], tile_sum[2];
    bool ok = true;
    for (int i = 0; i < 2 && ok; ++i) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[i], 0, abort_flag, args.status, kTimeoutTmemFull));
      // P_0 is written over Q, which the score MMAs of the second tile still read until s_full[1]
      if (ok && i == 0) ok = __all_sync(0xffffffffu, mbar_wait(&s_full[1], 0, abort_flag, args.status, kTimeoutTmemFull));
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t s_addr = tmem_base + lane_addr + i * 256 + half * 128;
      float m = -INFINITY;
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) m = fmaxf(m, __uint_as_float(r[j]));
      }
      row_max[half * 128 + row] = m;
      softmax_barrier();
      m = fmaxf(row_max[row], row_max[128 + row]);
      const float shift = m * args.scale_log2;
      float l = 0.f;
      uint8_t* p_smem = i == 0 ? q_smem : k_smem;
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float p0 = exp2_approx(fmaf(__uint_as_float(r[2 * j]), args.scale_log2, -shift));
          const float p1 = exp2_approx(fmaf(__uint_as_float(r[2 * j + 1]), args.scale_log2, -shift));
          l += p0 + p1;
          packed[j] = pack16(p0, p1, args.dtype);
        }
        // keys half * 128 + c * 32 .. + 31 of this row: 64-key block (half * 2 + c / 2), 16-byte pieces (c % 2) * 4 ..
        uint8_t* block_row = p_smem + (half * 2 + (c >> 1)) * (128 * 128) + row * 128;
#pragma unroll
        for (int p = 0; p < 4; ++p)
          *reinterpret_cast<uint4*>(block_row + ((((c & 1) * 4 + p) ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * p], packed[4 * p + 1], packed[4 * p + 2], packed[4 * p + 3]);
      }
      row_sum[half * 128 + row] = l;
      fence_proxy_async_smem();                                     // P_i is read by the tensor core (async proxy)
      tc_fence_before_sync();
      softmax_barrier();
      if (lane == 0) mbar_arrive(&p_ready[i]);
      tile_max[i] = m;
      tile_sum[i] = row_sum[row] + row_sum[128 + row];
      softmax_barrier();                                            // row_max / row_sum are reused by the next tile
    }
    // O_i: the warps of half i finish tile i
    if (ok) {
      const int i = half;
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[i], 0, abort_flag, args.status, kTimeoutTmemFull));
      if (ok) {
        tc_fence_after_sync();
        const float inv = 1.f / tile_sum[i];
        const long long token = (long long)b * kTokens + i * 128 + row;
        uint8_t* out_row = reinterpret_cast<uint8_t*>(args.out) + ((token * args.heads + h) * args.head_dim) * 2;
        const int pieces = args.head_dim / 8;                       // 16-byte pieces of the output row
        for (int c = 0; c * 32 < args.head_dim; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + lane_addr + i * 256 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            if (c * 4 + p < pieces) {
              uint4 t;
              t.x = pack16(__uint_as_float(r[8 * p + 0]) * inv, __uint_as_float(r[8 * p + 1]) * inv, args.dtype);
              t.y = pack16(__uint_as_float(r[8 * p + 2]) * inv, __uint_as_float(r[8 * p + 3]) * inv, args.dtype);
              t.z = pack16(__uint_as_float(r[8 * p + 4]) * inv, __uint_as_float(r[8 * p + 5]) * inv, args.dtype);
              t.w = pack16(__uint_as_float(r[8 * p + 6]) * inv, __uint_as_float(r[8 * p + 7]) * inv, args.dtype);
              *reinterpret_cast<uint4*>(out_row + (c * 4 + p) * 16) = t;
            }
          }
        }
        if (args.lse != nullptr)
          args.lse[((long long)b * args.heads + h) * kTokens + i * 128 + row] = tile_max[i] * args.scale + __logf(tile_sum[i]);
      }
    }
  }

  // teardown: on the error path give copies in flight a bounded grace period before the shared memory goes away
  if (*abort_flag) {
    const long long start = clock64();
    while (clock64() - start < 2000000LL) { __nanosleep(256); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

}  // namespace attn
}  // namespace vb

using namespace vb;

// qkv: [batch, 256, 3, heads, head_dim] contiguous, 16-bit; out: [batch, 256, heads, head_dim]; lse: [batch, heads, 256]
extern "C" int vb_attention_forward(const void* qkv, int dtype, int batch, int tokens, int heads, int head_dim, float scale,
                                    void* out, float* lse, int* status, cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (tokens != attn::kTokens || head_dim % 8 != 0 || head_dim < 16 || head_dim > 128 || heads <= 0 || (dtype != 1 && dtype != 2) ||
      (reinterpret_cast<uintptr_t>(qkv) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return (int)cudaErrorInvalidValue;
  attn::EncodeTiledFn encode = attn::encode_fn();
  if (encode == nullptr) return (int)cudaErrorNotSupported;
  CUtensorMap map;
  const cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)heads, 3, (cuuint64_t)batch * tokens};
  const cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)heads * head_dim * 2, (cuuint64_t)3 * heads * head_dim * 2};
  const cuuint32_t box[4] = {64, 1, 1, (cuuint32_t)attn::kTokens};
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  if (encode(&map, dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(qkv),
             dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return (int)cudaErrorInvalidValue;
  attn::Args args{};
  args.batch = batch; args.heads = heads; args.head_dim = head_dim;
  args.scale = scale;
  args.scale_log2 = scale * 1.4426950408889634f;
  args.out = out; args.lse = lse; args.dtype = dtype;
  const int fmt = dtype == 1 ? 1 : 0;
  args.idesc_s = make_idesc(fmt, fmt, 128, 256, 0, 0);
  args.idesc_o = make_idesc(fmt, fmt, 128, (head_dim + 15) / 16 * 16, 0, 1);
  args.status = status;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn::attention_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  attn::attention_forward_kernel<<<batch * heads, attn::kThreads, attn::kSmemBytes, stream>>>(map, args);
  return (int)cudaGetLastError();
}
