// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, never
// cluster-multicast), tcgen05 (TMEM alloc / mma / commit / ld) and the bounded-wait
// convention used by every kernel in this library.
//
// Bounded waits: no spin in this library is unbounded.  A wait that exceeds its
// budget records a code in a global status word, raises a CTA-wide abort flag in
// shared memory and returns false; every role then falls through to the common
// teardown (TMEM is freed, the kernel returns) and the host raises after the
// stream synchronises.  Nothing traps and nothing loops forever.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace vb {

// ---------------------------------------------------------------------------------
// status word layout (one int[8] per library call site, zeroed by the host)
// [0] = first error code (0 = ok), [1] = blockIdx.x, [2] = role/warp, [3] = detail
// ---------------------------------------------------------------------------------
enum StatusCode : int {
  kOk = 0,
  kTimeoutFull = 1,       // consumer waited for TMA data
  kTimeoutEmpty = 2,      // producer waited for a free smem stage
  kTimeoutTmemFull = 3,   // epilogue waited for the MMA commit
  kTimeoutTmemEmpty = 4,  // MMA waited for the epilogue to drain TMEM
  kTimeoutPeerFlag = 5,   // waited on a flag another GPU writes
  kTimeoutPanel = 6,      // waited on a gathered weight panel
  kBadArgument = 7,
  kTimeoutSplit = 8,      // a split-K unit waited for the unit before it on the same tile
};

__device__ __forceinline__ void report(int* status, int code, int detail) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = (int)blockIdx.x;
    status[2] = (int)(threadIdx.x >> 5);
    status[3] = detail;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 R;\n\t"
      "elect.sync R|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wait budget in SM clocks (~1.3-1.9 GHz): about a quarter of a second.  Every
// kernel here finishes in milliseconds, so an expiry means a protocol error.
constexpr long long kWaitBudgetClocks = 400000000LL;

// Bounded wait.  `abort_flag` is a CTA-shared int: once any role gives up the
// others stop waiting at their next poll instead of burning their own budget.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 63u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - start > kWaitBudgetClocks) {
        *abort_flag = 1;
        report(status, code, (int)parity);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// TMA (tiled, 2-D / 3-D), always CTA-local destinations, never multicast
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x),
        "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x),
        "r"(y), "r"(z)
      : "memory");
}

// TMA store: shared (this CTA) -> global through a tensor map; completion is tracked per thread in
// bulk async-groups.  The x coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
// TMA reduce: the shared-memory tile is ADDED to global memory (element type of the tensor map; fp32 here)
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until at most N of this thread's committed groups still READ their shared-memory source
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}
// CTA-pair forms: one warp of EACH CTA of the pair executes them
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on `bar` when every tcgen05.mma issued so far by this thread retires.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc];  kind::f16 covers bf16/fp16 inputs.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      :
      : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f8f6f4 covers every e4m3/e5m2 operand combination (formats live in idesc).
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
      :
      : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------------------------
// CTA pairs (cluster of two, tcgen05 cta_group::2): one 256-row MMA spans both CTAs' shared and tensor memory
// ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
// all threads of both CTAs: arrive, then wait (also a CTA-wide barrier)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Arrives once on the barrier at `cluster_addr` (this CTA's or the peer's) when every tcgen05.mma issued so far by
// this thread has retired in both CTAs.
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      :
      : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f8_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
      :
      : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// TMA load into this CTA's shared memory whose completion bytes are counted on a barrier of either CTA of the
// pair (given as a shared::cluster address): both CTAs feed the leader's "stage full" barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i receives lane (base_lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand tile whose rows are exactly
// one 128-byte swizzle span (TMA SWIZZLE_128B, rows packed at a 128 B pitch, 8-row
// groups 1024 B apart).  Bits: [0,14) addr>>4, [16,30) LBO>>4 (ignored for swizzled
// K-major, set to 1), [32,46) SBO>>4 = 64, [46,48) version = 1, [61,64) layout = 2.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Descriptor for an MN-major operand tile (the MN dimension is contiguous in memory): the tile is a
// sequence of blocks of 128 bytes of MN x (K rows), each loaded by one TMA box with SWIZZLE_128B
// (K-row pitch 128 B, 8-row swizzle groups 1024 B apart = SBO); LBO is the distance between
// consecutive MN blocks.  One MMA K-step advances the start address by (K rows per MMA) x 128 B.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((block_bytes >> 4) & 0x3FFFu) << 16;   // leading byte offset: next 128-byte MN block
  d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset: next group of 8 K rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16 / kind::f8f6f4 with an fp32 accumulator.
// a_fmt/b_fmt: f16 kind -> 0 = fp16, 1 = bf16;  f8f6f4 kind -> 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t make_idesc(int a_fmt, int b_fmt, int m, int n,
                                                  int a_mn_major = 0, int b_mn_major = 0) {
  return (1u << 4)                        // c_format = f32
         | ((uint32_t)a_fmt << 7)         // a_format
         | ((uint32_t)b_fmt << 10)        // b_format
         | ((uint32_t)a_mn_major << 15)   // a_major
         | ((uint32_t)b_mn_major << 16)   // b_major
         | ((uint32_t)(n >> 3) << 17)     // n_dim
         | ((uint32_t)(m >> 4) << 24);    // m_dim
}

// ---------------------------------------------------------------------------------
// Peer-memory access for the fused communication kernels
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(int* ptr, int value) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(ptr), "r"(value) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* ptr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* ptr) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
// Flags between CTAs of one launch (split-K hand-over): gpu scope is enough.
__device__ __forceinline__ void st_release_gpu(int* ptr, int value) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(ptr), "r"(value) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* ptr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
// orders this thread's generic-proxy accesses with its async-proxy (TMA) accesses to global memory
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
// Bounded wait until *flag == expected, written by another CTA of the same (fully resident) launch.
__device__ __forceinline__ bool wait_flag_eq_gpu(const int* flag, int expected, volatile int* abort_flag, int* status,
                                                 int code) {
  const long long start = clock64();
  uint32_t polls = 0;
  while (true) {
    const int seen = ld_acquire_gpu(flag);
    if (seen == expected) return true;
    if ((++polls & 31u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - start > kWaitBudgetClocks) {
        *abort_flag = 1;
        report(status, code, seen);
        return false;
      }
      __nanosleep(64);
    }
  }
}
// Bounded wait until *flag >= expected (flags only ever grow: generation counters).
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int expected, int* status, int code) {
  const long long start = clock64();
  uint32_t polls = 0;
  while (true) {
    int seen = ld_acquire_sys(flag);
    if (seen >= expected) return true;
    if ((++polls & 31u) == 0) {
      if (clock64() - start > kWaitBudgetClocks) {
        report(status, code, seen);
        return false;
      }
      __nanosleep(64);
    }
  }
}

}  // namespace vb
