// Fused compute + collective kernels over NVLink peer memory (sm_100a).
//
// Every rank maps every other rank's symmetric heap (same layout on all ranks), so a kernel can
// store into / load from a peer with plain st / ld (P2P through NVSwitch).  There is no NCCL call
// and no staging packet on these paths; signalling uses int32 generation counters in the peers'
// heaps written with st.release.sys after __threadfence_system() and read with ld.acquire.sys.
// No TMA is used here at all (and in particular no cluster-multicast load of peer memory).
//
//   path 1  reduce-to-owner      vb_reduce_push_fp8 (all non-owners) + vb_reduce_accumulate_fp8 (owner)
//           = quantise (fp32 -> e4m3/e5m2 codes + fp32 tile scale) fused with the push, and
//             dequantise + ascending-rank fp32 sum + "+=" into the gradient accumulator fused with
//             the receive.  Replaces pack -> gather -> unpack-reduce -> add
//             (viola/distributed/fp8.py:67-85, _fp8_kernels.py:18-69, gradients.py:101-125).
//   path 2  all-reduce with requantisation   vb_allreduce_push / _reduce / _unpack
//           (viola/distributed/fp8.py:48-65): reduce-scatter by push, second quantisation fused
//           with the all-gather push, dequantise.
//   path 3  parameter gather     vb_gather_pull: one kernel pulls every peer's row slab of every
//           parameter of a unit into the local full buffers (local slab first) and raises one flag
//           per (parameter, source rank).  The consuming GEMMs are ordered after it by a stream
//           event, not by polling those flags: a kernel that spins on a flag which a separate
//           launch on the same GPU has to write is not guaranteed to ever see that launch run.
//           The host starts the gather of the next sharding unit on a side stream while the
//           current unit computes, which hides it (viola/distributed/fsdp.py:67 gathers in line).
//   path 4  owner write-back     vb_multi_writeback: every master an owner holds, in two launches over a
//           device table: EMA lerp + per-tensor amax, then scale + FP8 encode (or cast) + 16-byte
//           stores into the row slab of whichever rank holds those rows + the layer header (scale,
//           amax history slot) into every rank.  vb_quantize_push / vb_byte_push are the
//           single-tensor forms; vb_signal / vb_wait_flags build the on-stream barriers.
//
// Waits on flags another GPU writes are bounded (``wait_clocks``); on expiry the kernel records
// kTimeoutPeerFlag in the status word and returns without touching the data.
#include "api.h"
#include "common/codec.cuh"
#include "common/ptx.cuh"

namespace vb {

struct Peers {
  uint8_t* heap[16];
  int world, rank;
};

__device__ __forceinline__ bool wait_flag_budget(const int* flag, int expected, long long budget, int* status) {
  const long long start = clock64();
  uint32_t polls = 0;
  while (true) {
    const int seen = ld_acquire_sys(flag);
    if (seen >= expected) return true;
    if ((++polls & 15u) == 0) {
      if (clock64() - start > budget) {
        report(status, kTimeoutPeerFlag, seen);
        return false;
      }
      __nanosleep(128);
    }
  }
}

// One resident warp that sleeps between polls: the stand-alone wait launched in front of a kernel whose every
// block would otherwise sit on an SM polling (a polling warp shares an issue port with the tensor-core
// kernels' epilogue warps and slowed them by up to 1.8x).  expected = *generation + delta; values < 1 mean
// "nothing to wait for yet".
__global__ void wait_generation_kernel(const int* flags, int count, int skip, const int* generation_ptr, int delta,
                                       long long budget, int* status) {
  if (threadIdx.x != 0) return;
  const int expected = *generation_ptr + delta;
  if (expected < 1) return;
  const long long start = clock64();
  for (int r = 0; r < count; ++r) {
    if (r == skip) continue;
    uint32_t polls = 0;
    while (true) {
      const int seen = ld_acquire_sys(flags + r);
      if (seen >= expected) break;
      __nanosleep(400);
      if ((++polls & 15u) == 0 && clock64() - start > budget) {
        report(status, kTimeoutPeerFlag, seen);
        return;
      }
    }
  }
}

// Block-wide: thread 0 waits on up to `count` flags (skipping index `skip`), everyone learns the result.
__device__ __forceinline__ bool block_wait_flags(const int* flags, int count, int skip, int expected, long long budget,
                                                 int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    int good = 1;
    for (int r = 0; r < count && good; ++r)
      if (r != skip) good = wait_flag_budget(flags + r, expected, budget, status) ? 1 : 0;
    ok = good;
  }
  __syncthreads();
  return ok != 0;
}

// Last block to arrive (after every thread fenced its peer stores) gets `true`; the counter resets itself.
// The counter word carries the number of arrived blocks in its low 24 bits and a "some block gave up"
// mark in bit 31: every block takes a ticket whether or not its wait succeeded, so one timed-out launch
// leaves the counter at zero for the next one, and the last block returns false when any block failed
// (the caller then publishes nothing).
__device__ __forceinline__ bool last_block_done(unsigned int* counter, bool ok = true) {
  __shared__ bool last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(counter, ok ? 1u : (1u | 0x80000000u));
    const bool failed = !ok || (ticket & 0x80000000u) != 0u;
    last = (ticket & 0x00ffffffu) == gridDim.x - 1;
    if (last) {
      *counter = 0u;
      __threadfence_system();
      last = !failed;
    }
  }
  __syncthreads();
  return last;
}

// ------------------------------------------------------------------------------------------
// path 1
// ------------------------------------------------------------------------------------------
template <int TILE>
__global__ void __launch_bounds__(256)
reduce_push_kernel(const float* __restrict__ bucket, long long n, int fmt, uint8_t* dst_codes, float* dst_scales,
                   int* dst_flag, const int* ack_flag, const int* generation_ptr, unsigned int* counter, long long budget,
                   int* status) {
  // The generation (= microbatch counter) lives in device memory so that a captured CUDA graph
  // signals a fresh value on every replay.
  const int generation = *generation_ptr;
  // The owner must have consumed the previous generation of this slot before it is overwritten.
  // A block whose wait ran out skips its share of the data but still takes its ticket below, so the
  // self-resetting counter ends at zero; the flag is then not raised (the failure is in the status word).
  const bool ready = generation <= 1 || block_wait_flags(ack_flag, 1, -1, generation - 1, budget, status);
  const long long tiles = (n + TILE - 1) / TILE;
  const int lane = threadIdx.x & 31;
  if (ready)
    for (long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); t < tiles; t += (long long)gridDim.x * 8)
      pack_tile<TILE>(bucket, t * TILE, n, fmt, dst_codes + t * TILE, dst_scales + t, lane);
  if (last_block_done(counter, ready) && threadIdx.x == 0) st_release_sys(dst_flag, generation);
}

// Quantise-dequantise of the owner's own contribution with exactly the codec's arithmetic.
template <int TILE>
__device__ __forceinline__ void fake_quantize_tile(float (&v)[TILE / 32], int fmt) {
  float m = 0.f;
#pragma unroll
  for (int e = 0; e < TILE / 32; ++e) m = fmaxf(m, abs_nan_to_inf(v[e]));
  m = warp_max(m);
  const float scale = fmaxf(m, 1e-30f) / fp8_max(fmt);
#pragma unroll
  for (int e = 0; e < TILE / 32; ++e) v[e] = fp8_decode(fp8_encode(v[e] / scale, fmt), fmt) * scale;
}

template <int TILE>
__global__ void __launch_bounds__(256)
reduce_accumulate_kernel(const float* __restrict__ bucket, long long n, int fmt, const uint8_t* recv, long long slot_stride,
                         long long scales_offset, const int* flags, Peers peers, long long ack_offset,
                         const int* generation_ptr, float* __restrict__ accum, unsigned int* counter, long long budget,
                         int* status) {
  const int generation = *generation_ptr;
  const bool ready = block_wait_flags(flags, peers.world, peers.rank, generation, budget, status);
  const long long tiles = (n + TILE - 1) / TILE;
  const int lane = threadIdx.x & 31;
  for (long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); ready && t < tiles; t += (long long)gridDim.x * 8) {
    float own[TILE / 32], result[TILE / 32];
    load_tile<TILE>(bucket, t * TILE, n, lane, own);
    fake_quantize_tile<TILE>(own, fmt);
#pragma unroll
    for (int e = 0; e < TILE / 32; ++e) result[e] = 0.f;
    for (int r = 0; r < peers.world; ++r) {   // ascending source rank, fp32
      if (r == peers.rank) {
#pragma unroll
        for (int e = 0; e < TILE / 32; ++e) result[e] += own[e];
      } else {
        const uint8_t* slot = recv + (long long)r * slot_stride;
        const float scale = reinterpret_cast<const float*>(slot + scales_offset)[t];
        accumulate_tile<TILE>(slot + t * TILE, scale, fmt, lane, result);
      }
    }
    store_tile<TILE>(accum, t * TILE, n, lane, result, true);
  }
  if (last_block_done(counter, ready) && threadIdx.x < peers.world && (int)threadIdx.x != peers.rank)
    st_release_sys(reinterpret_cast<int*>(peers.heap[threadIdx.x] + ack_offset), generation);
}

// Path 1 over a table of buckets: one launch pushes every bucket this rank does not own, one launch accumulates
// every bucket it owns.  Used when gradients are reduced once per optimizer step from a rank-local sum: the
// rendezvous cost (flag round trips, fences, launches) is then paid twice per step instead of twice per bucket.
struct ReduceDesc {            // 64 bytes per bucket
  const float* src;            // this rank's fp32 values of the bucket
  long long n;                 // elements
  uint8_t* codes;              // push: this rank's slot in the owner's heap; accumulate: slot of source rank 0 (local)
  float* scales;               // push: scales of that slot; accumulate: unused
  float* accum;                // accumulate: the owner's fp32 accumulator slice
  long long slot_stride;       // accumulate: bytes between the slots of consecutive source ranks
  long long scales_offset;     // accumulate: byte offset of the scales inside a slot
  long long reserved;
};

// bucket of global tile t: largest b with prefix[b] <= t (prefix[0] = 0, prefix[buckets] = total tiles)
__device__ __forceinline__ int bucket_of_tile(const long long* __restrict__ prefix, int buckets, long long t) {
  int lo = 0, hi = buckets - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <int TILE>
__global__ void __launch_bounds__(256)
reduce_push_many_kernel(const ReduceDesc* __restrict__ table, const long long* __restrict__ prefix, int buckets, int fmt,
                        Peers peers, long long flag_offset, const int* ack_flags, const int* generation_ptr,
                        unsigned int* counter, long long budget, int* status) {
  const int generation = *generation_ptr;
  // every owner must have consumed the previous generation of its slots before they are overwritten
  const bool ready = generation <= 1 || block_wait_flags(ack_flags, peers.world, peers.rank, generation - 1, budget, status);
  const long long tiles = prefix[buckets];
  const int lane = threadIdx.x & 31;
  if (ready)
    for (long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); t < tiles; t += (long long)gridDim.x * 8) {
      const int b = bucket_of_tile(prefix, buckets, t);
      const ReduceDesc d = table[b];
      const long long local = t - prefix[b];
      pack_tile<TILE>(d.src, local * TILE, d.n, fmt, d.codes + local * TILE, d.scales + local, lane);
    }
  if (last_block_done(counter, ready) && threadIdx.x < peers.world && (int)threadIdx.x != peers.rank)
    st_release_sys(reinterpret_cast<int*>(peers.heap[threadIdx.x] + flag_offset) + peers.rank, generation);
}

template <int TILE>
__global__ void __launch_bounds__(256)
reduce_accumulate_many_kernel(const ReduceDesc* __restrict__ table, const long long* __restrict__ prefix, int buckets,
                              int fmt, Peers peers, const int* flags, long long ack_offset, const int* generation_ptr,
                              unsigned int* counter, long long budget, int* status) {
  const int generation = *generation_ptr;
  const bool ready = block_wait_flags(flags, peers.world, peers.rank, generation, budget, status);
  const long long tiles = prefix[buckets];
  const int lane = threadIdx.x & 31;
  for (long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); ready && t < tiles; t += (long long)gridDim.x * 8) {
    const int b = bucket_of_tile(prefix, buckets, t);
    const ReduceDesc d = table[b];
    const long long local = t - prefix[b];
    float own[TILE / 32], result[TILE / 32];
    load_tile<TILE>(d.src, local * TILE, d.n, lane, own);
    fake_quantize_tile<TILE>(own, fmt);
#pragma unroll
    for (int e = 0; e < TILE / 32; ++e) result[e] = 0.f;
    for (int r = 0; r < peers.world; ++r) {   // ascending source rank, fp32
      if (r == peers.rank) {
#pragma unroll
        for (int e = 0; e < TILE / 32; ++e) result[e] += own[e];
      } else {
        const uint8_t* slot = d.codes + (long long)r * d.slot_stride;
        const float scale = reinterpret_cast<const float*>(slot + d.scales_offset)[local];
        accumulate_tile<TILE>(slot + local * TILE, scale, fmt, lane, result);
      }
    }
    store_tile<TILE>(d.accum, local * TILE, d.n, lane, result, true);
  }
  if (last_block_done(counter, ready) && threadIdx.x < peers.world && (int)threadIdx.x != peers.rank)
    st_release_sys(reinterpret_cast<int*>(peers.heap[threadIdx.x] + ack_offset) + peers.rank, generation);
}

// ------------------------------------------------------------------------------------------
// path 2
// ------------------------------------------------------------------------------------------
// value: n floats; chunk j = [j * width, (j + 1) * width), width = groups * TILE.  Rank j reduces chunk j.
// a2a region  (on every rank): world slots of `slot` bytes: [codes width][scales groups]; slot src holds src's chunk.
// gather region (on every rank): world slots of `slot` bytes: slot r holds rank r's re-quantised partial sum.
template <int TILE>
__global__ void __launch_bounds__(256)
allreduce_push_kernel(const float* __restrict__ value, long long n, int groups, int fmt, Peers peers, long long a2a_offset,
                      long long slot, long long flag_offset, int generation, unsigned int* counter) {
  const long long width = (long long)groups * TILE;
  const long long total = (long long)peers.world * groups;
  const int lane = threadIdx.x & 31;
  for (long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); t < total; t += (long long)gridDim.x * 8) {
    const int dst = (int)(t / groups), g = (int)(t % groups);
    if (dst == peers.rank) continue;
    uint8_t* base = peers.heap[dst] + a2a_offset + (long long)peers.rank * slot;
    pack_tile<TILE>(value, dst * width + (long long)g * TILE, n, fmt, base + (long long)g * TILE,
                    reinterpret_cast<float*>(base + width) + g, lane);
  }
  if (last_block_done(counter) && threadIdx.x < peers.world && (int)threadIdx.x != peers.rank)
    st_release_sys(reinterpret_cast<int*>(peers.heap[threadIdx.x] + flag_offset) + peers.rank, generation);
}

template <int TILE>
__global__ void __launch_bounds__(256)
allreduce_reduce_kernel(const float* __restrict__ value, long long n, int groups, int fmt, Peers peers, long long a2a_offset,
                        long long gather_offset, long long slot, long long a2a_flag_offset, long long gather_flag_offset,
                        int generation, unsigned int* counter, long long budget, int* status) {
  const int* flags = reinterpret_cast<const int*>(peers.heap[peers.rank] + a2a_flag_offset);
  const bool ready = block_wait_flags(flags, peers.world, peers.rank, generation, budget, status);
  const long long width = (long long)groups * TILE;
  const int lane = threadIdx.x & 31;
  const uint8_t* recv = peers.heap[peers.rank] + a2a_offset;
  for (long long g = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); ready && g < groups; g += (long long)gridDim.x * 8) {
    float own[TILE / 32], partial[TILE / 32];
    load_tile<TILE>(value, peers.rank * width + g * TILE, n, lane, own);
    fake_quantize_tile<TILE>(own, fmt);
#pragma unroll
    for (int e = 0; e < TILE / 32; ++e) partial[e] = 0.f;
    for (int r = 0; r < peers.world; ++r) {
      if (r == peers.rank) {
#pragma unroll
        for (int e = 0; e < TILE / 32; ++e) partial[e] += own[e];
      } else {
        const uint8_t* s = recv + (long long)r * slot;
        accumulate_tile<TILE>(s + g * TILE, reinterpret_cast<const float*>(s + width)[g], fmt, lane, partial);
      }
    }
    // second quantisation, written once per destination rank (including this one)
    float m = 0.f;
#pragma unroll
    for (int e = 0; e < TILE / 32; ++e) m = fmaxf(m, abs_nan_to_inf(partial[e]));
    m = warp_max(m);
    const float scale = fmaxf(m, 1e-30f) / fp8_max(fmt);
    using S = TileShape<TILE>;
    uint32_t words[S::IT];
#pragma unroll
    for (int it = 0; it < S::IT; ++it) {
      words[it] = 0;
#pragma unroll
      for (int e = 0; e < S::V; ++e) words[it] |= (uint32_t)fp8_encode(partial[it * S::V + e] / scale, fmt) << (8 * e);
    }
    for (int d = 0; d < peers.world; ++d) {
      uint8_t* base = peers.heap[d] + gather_offset + (long long)peers.rank * slot;
#pragma unroll
      for (int it = 0; it < S::IT; ++it) {
        uint8_t* dst = base + g * TILE + it * 32 * S::V + lane * S::V;
        if constexpr (S::V == 4) *reinterpret_cast<uint32_t*>(dst) = words[it];
        else if constexpr (S::V == 2) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)words[it];
        else *dst = (uint8_t)words[it];
      }
      if (lane == 0) reinterpret_cast<float*>(base + width)[g] = scale;
    }
  }
  if (last_block_done(counter, ready) && threadIdx.x < peers.world)
    st_release_sys(reinterpret_cast<int*>(peers.heap[threadIdx.x] + gather_flag_offset) + peers.rank, generation);
}

template <int TILE>
__global__ void __launch_bounds__(256)
allreduce_unpack_kernel(float* __restrict__ value, long long n, int groups, int fmt, Peers peers, long long gather_offset,
                        long long slot, long long gather_flag_offset, int generation, long long budget, int* status) {
  const int* flags = reinterpret_cast<const int*>(peers.heap[peers.rank] + gather_flag_offset);
  if (!block_wait_flags(flags, peers.world, -1, generation, budget, status)) return;
  const long long width = (long long)groups * TILE;
  const long long total = (long long)peers.world * groups;
  const int lane = threadIdx.x & 31;
  const uint8_t* recv = peers.heap[peers.rank] + gather_offset;
  for (long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); t < total; t += (long long)gridDim.x * 8) {
    const int r = (int)(t / groups), g = (int)(t % groups);
    const uint8_t* s = recv + (long long)r * slot;
    float result[TILE / 32];
#pragma unroll
    for (int e = 0; e < TILE / 32; ++e) result[e] = 0.f;
    accumulate_tile<TILE>(s + (long long)g * TILE, reinterpret_cast<const float*>(s + width)[g], fmt, lane, result);
    store_tile<TILE>(value, r * width + (long long)g * TILE, n, lane, result, false);
  }
}

// ------------------------------------------------------------------------------------------
// path 4
// ------------------------------------------------------------------------------------------
// master (fp32 / bf16 / fp16) -> optional EMA lerp -> FP8 codes with a per-tensor scale, stored into
// every rank (shard_rows == 0: full copy at dst_offset) or into the rank owning each row slab.
__global__ void __launch_bounds__(256)
quantize_push_kernel(const void* __restrict__ master, int mdt, long long rows, long long cols, const float* __restrict__ scale_ptr,
                     float limit, int fmt, void* __restrict__ ema, int edt, float decay, Peers peers, long long dst_offset,
                     long long shard_rows) {
  const long long n = rows * cols;
  const float scale = scale_ptr[0];
  for (long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i4 < n; i4 += (long long)gridDim.x * blockDim.x * 4) {
    uint32_t word = 0;
    const int count = (int)min(4LL, n - i4);
    for (int e = 0; e < count; ++e) {
      const float v = load_as_float(master, i4 + e, mdt);
      if (ema != nullptr) store_from_float(ema, i4 + e, edt, fmaf(1.f - decay, v, load_as_float(ema, i4 + e, edt) * decay));
      word |= (uint32_t)fp8_encode(scaled_clamp(v, scale, limit), fmt) << (8 * e);
    }
    // cols % 4 == 0 is required by the launcher, so the 4 codes share a row and a destination slab
    if (shard_rows == 0) {
      for (int d = 0; d < peers.world; ++d) *reinterpret_cast<uint32_t*>(peers.heap[d] + dst_offset + i4) = word;
    } else {
      const long long row = i4 / cols;
      const int d = (int)(row / shard_rows);
      *reinterpret_cast<uint32_t*>(peers.heap[d] + dst_offset + (i4 - (long long)d * shard_rows * cols)) = word;
    }
  }
}

// ------------------------------------------------------------------------------------------
// path 4, whole write-back of an owner in two launches over a device-resident table
// ------------------------------------------------------------------------------------------
// One row per parameter this rank owns.  The reference does, per parameter and per step: amax -> scale ->
// quantise on the owner, scatter / broadcast of the codes, three small broadcasts (scale, amax history,
// call index) with a host sync, and later a separate EMA lerp (viola/distributed/parameters.py:121-147,
// viola/distributed/ema.py:100-113).  Here launch A reads every owned master once (EMA lerp + per-tensor
// amax), launch B reads it again (from L2 for all but the largest sets), encodes and stores the codes into
// the row slab of whichever rank holds those rows, and stores the layer header (scale, history slot) into
// every rank's copy of it.
struct WriteDesc {
  long long master;         // pointer: the updated master weight (fp32 / bf16 / fp16), contiguous
  long long ema;            // pointer: its running average, or 0
  long long amax;           // pointer: one uint32 slot (float bits), zeroed by the host before launch A
  long long n;              // elements
  long long slab_elems;     // elements per destination row slab (shard rows x row length); rank = element / slab_elems
  long long dst_offset;     // byte offset of this parameter's slab inside every rank's heap
  long long header_offset;  // byte offset of [scale, history[0..len)] inside every rank's heap, or -1
  long long base_index;     // quantizer call index when the table was built
  float limit;              // quantisation limit of FP8 rows
  int history_len;
  int master_dtype, ema_dtype;
  int mode;                 // 0 = e4m3 codes, 1 = e5m2 codes, 2 = cast to out_dtype
  int out_dtype;
  long long reserved[5];
};
static_assert(sizeof(WriteDesc) == 128, "write-back descriptor is 16 x 8 bytes");

constexpr int kWriteChunk = 4096;

__device__ __forceinline__ int find_row(const int* __restrict__ prefix, int rows, int block) {
  int lo = 0, hi = rows;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= block) lo = mid; else hi = mid;
  }
  return lo;
}

// Launch A: ema <- decay * ema + (1 - decay) * master (when the row has an average and with_ema) and the
// per-tensor amax of FP8 rows (NaN ignored, as the stand-alone amax kernel does).
__global__ void __launch_bounds__(256)
writeback_amax_kernel(const WriteDesc* __restrict__ table, const int* __restrict__ prefix, int rows, float decay,
                      int with_ema) {
  const int t = find_row(prefix, rows, blockIdx.x);
  const WriteDesc d = table[t];
  const long long begin = (long long)(blockIdx.x - prefix[t]) * kWriteChunk;
  const long long end = min(begin + kWriteChunk, d.n);
  const void* master = reinterpret_cast<const void*>(d.master);
  void* ema = with_ema ? reinterpret_cast<void*>(d.ema) : nullptr;
  if (ema == nullptr && d.mode == 2) return;
  float m = 0.f;
  const bool vec = d.master_dtype == kF32 && (d.master & 15) == 0 && (ema == nullptr || (d.ema_dtype == kF32 && (d.ema & 15) == 0));
  if (vec) {
    const long long vend = begin + ((end - begin) & ~3LL);
    for (long long i = begin + 4LL * threadIdx.x; i < vend; i += 4LL * blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(master) + i);
      if (ema != nullptr) {
        float4 e = *reinterpret_cast<float4*>(reinterpret_cast<float*>(ema) + i);
        e.x = fmaf(1.f - decay, v.x, e.x * decay);
        e.y = fmaf(1.f - decay, v.y, e.y * decay);
        e.z = fmaf(1.f - decay, v.z, e.z * decay);
        e.w = fmaf(1.f - decay, v.w, e.w * decay);
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(ema) + i) = e;
      }
      m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
    for (long long i = vend + threadIdx.x; i < end; i += blockDim.x) {
      const float v = reinterpret_cast<const float*>(master)[i];
      if (ema != nullptr) reinterpret_cast<float*>(ema)[i] = fmaf(1.f - decay, v, reinterpret_cast<float*>(ema)[i] * decay);
      m = fmaxf(m, fabsf(v));
    }
  } else {
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
      const float v = load_as_float(master, i, d.master_dtype);
      if (ema != nullptr) store_from_float(ema, i, d.ema_dtype, fmaf(1.f - decay, v, load_as_float(ema, i, d.ema_dtype) * decay));
      m = fmaxf(m, fabsf(v));
    }
  }
  if (d.mode == 2) return;
  m = warp_max(m);
  __shared__ float warp_m[8];
  if ((threadIdx.x & 31) == 0) warp_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = 0.f;
    for (int i = 0; i < 8; ++i) b = fmaxf(b, warp_m[i]);
    atomicMax(reinterpret_cast<unsigned int*>(d.amax), __float_as_uint(b));   // non-negative floats order like uints
  }
}

__device__ __forceinline__ uint8_t* slab_address(const Peers& peers, const WriteDesc& d, long long element, int bytes_per_element) {
  const int rank = d.slab_elems > 0 ? (int)(element / d.slab_elems) : 0;
  const long long local = element - (long long)rank * d.slab_elems;
  return peers.heap[rank] + d.dst_offset + local * bytes_per_element;
}

// Launch B: scale = max(amax, 1e-30) / limit (current scaling); codes = round(clamp(master / scale)) stored into
// the slab of the rank that holds each row; the first block of a row also stores the header everywhere.
// `calls` = write-backs since the table was built (the history slot is (base_index + calls) % history_len).
__global__ void __launch_bounds__(256)
writeback_push_kernel(const WriteDesc* __restrict__ table, const int* __restrict__ prefix, int rows, Peers peers,
                      long long calls) {
  const int t = find_row(prefix, rows, blockIdx.x);
  const WriteDesc d = table[t];
  const long long begin = (long long)(blockIdx.x - prefix[t]) * kWriteChunk;
  const long long end = min(begin + kWriteChunk, d.n);
  const void* master = reinterpret_cast<const void*>(d.master);
  if (d.mode == 2) {
    const int width = d.out_dtype == kF32 ? 4 : 2;
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x)
      store_from_float(slab_address(peers, d, i, width), 0, d.out_dtype, load_as_float(master, i, d.master_dtype));
    return;
  }
  const float amax = __uint_as_float(*reinterpret_cast<const unsigned int*>(d.amax));
  const float scale = fmaxf(amax, 1e-30f) / d.limit;
  if (blockIdx.x == prefix[t] && d.header_offset >= 0 && (int)threadIdx.x < peers.world) {
    float* header = reinterpret_cast<float*>(peers.heap[threadIdx.x] + d.header_offset);
    header[0] = scale;
    if (d.history_len > 0) header[1 + (int)((d.base_index + calls) % d.history_len)] = amax;
  }
  const bool vec = d.master_dtype == kF32 && (d.master & 15) == 0 && (d.slab_elems % 16) == 0 && (d.dst_offset % 16) == 0;
  long long i = begin;
  if (vec) {
    const long long vend = begin + ((end - begin) & ~15LL);
    for (long long j = begin + 16LL * threadIdx.x; j < vend; j += 16LL * blockDim.x) {
      uint32_t words[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(master) + j + 4 * q);
        words[q] = (uint32_t)fp8_encode(scaled_clamp(v.x, scale, d.limit), d.mode)
                 | (uint32_t)fp8_encode(scaled_clamp(v.y, scale, d.limit), d.mode) << 8
                 | (uint32_t)fp8_encode(scaled_clamp(v.z, scale, d.limit), d.mode) << 16
                 | (uint32_t)fp8_encode(scaled_clamp(v.w, scale, d.limit), d.mode) << 24;
      }
      *reinterpret_cast<uint4*>(slab_address(peers, d, j, 1)) = make_uint4(words[0], words[1], words[2], words[3]);
    }
    i = vend;
  }
  for (long long j = i + threadIdx.x; j < end; j += blockDim.x)
    *slab_address(peers, d, j, 1) = fp8_encode(scaled_clamp(load_as_float(master, j, d.master_dtype), scale, d.limit), d.mode);
}

// Plain byte push of an already encoded payload (16-byte vectors): full copy to everyone or one slab per rank.
__global__ void __launch_bounds__(256)
byte_push_kernel(const uint8_t* __restrict__ src, long long bytes, Peers peers, long long dst_offset, long long shard_bytes) {
  const long long vectors = bytes / 16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vectors; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(src)[i];
    if (shard_bytes == 0) {
      for (int d = 0; d < peers.world; ++d) reinterpret_cast<uint4*>(peers.heap[d] + dst_offset)[i] = v;
    } else {
      const int d = (int)(i * 16 / shard_bytes);
      *reinterpret_cast<uint4*>(peers.heap[d] + dst_offset + (i * 16 - (long long)d * shard_bytes)) = v;
    }
  }
  // tail (< 16 bytes)
  if (blockIdx.x == 0 && threadIdx.x < bytes - vectors * 16) {
    const long long i = vectors * 16 + threadIdx.x;
    if (shard_bytes == 0) {
      for (int d = 0; d < peers.world; ++d) peers.heap[d][dst_offset + i] = src[i];
    } else {
      const int d = (int)(i / shard_bytes);
      peers.heap[d][dst_offset + (i - (long long)d * shard_bytes)] = src[i];
    }
  }
}

__global__ void signal_kernel(Peers peers, long long flag_offset, int value, int include_self) {
  __threadfence_system();
  const int d = threadIdx.x;
  if (d < peers.world && (include_self || d != peers.rank))
    st_release_sys(reinterpret_cast<int*>(peers.heap[d] + flag_offset) + peers.rank, value);
}

__global__ void wait_flags_kernel(const int* flags, int count, int skip, int expected, long long budget, int* status) {
  block_wait_flags(flags, count, skip, expected, budget, status);
}

// ------------------------------------------------------------------------------------------
// path 3
// ------------------------------------------------------------------------------------------
struct GatherEntry {
  long long shard_offset;   // bytes inside the peers' shard region
  long long shard_bytes;    // bytes of one rank's slab
  long long full_offset;    // bytes inside the local full buffer (slab r lands at full_offset + r * shard_bytes)
};

// One CTA copies one 64 KiB piece of one (entry, source rank) slab with 16-byte loads from the
// peer.  piece_counts[entry * world + rank] counts finished pieces; the CTA that completes a slab
// raises panel_flags[entry * world + rank] = generation.
__global__ void __launch_bounds__(256)
gather_pull_kernel(const GatherEntry* __restrict__ entries, int num_entries, Peers peers, long long shard_region_offset,
                   uint8_t* __restrict__ full, const long long* __restrict__ piece_prefix, unsigned int* piece_counts,
                   int* panel_flags, int generation) {
  constexpr long long kPiece = 65536;
  __shared__ bool last;
  const long long total_pieces = piece_prefix[num_entries * peers.world];
  for (long long piece = blockIdx.x; piece < total_pieces; piece += gridDim.x) {
    // locate (entry, rank) by a linear scan of the prefix table (tens of entries)
    int slab = 0;
    while (piece >= piece_prefix[slab + 1]) ++slab;
    const int entry = slab / peers.world;
    // visit the local slab first, then the peers in ring order, so early consumers find local rows ready
    const int rank = (peers.rank + slab % peers.world) % peers.world;
    const int slot = entry * peers.world + rank;
    const GatherEntry e = entries[entry];
    const long long first = (piece - piece_prefix[slab]) * kPiece;
    const long long bytes = min(kPiece, e.shard_bytes - first);
    const uint8_t* src = peers.heap[rank] + shard_region_offset + e.shard_offset + first;
    uint8_t* dst = full + e.full_offset + (long long)rank * e.shard_bytes + first;
    const long long vectors = bytes / 16;
    long long i = threadIdx.x;
    for (; i + 3 * (long long)blockDim.x < vectors; i += 4 * (long long)blockDim.x) {   // four peer loads in flight per thread
      const uint4 v0 = reinterpret_cast<const uint4*>(src)[i];
      const uint4 v1 = reinterpret_cast<const uint4*>(src)[i + blockDim.x];
      const uint4 v2 = reinterpret_cast<const uint4*>(src)[i + 2 * blockDim.x];
      const uint4 v3 = reinterpret_cast<const uint4*>(src)[i + 3 * blockDim.x];
      reinterpret_cast<uint4*>(dst)[i] = v0;
      reinterpret_cast<uint4*>(dst)[i + blockDim.x] = v1;
      reinterpret_cast<uint4*>(dst)[i + 2 * blockDim.x] = v2;
      reinterpret_cast<uint4*>(dst)[i + 3 * blockDim.x] = v3;
    }
    for (; i < vectors; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    for (long long j = vectors * 16 + threadIdx.x; j < bytes; j += blockDim.x) dst[j] = src[j];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int pieces = (unsigned int)(piece_prefix[slab + 1] - piece_prefix[slab]);
      last = atomicAdd(&piece_counts[slot], 1u) == pieces - 1;
      if (last) {
        piece_counts[slot] = 0u;
        __threadfence();
        atomicExch(&panel_flags[slot], generation);
      }
    }
    __syncthreads();
  }
}

static Peers make_peers(const VbPeerTable* table) {
  Peers p{};
  p.world = table->world;
  p.rank = table->rank;
  for (int i = 0; i < 16; ++i) p.heap[i] = reinterpret_cast<uint8_t*>(table->buffers[i]);
  return p;
}

}  // namespace vb

using namespace vb;

#define VB_TILE_SWITCH(tile, ...)                              \
  switch (tile) {                                              \
    case 32: { constexpr int T = 32; __VA_ARGS__; } break;     \
    case 64: { constexpr int T = 64; __VA_ARGS__; } break;     \
    case 128: { constexpr int T = 128; __VA_ARGS__; } break;   \
    case 256: { constexpr int T = 256; __VA_ARGS__; } break;   \
    case 512: { constexpr int T = 512; __VA_ARGS__; } break;   \
    case 1024: { constexpr int T = 1024; __VA_ARGS__; } break; \
    default: return (int)cudaErrorInvalidValue;                \
  }

static int blocks_for(long long warps_needed, int max_blocks) {
  long long b = (warps_needed + 7) / 8;
  if (b < 1) b = 1;
  return (int)std::min<long long>(b, max_blocks);
}

extern "C" int vb_reduce_push_fp8(const float* bucket, long long n, int tile, int fmt, void* dst_codes, float* dst_scales,
                                  int* dst_flag, const int* ack_flag, const int* generation, unsigned int* counter,
                                  long long wait_clocks, int max_blocks, int* status, cudaStream_t stream) {
  const long long tiles = (n + tile - 1) / tile;
  const int grid = blocks_for(tiles, max_blocks);
  wait_generation_kernel<<<1, 32, 0, stream>>>(ack_flag, 1, -1, generation, -1, wait_clocks, status);
  VB_TILE_SWITCH(tile, (reduce_push_kernel<T><<<grid, 256, 0, stream>>>(bucket, n, fmt, (uint8_t*)dst_codes, dst_scales, dst_flag,
                                                                       ack_flag, generation, counter, wait_clocks, status)));
  return (int)cudaGetLastError();
}

extern "C" int vb_reduce_accumulate_fp8(const float* bucket, long long n, int tile, int fmt, const void* recv,
                                        long long slot_stride, long long scales_offset, const int* flags,
                                        const VbPeerTable* peers, long long ack_offset, const int* generation, float* accum,
                                        unsigned int* counter, long long wait_clocks, int max_blocks, int* status,
                                        cudaStream_t stream) {
  const long long tiles = (n + tile - 1) / tile;
  const int grid = blocks_for(tiles, max_blocks);
  wait_generation_kernel<<<1, 32, 0, stream>>>(flags, peers->world, peers->rank, generation, 0, wait_clocks, status);
  VB_TILE_SWITCH(tile, (reduce_accumulate_kernel<T><<<grid, 256, 0, stream>>>(bucket, n, fmt, (const uint8_t*)recv, slot_stride,
                                                                             scales_offset, flags, make_peers(peers), ack_offset,
                                                                             generation, accum, counter, wait_clocks, status)));
  return (int)cudaGetLastError();
}

extern "C" int vb_reduce_push_many(const void* table, const long long* prefix, int buckets, long long total_tiles, int tile,
                                   int fmt, const VbPeerTable* peers, long long flag_offset, const int* ack_flags,
                                   const int* generation, unsigned int* counter, long long wait_clocks, int max_blocks,
                                   int* status, cudaStream_t stream) {
  if (buckets < 0 || total_tiles < 0) return 0;      // an empty table still raises this rank's flag at every peer
  const int grid = blocks_for(total_tiles, max_blocks);
  wait_generation_kernel<<<1, 32, 0, stream>>>(ack_flags, peers->world, peers->rank, generation, -1, wait_clocks, status);
  VB_TILE_SWITCH(tile, (reduce_push_many_kernel<T><<<grid, 256, 0, stream>>>(
                           reinterpret_cast<const ReduceDesc*>(table), prefix, buckets, fmt, make_peers(peers), flag_offset,
                           ack_flags, generation, counter, wait_clocks, status)));
  return (int)cudaGetLastError();
}

extern "C" int vb_reduce_accumulate_many(const void* table, const long long* prefix, int buckets, long long total_tiles,
                                         int tile, int fmt, const VbPeerTable* peers, const int* flags, long long ack_offset,
                                         const int* generation, unsigned int* counter, long long wait_clocks, int max_blocks,
                                         int* status, cudaStream_t stream) {
  if (buckets < 0 || total_tiles < 0) return 0;      // an empty table still waits and acknowledges
  const int grid = blocks_for(total_tiles, max_blocks);
  wait_generation_kernel<<<1, 32, 0, stream>>>(flags, peers->world, peers->rank, generation, 0, wait_clocks, status);
  VB_TILE_SWITCH(tile, (reduce_accumulate_many_kernel<T><<<grid, 256, 0, stream>>>(
                           reinterpret_cast<const ReduceDesc*>(table), prefix, buckets, fmt, make_peers(peers), flags,
                           ack_offset, generation, counter, wait_clocks, status)));
  return (int)cudaGetLastError();
}

extern "C" int vb_allreduce_requant_fp8(float* value, long long n, int tile, int fmt, const VbPeerTable* peers,
                                        long long a2a_offset, long long gather_offset, long long slot,
                                        long long a2a_flag_offset, long long gather_flag_offset, int generation,
                                        unsigned int* counters, long long wait_clocks, int max_blocks, int* status,
                                        cudaStream_t stream) {
  const int world = peers->world;
  const int groups = (int)((n + (long long)world * tile - 1) / ((long long)world * tile));
  const Peers p = make_peers(peers);
  const int grid_all = blocks_for((long long)world * groups, max_blocks);
  const int grid_own = blocks_for(groups, max_blocks);
  VB_TILE_SWITCH(tile, {
    allreduce_push_kernel<T><<<grid_all, 256, 0, stream>>>(value, n, groups, fmt, p, a2a_offset, slot, a2a_flag_offset,
                                                          generation, counters);
    // stand-alone single-warp waits in front of the kernels whose blocks would otherwise all poll
    wait_flags_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const int*>(p.heap[p.rank] + a2a_flag_offset), world, p.rank,
                                            generation, wait_clocks, status);
    allreduce_reduce_kernel<T><<<grid_own, 256, 0, stream>>>(value, n, groups, fmt, p, a2a_offset, gather_offset, slot,
                                                            a2a_flag_offset, gather_flag_offset, generation, counters + 1,
                                                            wait_clocks, status);
    wait_flags_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const int*>(p.heap[p.rank] + gather_flag_offset), world, p.rank,
                                            generation, wait_clocks, status);
    allreduce_unpack_kernel<T><<<grid_all, 256, 0, stream>>>(value, n, groups, fmt, p, gather_offset, slot, gather_flag_offset,
                                                            generation, wait_clocks, status);
  });
  return (int)cudaGetLastError();
}

extern "C" int vb_quantize_push(const void* master, int master_dtype, long long rows, long long cols, const float* scale,
                                float limit, int fmt, void* ema, int ema_dtype, float decay, const VbPeerTable* peers,
                                long long dst_offset, long long shard_rows, int max_blocks, cudaStream_t stream) {
  if (cols % 4 != 0 || dst_offset % 4 != 0) return (int)cudaErrorInvalidValue;
  const long long n = rows * cols;
  if (n <= 0) return 0;
  const int grid = (int)std::min<long long>((n / 4 + 255) / 256, max_blocks);
  quantize_push_kernel<<<grid, 256, 0, stream>>>(master, master_dtype, rows, cols, scale, limit, fmt, ema, ema_dtype, decay,
                                                 make_peers(peers), dst_offset, shard_rows);
  return (int)cudaGetLastError();
}

extern "C" int vb_byte_push(const void* src, long long bytes, const VbPeerTable* peers, long long dst_offset,
                            long long shard_bytes, int max_blocks, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  if (dst_offset % 16 != 0 || (shard_bytes % 16) != 0 || (reinterpret_cast<uintptr_t>(src) & 15) != 0)
    return (int)cudaErrorMisalignedAddress;
  const int grid = (int)std::max<long long>(1, std::min<long long>((bytes / 16 + 255) / 256, max_blocks));
  byte_push_kernel<<<grid, 256, 0, stream>>>((const uint8_t*)src, bytes, make_peers(peers), dst_offset, shard_bytes);
  return (int)cudaGetLastError();
}

extern "C" int vb_signal(const VbPeerTable* peers, long long flag_offset, int value, int include_self, cudaStream_t stream) {
  signal_kernel<<<1, 32, 0, stream>>>(make_peers(peers), flag_offset, value, include_self);
  return (int)cudaGetLastError();
}

extern "C" int vb_wait_flags(const int* flags, int count, int skip, int expected, long long wait_clocks, int* status,
                             cudaStream_t stream) {
  wait_flags_kernel<<<1, 32, 0, stream>>>(flags, count, skip, expected, wait_clocks, status);
  return (int)cudaGetLastError();
}

extern "C" int vb_gather_pull(const void* entries, int num_entries, const VbPeerTable* peers, long long shard_region_offset,
                              void* full, const long long* piece_prefix, unsigned int* piece_counts, int* panel_flags,
                              int generation, long long total_pieces, int max_blocks, cudaStream_t stream) {
  if (total_pieces <= 0) return 0;
  const int grid = (int)std::min<long long>(total_pieces, max_blocks);
  gather_pull_kernel<<<grid, 256, 0, stream>>>((const GatherEntry*)entries, num_entries, make_peers(peers), shard_region_offset,
                                               (uint8_t*)full, piece_prefix, piece_counts, panel_flags, generation);
  return (int)cudaGetLastError();
}

// Fused owner write-back (see WriteDesc).  `amax_slots` (uint32 per row, referenced by the table) must be zero on
// entry; they are left holding the amax bits.  With world == 1 and peers->buffers[0] == nullptr the offsets of the
// table are absolute addresses, which lets a single process without a symmetric heap use the same kernels.
extern "C" int vb_multi_writeback(const void* table, const int* prefix, int rows, int blocks, float decay, int with_ema,
                                  const VbPeerTable* peers, long long calls, cudaStream_t stream) {
  if (blocks <= 0 || rows <= 0) return 0;
  writeback_amax_kernel<<<blocks, 256, 0, stream>>>((const WriteDesc*)table, prefix, rows, decay, with_ema);
  writeback_push_kernel<<<blocks, 256, 0, stream>>>((const WriteDesc*)table, prefix, rows, make_peers(peers), calls);
  return (int)cudaGetLastError();
}
