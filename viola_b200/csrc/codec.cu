// FP8 wire codec (sm_100a): fp32 gradients <-> packets of [codes | fp32 tile scales].
// Standalone pack / unpack are the unfused building blocks (and the NCCL-path
// baseline); the fused communication kernels in comm.cu reuse the same device
// functions so that both paths produce identical bytes.
//
// Packet row layout (viola/distributed/_fp8_kernels.py:10-15, fp8.py:9-11):
//   [groups * tile codes][groups fp32 scales], row stride padded to 16 bytes.
// amax maps NaN to +inf so a non-finite input poisons its whole tile
// (_fp8_kernels.py:35-37); reduction sums source ranks serially in ascending
// order in fp32 (_fp8_kernels.py:58-61).
#include "api.h"
#include "common/numerics.cuh"
#include "common/codec.cuh"

namespace vb {

template <int TILE>
__global__ void __launch_bounds__(256)
wire_pack_kernel(const float* __restrict__ x, long long n, int rows, int groups, int fmt,
                 uint8_t* __restrict__ packet, long long row_stride) {
  const long long total = (long long)rows * groups;
  const long long width = (long long)groups * TILE;
  const int lane = threadIdx.x & 31;
  for (long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < total;
       t += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int row = (int)(t / groups), group = (int)(t % groups);
    const long long src0 = (long long)row * width + (long long)group * TILE;
    uint8_t* codes = packet + (long long)row * row_stride + (long long)group * TILE;
    float* scale = reinterpret_cast<float*>(packet + (long long)row * row_stride + width) + group;
    pack_tile<TILE>(x, src0, n, fmt, codes, scale, lane);
  }
}

template <int TILE>
__global__ void __launch_bounds__(256)
wire_unpack_kernel(const uint8_t* __restrict__ packet, long long row_stride, int rows, int groups, int fmt,
                   int reduce, float* __restrict__ out, long long n, int accumulate) {
  const long long width = (long long)groups * TILE;
  const int out_rows = reduce ? 1 : rows;
  const long long total = (long long)out_rows * groups;
  const int lane = threadIdx.x & 31;
  constexpr int EPL = TILE / 32;
  for (long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < total;
       t += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int row = (int)(t / groups), group = (int)(t % groups);
    float result[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) result[e] = 0.f;
    const int first = reduce ? 0 : row, last = reduce ? rows : row + 1;
    for (int r = first; r < last; ++r) {
      const uint8_t* codes = packet + (long long)r * row_stride + (long long)group * TILE;
      const float s = *(reinterpret_cast<const float*>(packet + (long long)r * row_stride + width) + group);
      accumulate_tile<TILE>(codes, s, fmt, lane, result);
    }
    const long long dst0 = (reduce ? 0 : (long long)row * width) + (long long)group * TILE;
    store_tile<TILE>(out, dst0, n, lane, result, accumulate != 0);
  }
}

}  // namespace vb

using namespace vb;

#define VB_TILE_SWITCH(tile, ...)                         \
  switch (tile) {                                          \
    case 32: { constexpr int T = 32; __VA_ARGS__; } break;   \
    case 64: { constexpr int T = 64; __VA_ARGS__; } break;   \
    case 128: { constexpr int T = 128; __VA_ARGS__; } break; \
    case 256: { constexpr int T = 256; __VA_ARGS__; } break; \
    case 512: { constexpr int T = 512; __VA_ARGS__; } break; \
    case 1024: { constexpr int T = 1024; __VA_ARGS__; } break; \
    default: return (int)cudaErrorInvalidValue;            \
  }

extern "C" int vb_wire_pack(const float* x, long long n, int rows, int groups, int tile, int fmt, uint8_t* packet,
                            long long row_stride, cudaStream_t stream) {
  const long long total = (long long)rows * groups;
  if (total <= 0) return 0;
  const int grid = (int)std::min<long long>((total + 7) / 8, 148LL * 16);
  VB_TILE_SWITCH(tile, (wire_pack_kernel<T><<<grid, 256, 0, stream>>>(x, n, rows, groups, fmt, packet, row_stride)));
  return (int)cudaGetLastError();
}

extern "C" int vb_wire_unpack(const uint8_t* packet, long long row_stride, int rows, int groups, int tile, int fmt,
                              int reduce, float* out, long long n, int accumulate, cudaStream_t stream) {
  const long long total = (long long)(reduce ? 1 : rows) * groups;
  if (total <= 0) return 0;
  const int grid = (int)std::min<long long>((total + 7) / 8, 148LL * 16);
  VB_TILE_SWITCH(tile, (wire_unpack_kernel<T><<<grid, 256, 0, stream>>>(packet, row_stride, rows, groups, fmt, reduce,
                                                                      out, n, accumulate)));
  return (int)cudaGetLastError();
}
