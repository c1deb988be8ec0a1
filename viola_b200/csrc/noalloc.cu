// Allocation-free variant of the amax -> scale kernel (see noalloc.h for the contract and for who
// needs it).  The per-block partial maxima and the ticket counter live in a file-scope device
// array instead of caller-provided scratch.
#include <cstdio>
#include <cstring>
#include <mutex>
#include "noalloc.h"
#include "common/numerics.cuh"

namespace {

constexpr int kMaxBlocks = 4096;
constexpr int kElementsPerBlock = 8192;
constexpr int kCounterIndex = kMaxBlocks;      // word after the partial maxima
constexpr int kMaxDevices = 64;

// [0, kMaxBlocks): per-block amax as float bits; [kCounterIndex]: ticket counter.
static __device__ __align__(256) unsigned int g_scratch[kMaxBlocks + 64];

__global__ void __launch_bounds__(256)
noalloc_scale_kernel(const void* __restrict__ x, long long n, int dtype, float limit, float* __restrict__ scale_out,
                     unsigned int* __restrict__ scratch) {
  const long long begin = (long long)blockIdx.x * kElementsPerBlock;
  const long long end = begin + kElementsPerBlock < n ? begin + kElementsPerBlock : n;
  float m = 0.f;
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) m = fmaxf(m, fabsf(vb::load_as_float(x, i, dtype)));
  m = vb::warp_max(m);
  __shared__ float warp_m[8];
  __shared__ bool last;
  if ((threadIdx.x & 31) == 0) warp_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = 0.f;
    for (int i = 0; i < 8; ++i) b = fmaxf(b, warp_m[i]);
    scratch[blockIdx.x] = __float_as_uint(b);
    __threadfence();
    last = atomicAdd(&scratch[kCounterIndex], 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  float total = 0.f;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x)
    total = fmaxf(total, __uint_as_float(reinterpret_cast<volatile unsigned int*>(scratch)[i]));
  total = vb::warp_max(total);
  if ((threadIdx.x & 31) == 0) warp_m[threadIdx.x >> 5] = total;
  __syncthreads();
  if (threadIdx.x == 0) {
    float amax = 0.f;
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, warp_m[i]);
    scale_out[0] = fmaxf(amax, 1e-30f) / limit;
    scratch[kCounterIndex] = 0u;
  }
}

std::mutex g_mutex;
unsigned int* g_scratch_address[kMaxDevices] = {};

int fail(int code, const char* text, char* message, size_t capacity) {
  if (message != nullptr && capacity > 0) {
    std::strncpy(message, text, capacity - 1);
    message[capacity - 1] = '\0';
  }
  return code;
}

}  // namespace

extern "C" int vb_tensor_scale_noalloc(const void* x, long long n, int dtype, float limit, float* scale_out,
                                       cudaStream_t stream, char* error_message, size_t error_capacity) {
  if (x == nullptr || scale_out == nullptr || n <= 0)
    return fail((int)cudaErrorInvalidValue, "vb_tensor_scale_noalloc: x and scale_out must be set and n positive",
                error_message, error_capacity);
  if (dtype < 0 || dtype > 2)
    return fail((int)cudaErrorInvalidValue, "vb_tensor_scale_noalloc: dtype must be 0 (fp32), 1 (bf16) or 2 (fp16)",
                error_message, error_capacity);
  if (!(limit > 0.0f) || limit > 3.0e38f)       // also catches NaN: a scale of amax / limit must be finite and positive
    return fail((int)cudaErrorInvalidValue, "vb_tensor_scale_noalloc: limit must be a finite number greater than 0",
                error_message, error_capacity);
  if (n > VB_NOALLOC_MAX_ELEMENTS) {
    char text[192];
    std::snprintf(text, sizeof(text), "vb_tensor_scale_noalloc: n = %lld exceeds the built-in scratch limit of %lld elements",
                  n, (long long)VB_NOALLOC_MAX_ELEMENTS);
    return fail((int)cudaErrorInvalidValue, text, error_message, error_capacity);
  }
  int device = 0;
  cudaError_t rc = cudaGetDevice(&device);
  if (rc != cudaSuccess) return fail((int)rc, "vb_tensor_scale_noalloc: cudaGetDevice failed", error_message, error_capacity);
  if (device < 0 || device >= kMaxDevices)
    return fail((int)cudaErrorInvalidDevice, "vb_tensor_scale_noalloc: device ordinal out of range", error_message,
                error_capacity);
  unsigned int* scratch = nullptr;
  {
    // First call on this device: turn the host-side stand-in `g_scratch` into this device's address.
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_address[device] == nullptr) {
      unsigned int* resolved = nullptr;
      rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&resolved), g_scratch);
      if (rc != cudaSuccess || resolved == nullptr)
        return fail((int)(rc != cudaSuccess ? rc : cudaErrorInvalidSymbol),
                    "vb_tensor_scale_noalloc: cudaGetSymbolAddress on the scratch array failed", error_message,
                    error_capacity);
      g_scratch_address[device] = resolved;
    }
    scratch = g_scratch_address[device];
  }
  // The array keeps whatever the previous call left; only the ticket counter must start at zero.
  rc = cudaMemsetAsync(scratch + kCounterIndex, 0, sizeof(unsigned int), stream);
  if (rc != cudaSuccess) return fail((int)rc, "vb_tensor_scale_noalloc: clearing the ticket counter failed", error_message,
                                     error_capacity);
  const int blocks = (int)((n + kElementsPerBlock - 1) / kElementsPerBlock);
  noalloc_scale_kernel<<<blocks, 256, 0, stream>>>(x, n, dtype, limit, scale_out, scratch);
  rc = cudaGetLastError();
  if (rc != cudaSuccess) return fail((int)rc, "vb_tensor_scale_noalloc: kernel launch failed", error_message, error_capacity);
  return 0;
}
