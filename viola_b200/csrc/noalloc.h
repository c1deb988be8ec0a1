// Allocation-free tensor-scale entry point.
//
// This entry point has no counterpart in the reference implementation.  It exists for callers
// that are not allowed to allocate device memory at the point where they need an FP8 scale:
// code running inside a memory-pool snapshot or under a fixed-footprint serving budget, host
// threads that do not own a CUDA allocator (a data-loader or communication thread), and
// embedders that link this library from C without PyTorch's caching allocator.  The regular
// entry point (vb_amax_scale in api.h) needs a caller-provided, zero-initialised scratch buffer,
// which those callers have no way to obtain; this variant keeps its scratch inside the library.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest input this entry point accepts (elements).  Bigger inputs are rejected, never truncated.
#define VB_NOALLOC_MAX_ELEMENTS (4096LL * 8192LL)

// scale_out[0] = max(amax(|x|), 1e-30) / limit for the n elements at x (dtype: 0 fp32, 1 bf16, 2 fp16);
// limit must be finite and greater than 0 (448 for e4m3, 57344 for e5m2, or a reduced range).
//
//  * x and scale_out are device pointers supplied by the caller; nothing else is needed.
//  * The scratch (4096 partial maxima + one ticket counter, 16.6 KB) is a file-scope device array
//    that every GPU loading this library holds until the process exits.
//  * The first call on a device resolves the array's device address (cudaGetSymbolAddress).  Make
//    that first call before starting any stream capture on that device.
//  * No cudaMalloc / cudaFree / allocating library routine is called, on any path.
//  * All calls on one device share the scratch array and it keeps the previous call's contents; the
//    entry point re-zeroes the ticket counter on the caller's stream before each launch.  Two calls
//    whose kernels can overlap on the same GPU (different streams, no ordering) race on it: order
//    them on one stream or with events.
//  * Returns 0 on success.  On failure returns a non-zero cudaError_t value and, when
//    error_message is not NULL, writes a NUL-terminated explanation of at most error_capacity bytes
//    (for example when n exceeds VB_NOALLOC_MAX_ELEMENTS).
int vb_tensor_scale_noalloc(const void* x, long long n, int dtype, float limit, float* scale_out,
                            cudaStream_t stream, char* error_message, size_t error_capacity);

#ifdef __cplusplus
}
#endif
