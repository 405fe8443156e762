// C declarations of entry points that C/C++ hosts may call without going through the Python binding.
// Every function returns 0 on success or a negative lvb error code (see common.cuh).
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// out[0] (+)= sum(x[i]^2), i < n.  x is fp32 (is_bf16 = 0) or bf16; scratch is caller-provided fp32 [1024] on the same device.
int lvb_sumsq(const void* x, long long n, int is_bf16, float* scratch, float* out, int accumulate, void* stream);

// Same result as lvb_sumsq, but the partial-sum scratch is a fixed array inside the library, so the call performs no device
// allocation of any kind.  This entry point has no counterpart in the reference framework; it exists for hosts that must
// not allocate (see the comment above its definition in optim.cu).
//   * `stream` must be a stream of the device that is current (cudaGetDevice) at the call: the scratch address is looked up
//     for the current device, and a stream of another device is not detected here.
//   * The scratch address is cached per device for the life of the process; cudaDeviceReset (or anything else that destroys
//     the primary context) invalidates it, and the entry point must not be called again in that process afterwards.
//   * n must be in [1, lvb_sumsq_noalloc_max_elems()]; larger n returns -4 and lvb_sumsq_noalloc_last_error() says why.
//   * The first call on each device resolves the scratch address (a one-time set-up with that device current); make that
//     first call before starting any stream capture.
//   * The scratch is one per device: two calls that overlap on the GPU (different streams, no ordering) race on it.
int lvb_sumsq_noalloc(const void* x, long long n, int is_bf16, float* out, int accumulate, void* stream);
long long lvb_sumsq_noalloc_max_elems(void);
const char* lvb_sumsq_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
