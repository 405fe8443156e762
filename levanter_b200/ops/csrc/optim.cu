// Optimizer kernels over flat parameter shards.
//
//  * sumsq: deterministic two-stage sum of squares (global gradient norm; the cross-rank part is a
//    tiny all-reduce done by the caller)
//  * clip_coef: min(1, max_norm / (norm + 1e-6)) kept on the device so no host sync is needed
//  * adamw: clip -> Adam moments -> bias correction -> decoupled weight decay -> -lr, in the order
//    of the reference's optax chain (src/levanter/optim/config.py:458-494), writing the fp32 master
//    weights and the bf16 compute copy in one pass.
#include "common.cuh"

namespace lvb {
namespace optim {

constexpr int kBlock = 256;
constexpr int kMaxParts = 1024;

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(kBlock) sumsq_partial_kernel(const T* __restrict__ x, long long n,
                                                               float* __restrict__ partial) {
  float acc = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * kBlock) {
    float v = ldf<T>(x, i);
    acc += v * v;
  }
  acc = warp_sum(acc);
  __shared__ float sm[kBlock / 32];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < kBlock / 32; ++w) s += sm[w];
    partial[blockIdx.x] = s;
  }
}

__global__ void sumsq_final_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out,
                                   int accumulate) {
  // single warp, fixed order: deterministic
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 32) acc += partial[i];
  acc = warp_sum(acc);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc : acc;
}

__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float* __restrict__ coef,
                                 float* __restrict__ norm_out) {
  const float norm = sqrtf(sumsq[0]);
  if (norm_out != nullptr) norm_out[0] = norm;
  coef[0] = (max_norm > 0.f && norm > max_norm) ? max_norm / (norm + 1e-6f) : 1.f;
}

__device__ __forceinline__ void adamw_one(float& pi, float& mi, float& vi, float gi, float lr, float b1, float b2, float eps, float wd,
                                          float bc1, float bc2, int nesterov) {
  mi = b1 * mi + (1.f - b1) * gi;
  vi = b2 * vi + (1.f - b2) * gi * gi;
  // optax scale_by_adam: nesterov uses b1 * m_hat(t+1 correction) + (1 - b1) * g / bc1
  float mhat = mi / bc1;
  if (nesterov) mhat = b1 * (mi / (1.f - (1.f - bc1) * b1)) + (1.f - b1) * gi / bc1;
  const float vhat = vi / bc2;
  float u = mhat / (sqrtf(vhat) + eps);
  u += wd * pi;
  pi = pi - lr * u;
}

// Four elements per thread and iteration through 16-byte accesses (every array 16-byte aligned: checked by the launcher, which
// otherwise passes vec = 0); the last n % 4 elements, or everything when vec = 0, go one by one.
template <typename G>
__global__ void __launch_bounds__(kBlock)
adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const G* __restrict__ g,
             __nv_bfloat16* __restrict__ p_bf16, long long n, float lr, float b1, float b2, float eps, float wd,
             float bc1, float bc2, const float* __restrict__ grad_scale, float grad_mul, int nesterov, int vec) {
  const float gs = (grad_scale != nullptr ? grad_scale[0] : 1.f) * grad_mul;
  const long long tid = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  const long long n4 = vec ? n / 4 : 0;
  for (long long q = tid; q < n4; q += stride) {
    float4 pp = reinterpret_cast<float4*>(p)[q], mm = reinterpret_cast<float4*>(m)[q], vv = reinterpret_cast<float4*>(v)[q];
    float gg[4];
    if constexpr (sizeof(G) == 4) {
      const float4 t = reinterpret_cast<const float4*>(g)[q];
      gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2*>(g)[q];
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
      gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
    }
    adamw_one(pp.x, mm.x, vv.x, gg[0] * gs, lr, b1, b2, eps, wd, bc1, bc2, nesterov);
    adamw_one(pp.y, mm.y, vv.y, gg[1] * gs, lr, b1, b2, eps, wd, bc1, bc2, nesterov);
    adamw_one(pp.z, mm.z, vv.z, gg[2] * gs, lr, b1, b2, eps, wd, bc1, bc2, nesterov);
    adamw_one(pp.w, mm.w, vv.w, gg[3] * gs, lr, b1, b2, eps, wd, bc1, bc2, nesterov);
    reinterpret_cast<float4*>(p)[q] = pp;
    reinterpret_cast<float4*>(m)[q] = mm;
    reinterpret_cast<float4*>(v)[q] = vv;
    if (p_bf16 != nullptr) reinterpret_cast<uint2*>(p_bf16)[q] = make_uint2(pack_bf16x2(pp.x, pp.y), pack_bf16x2(pp.z, pp.w));
  }
  for (long long i = 4 * n4 + tid; i < n; i += stride) {
    float pi = p[i], mi = m[i], vi = v[i];
    adamw_one(pi, mi, vi, ldf<G>(g, i) * gs, lr, b1, b2, eps, wd, bc1, bc2, nesterov);
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
    if (p_bf16 != nullptr) p_bf16[i] = __float2bfloat16(pi);
  }
}

inline int grid_for(long long n) {
  long long g = (n + kBlock - 1) / kBlock;
  long long cap = static_cast<long long>(num_sms()) * 8;
  if (cap > kMaxParts) cap = kMaxParts;
  return static_cast<int>(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace optim
}  // namespace lvb

// out[0] (+)= sum(x^2).  x is fp32 (is_bf16 = 0) or bf16.  scratch: fp32 [1024].
extern "C" int lvb_sumsq(const void* x, long long n, int is_bf16, float* scratch, float* out, int accumulate,
                         void* stream) {
  using namespace lvb;
  using namespace lvb::optim;
  if (n <= 0) return kErrBadArg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(n);
  if (is_bf16)
    sumsq_partial_kernel<__nv_bfloat16><<<grid, kBlock, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), n, scratch);
  else
    sumsq_partial_kernel<float><<<grid, kBlock, 0, s>>>(reinterpret_cast<const float*>(x), n, scratch);
  sumsq_final_kernel<<<1, 32, 0, s>>>(scratch, grid, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

extern "C" int lvb_clip_coef(const float* sumsq, float max_norm, float* coef, float* norm_out, void* stream) {
  lvb::optim::clip_coef_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sumsq, max_norm, coef, norm_out);
  return cudaGetLastError() == cudaSuccess ? lvb::kErrOk : lvb::kErrCuda;
}

// Fused AdamW over a flat shard.  p/m/v fp32 [n]; g fp32 or bf16 [n]; p_bf16 optional bf16 [n].
// grad_scale: optional device scalar (clip coefficient); grad_mul: host scalar (e.g. 1/accum_steps).
// bc1 = 1 - b1^t, bc2 = 1 - b2^t.
extern "C" int lvb_adamw(float* p, float* m, float* v, const void* g, int g_is_bf16, void* p_bf16, long long n, float lr,
                         float b1, float b2, float eps, float wd, float bc1, float bc2, const float* grad_scale,
                         float grad_mul, int nesterov, void* stream) {
  using namespace lvb;
  using namespace lvb::optim;
  if (n <= 0) return kErrBadArg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  long long gl = (n + kBlock - 1) / kBlock;
  long long cap = static_cast<long long>(num_sms()) * 16;
  const int grid = static_cast<int>(gl < cap ? gl : cap);
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(g) | (reinterpret_cast<uintptr_t>(p_bf16) << 1);  // bf16: 8-byte accesses
  const int vec = (bits & 15) == 0 ? 1 : 0;
  if (g_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, kBlock, 0, s>>>(p, m, v, reinterpret_cast<const __nv_bfloat16*>(g),
                                                        reinterpret_cast<__nv_bfloat16*>(p_bf16), n, lr, b1, b2, eps, wd,
                                                        bc1, bc2, grad_scale, grad_mul, nesterov,
                                                        vec && (reinterpret_cast<uintptr_t>(g) & 7) == 0);
  else
    adamw_kernel<float><<<grid, kBlock, 0, s>>>(p, m, v, reinterpret_cast<const float*>(g),
                                                reinterpret_cast<__nv_bfloat16*>(p_bf16), n, lr, b1, b2, eps, wd, bc1,
                                                bc2, grad_scale, grad_mul, nesterov, vec);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// ---------------------------------------------------------------------------------------------------------------------
// Sum of squares without any allocation.
//
// lvb_sumsq takes its 4 KB of partial-sum scratch from the caller, which in practice means from an allocator.  Some hosts
// cannot go to one at the moment they need a gradient norm:
//   * a plain C/C++ host has no caching allocator, and the driver's own allocate/free calls synchronise the whole device,
//     which would stall a step whose collectives and copies are in flight on other streams;
//   * a health-check or watchdog thread that samples the gradient norm while the training thread is inside the framework's
//     allocator must not take that lock or change the memory plan that was sized for the step.
// For them the scratch lives in the library image itself: a file-scope device array, whose address is looked up once per
// device.  Nothing is allocated, freed or resized here, by this code or by a library routine.
//
// Limits and rules:
//   * n <= kNoAllocMaxElems (2^31 elements); beyond that the call is rejected with kErrTooLarge and a message.
//   * The first call on a device does the address look-up (cudaGetSymbolAddress, with that device current); it should be
//     made before any stream capture begins, since the look-up is not a stream operation.
//   * The slots this call will read are cleared on the stream first, so partial sums left by an earlier call are never seen.
//   * One scratch per device: calls that may overlap on the GPU race on it.  Order them on one stream or with events.
#include "lvb_api.h"

#include <cstdio>
#include <mutex>

namespace lvb {
namespace optim {

constexpr long long kNoAllocMaxElems = 1LL << 31;
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) float g_noalloc_scratch[kMaxParts];

static float* g_noalloc_ptr[kNoAllocMaxDevices] = {};
static std::mutex g_noalloc_mu;
static thread_local char g_noalloc_err[192] = "";

static int noalloc_fail(int code, const char* fmt, long long a = 0, long long b = 0) {
  std::snprintf(g_noalloc_err, sizeof(g_noalloc_err), fmt, a, b);
  return code;
}

// Address of this device's copy of the scratch array; resolved on first use.
static int noalloc_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return noalloc_fail(kErrCuda, "lvb_sumsq_noalloc: no current CUDA device");
  if (dev >= kNoAllocMaxDevices)
    return noalloc_fail(kErrBadArg, "lvb_sumsq_noalloc: device index %lld is beyond the supported %lld", dev, kNoAllocMaxDevices);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return noalloc_fail(kErrCuda, "lvb_sumsq_noalloc: cudaGetSymbolAddress failed with CUDA error %lld", static_cast<long long>(e));
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return kErrOk;
}

}  // namespace optim
}  // namespace lvb

extern "C" long long lvb_sumsq_noalloc_max_elems(void) { return lvb::optim::kNoAllocMaxElems; }

extern "C" const char* lvb_sumsq_noalloc_last_error(void) { return lvb::optim::g_noalloc_err; }

extern "C" int lvb_sumsq_noalloc(const void* x, long long n, int is_bf16, float* out, int accumulate, void* stream) {
  using namespace lvb;
  using namespace lvb::optim;
  g_noalloc_err[0] = '\0';
  if (x == nullptr || out == nullptr) return noalloc_fail(kErrBadArg, "lvb_sumsq_noalloc: null pointer argument");
  if (n <= 0) return noalloc_fail(kErrBadArg, "lvb_sumsq_noalloc: n = %lld must be positive", n);
  if (n > kNoAllocMaxElems)
    return noalloc_fail(kErrTooLarge, "lvb_sumsq_noalloc: n = %lld exceeds the maximum of %lld elements", n, kNoAllocMaxElems);
  float* scratch = nullptr;
  int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc != kErrOk) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(n);
  if (cudaMemsetAsync(scratch, 0, sizeof(float) * grid, s) != cudaSuccess)
    return noalloc_fail(kErrCuda, "lvb_sumsq_noalloc: clearing the scratch failed");
  if (is_bf16)
    sumsq_partial_kernel<__nv_bfloat16><<<grid, kBlock, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), n, scratch);
  else
    sumsq_partial_kernel<float><<<grid, kBlock, 0, s>>>(reinterpret_cast<const float*>(x), n, scratch);
  sumsq_final_kernel<<<1, 32, 0, s>>>(scratch, grid, out, accumulate);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return noalloc_fail(kErrCuda, "lvb_sumsq_noalloc: launch failed with CUDA error %lld", static_cast<long long>(e));
  return kErrOk;
}
