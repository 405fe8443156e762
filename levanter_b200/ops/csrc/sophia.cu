// Sophia's parameter-wise update in one pass (src/levanter/optim/sophia.py:341-353 in the reference):
//
//   mu   <- b1 mu + (1 - b1) g
//   u     = clip(mu / (1 - b1^t) / max(gamma h, eps), +-rho)
//
// together with the four statistics the optimizer logs every step (sums of squares of the bias-corrected momentum, of the
// Hessian estimate and of the parameters, and the number of entries that were not clipped), so that the optimizer reads
// each of its state tensors once per step instead of once per statistic.
#include "common.cuh"

namespace lvb {
namespace sophia {

__global__ void sophia_update_kernel(const float* __restrict__ g, float* __restrict__ mu, const float* __restrict__ h,
                                     const float* __restrict__ param, float* __restrict__ u, long long n, float b1, float inv_bc1,
                                     float gamma, float eps, float rho, float* __restrict__ stats) {
  float s_mom = 0.f, s_h = 0.f, s_p = 0.f, s_unclipped = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float m = b1 * mu[i] + (1.f - b1) * g[i];
    mu[i] = m;
    const float mh = m * inv_bc1;
    const float hv = h[i];
    float v = mh / fmaxf(gamma * hv, eps);
    if (rho > 0.f) {
      s_unclipped += (fabsf(v) < rho) ? 1.f : 0.f;
      v = fminf(fmaxf(v, -rho), rho);
    }
    u[i] = v;
    s_mom += mh * mh;
    s_h += hv * hv;
    if (param != nullptr) {
      const float pv = param[i];
      s_p += pv * pv;
    }
  }
  s_mom = warp_sum(s_mom);
  s_h = warp_sum(s_h);
  s_p = warp_sum(s_p);
  s_unclipped = warp_sum(s_unclipped);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(stats + 0, s_mom);
    atomicAdd(stats + 1, s_h);
    atomicAdd(stats + 2, s_p);
    atomicAdd(stats + 3, s_unclipped);
  }
}

}  // namespace sophia
}  // namespace lvb

// fp32 tensors of n elements; `param` may be null; rho <= 0 disables clipping; stats: float[4] that the caller zeroes (sums of
// squares of the bias-corrected momentum, the Hessian estimate, the parameters, and the count of unclipped entries are added).
extern "C" int lvb_sophia_update(const float* g, float* mu, const float* h, const float* param, float* u, long long n, float b1,
                                 float bias_correction1, float gamma, float eps, float rho, float* stats, void* stream) {
  using namespace lvb;
  if (n <= 0 || stats == nullptr) return kErrBadArg;
  long long blocks = (n + 255) / 256;
  const long long cap = 8ll * num_sms();
  if (blocks > cap) blocks = cap;
  sophia::sophia_update_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      g, mu, h, param, u, n, b1, 1.f / bias_correction1, gamma, eps, rho, stats);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
