// Dropout with a counter-based generator, optionally fused with a residual add.
//
//   out[i] = (residual ? residual[i] : 0) + keep(i) * x[i] / (1 - p),   keep(i) = [philox(seed, i) >= p]
//
// The mask is a pure function of (seed, element index): nothing is stored for the backward pass, which applies the same
// kernel to the output gradient with the same seed.  Replaces hnn.Dropout's mask generation and multiply
// (e.g. src/levanter/models/gpt2.py:232,297), which the reference keys per layer from the step's PRNG key.
#include "common.cuh"

namespace lvb {
namespace drop {

__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// 8 elements per thread and step: two generator calls give the eight 32-bit draws.
__global__ void dropout_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                               long long n8, uint32_t threshold, float inv_keep, uint2 key) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 r0 = philox4x32_10(make_uint4(static_cast<uint32_t>(i), static_cast<uint32_t>(i >> 32), 0u, 0u), key);
    const uint4 r1 = philox4x32_10(make_uint4(static_cast<uint32_t>(i), static_cast<uint32_t>(i >> 32), 1u, 0u), key);
    const uint32_t rnd[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(x) + i);
    uint4 rs = make_uint4(0, 0, 0, 0);
    if (residual != nullptr) rs = __ldg(reinterpret_cast<const uint4*>(residual) + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
    const __nv_bfloat162* hr = reinterpret_cast<const __nv_bfloat162*>(&rs);
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = __bfloat1622float2(h[q]);
      const float2 g = __bfloat1622float2(hr[q]);
      const float a = (rnd[2 * q] >= threshold ? f.x * inv_keep : 0.f) + g.x;
      const float b = (rnd[2 * q + 1] >= threshold ? f.y * inv_keep : 0.f) + g.y;
      o[q] = pack_bf16x2(a, b);
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace drop
}  // namespace lvb

// out = residual + dropout(x); bf16, n a multiple of 8, pointers 16-byte aligned; residual may be null; out may alias x.
// p in [0, 1): the probability of dropping an element.  (seed_lo, seed_hi) selects the mask.
extern "C" int lvb_dropout(const void* x, const void* residual, void* out, long long n, float p, unsigned seed_lo, unsigned seed_hi,
                           void* stream) {
  using namespace lvb;
  if (n <= 0 || (n & 7) || p < 0.f || p >= 1.f) return kErrBadArg;
  const long long n8 = n >> 3;
  const double thr = static_cast<double>(p) * 4294967296.0;
  const uint32_t threshold = thr >= 4294967295.0 ? 4294967295u : static_cast<uint32_t>(thr);
  long long blocks = (n8 + 255) / 256;
  const long long cap = 16ll * num_sms();
  if (blocks > cap) blocks = cap;
  drop::dropout_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<__nv_bfloat16*>(out), n8,
      threshold, 1.f / (1.f - p), make_uint2(seed_lo, seed_hi));
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
