// Mixture-of-experts routing in one pass per direction: softmax over the experts, top-k, renormalised top-k weights,
// tokens per expert, the per-expert probability sums (load-balancing loss) and the log-sum-exp (router z-loss)
// (the reference computes these with separate XLA ops, src/levanter/models/mixtral.py:336-347,423-468).
// One thread per token; experts <= 64.  The probability sums are reduced per block and then in a fixed order by a second
// kernel, so the result does not depend on scheduling.
#include "common.cuh"

namespace lvb {
namespace moe {

constexpr int kMaxExperts = 64;
constexpr int kMaxTopK = 8;
constexpr int kBlock = 128;

__global__ void __launch_bounds__(kBlock)
route_fwd_kernel(const float* __restrict__ logits, int T, int E, int k, int* __restrict__ topk_idx, float* __restrict__ topk_w,
                 float* __restrict__ probs, float* __restrict__ lse, int* __restrict__ counts, float* __restrict__ psum_partial) {
  __shared__ float s_psum[kBlock / 32][kMaxExperts];  // one row per warp, summed in warp order below
  __shared__ int s_cnt[kMaxExperts];
  for (int e = threadIdx.x; e < E; e += kBlock) s_cnt[e] = 0;
  __syncthreads();
  const int t = blockIdx.x * kBlock + threadIdx.x;
  float p[kMaxExperts];
  for (int e = 0; e < E; ++e) p[e] = 0.f;
  if (t < T) {
    const float* z = logits + static_cast<size_t>(t) * E;
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) { p[e] = z[e]; mx = fmaxf(mx, p[e]); }
    float sum = 0.f;
    for (int e = 0; e < E; ++e) { p[e] = __expf(p[e] - mx); sum += p[e]; }
    const float inv = 1.f / sum;
    lse[t] = mx + __logf(sum);
    for (int e = 0; e < E; ++e) {
      p[e] *= inv;
      probs[static_cast<size_t>(t) * E + e] = p[e];
    }
    // top-k by repeated selection (k <= 8, E <= 64); ties go to the lower expert index
    unsigned long long taken = 0ull;
    int idx[kMaxTopK];
    float w[kMaxTopK];
    float wsum = 0.f;
    for (int j = 0; j < k; ++j) {
      int best = -1;
      float bv = -1.f;
      for (int e = 0; e < E; ++e)
        if (!((taken >> e) & 1ull) && p[e] > bv) { bv = p[e]; best = e; }
      taken |= 1ull << best;
      idx[j] = best;
      w[j] = bv;
      wsum += bv;
    }
    for (int j = 0; j < k; ++j) {
      topk_idx[static_cast<size_t>(t) * k + j] = idx[j];
      topk_w[static_cast<size_t>(t) * k + j] = w[j] / wsum;
      atomicAdd(&s_cnt[idx[j]], 1);
    }
  }
  // probability sums: butterfly within the warp, then the warps in order, then (second kernel) the blocks in order
  for (int e = 0; e < E; ++e) {
    float v = p[e];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) s_psum[threadIdx.x >> 5][e] = v;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kBlock) {
    float v = 0.f;
    for (int w = 0; w < kBlock / 32; ++w) v += s_psum[w][e];
    psum_partial[static_cast<size_t>(blockIdx.x) * E + e] = v;
    if (s_cnt[e]) atomicAdd(&counts[e], s_cnt[e]);
  }
}

__global__ void psum_reduce_kernel(const float* __restrict__ partial, int blocks, int E, float* __restrict__ psum) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[static_cast<size_t>(b) * E + e];
  psum[e] = s;
}

// dlogits from the gradients of the renormalised weights, of the probability sums and of the log-sum-exp
__global__ void __launch_bounds__(kBlock)
route_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ topk_idx, const float* __restrict__ d_w,
                 const float* __restrict__ d_psum, const float* __restrict__ d_lse, int T, int E, int k, float* __restrict__ dlogits) {
  const int t = blockIdx.x * kBlock + threadIdx.x;
  if (t >= T) return;
  float p[kMaxExperts], dp[kMaxExperts];
  for (int e = 0; e < E; ++e) {
    p[e] = probs[static_cast<size_t>(t) * E + e];
    dp[e] = d_psum != nullptr ? d_psum[e] : 0.f;
  }
  if (d_w != nullptr) {
    float s = 0.f, dot = 0.f;
    for (int j = 0; j < k; ++j) s += p[topk_idx[static_cast<size_t>(t) * k + j]];
    for (int j = 0; j < k; ++j) {
      const int e = topk_idx[static_cast<size_t>(t) * k + j];
      dot += d_w[static_cast<size_t>(t) * k + j] * (p[e] / s);
    }
    for (int j = 0; j < k; ++j) {
      const int e = topk_idx[static_cast<size_t>(t) * k + j];
      dp[e] += (d_w[static_cast<size_t>(t) * k + j] - dot) / s;
    }
  }
  float pd = 0.f;
  for (int e = 0; e < E; ++e) pd += p[e] * dp[e];
  const float dl = d_lse != nullptr ? d_lse[t] : 0.f;
  for (int e = 0; e < E; ++e) dlogits[static_cast<size_t>(t) * E + e] = p[e] * (dp[e] - pd + dl);
}

}  // namespace moe
}  // namespace lvb

// scratch: at least ceil(T / 128) * E floats.  counts must be zero on entry.
extern "C" int lvb_moe_route_fwd(const float* logits, int T, int E, int k, int* topk_idx, float* topk_w, float* probs, float* lse,
                                 int* counts, float* psum, float* scratch, void* stream) {
  using namespace lvb;
  using namespace lvb::moe;
  if (T <= 0 || E <= 0 || E > kMaxExperts || k <= 0 || k > kMaxTopK || k > E) return kErrBadArg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int blocks = (T + kBlock - 1) / kBlock;
  route_fwd_kernel<<<blocks, kBlock, 0, s>>>(logits, T, E, k, topk_idx, topk_w, probs, lse, counts, scratch);
  psum_reduce_kernel<<<1, 64, 0, s>>>(scratch, blocks, E, psum);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

extern "C" int lvb_moe_route_bwd(const float* probs, const int* topk_idx, const float* d_w, const float* d_psum, const float* d_lse,
                                 int T, int E, int k, float* dlogits, void* stream) {
  using namespace lvb;
  using namespace lvb::moe;
  if (T <= 0 || E <= 0 || E > kMaxExperts || k <= 0 || k > kMaxTopK) return kErrBadArg;
  route_bwd_kernel<<<(T + kBlock - 1) / kBlock, kBlock, 0, reinterpret_cast<cudaStream_t>(stream)>>>(probs, topk_idx, d_w, d_psum,
                                                                                                   d_lse, T, E, k, dlogits);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
