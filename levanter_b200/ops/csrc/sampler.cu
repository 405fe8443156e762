// Token sampling: per row, greedy arg-max when the temperature is 0, otherwise a categorical draw from softmax(z / T) by
// the Gumbel-max trick, plus the log-probability of the chosen token (src/levanter/layers/sampler.py:35-81).
//
// One CTA per row makes a single pass over the vocabulary: each thread keeps an online log-sum-exp (running max, scaled
// sum), the best perturbed score z/T + g and the best raw score; the noise g = -log(-log(u)) comes from a counter-based
// hash of (row seed, vocabulary index), so a row's draw depends only on its own seed, never on what else is in the batch.
// Ties go to the lower index, which keeps the result independent of the block size.
#include "common.cuh"

namespace lvb {
namespace sampler {

constexpr int kThreads = 256;

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ float gumbel(unsigned long long seed, int idx) {
  const unsigned long long h = mix64(seed ^ (static_cast<unsigned long long>(idx) * 0x9E3779B97F4A7C15ull));
  const float u = (static_cast<float>(h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
  return -__logf(-__logf(u));
}

struct Acc {
  float m, s;        // online log-sum-exp of z / T
  float best;        // best perturbed score
  int best_idx;
  float zbest;       // z / T at best_idx
};

__device__ __forceinline__ void merge(Acc& a, const Acc& b) {
  const float m = fmaxf(a.m, b.m);
  a.s = (a.m == -INFINITY ? 0.f : a.s * __expf(a.m - m)) + (b.m == -INFINITY ? 0.f : b.s * __expf(b.m - m));
  a.m = m;
  if (b.best > a.best || (b.best == a.best && b.best_idx < a.best_idx)) {
    a.best = b.best;
    a.best_idx = b.best_idx;
    a.zbest = b.zbest;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) sample_kernel(const T* __restrict__ logits, long long row_stride, int vocab,
                                                          const float* __restrict__ temps, const long long* __restrict__ seeds,
                                                          int* __restrict__ tokens, float* __restrict__ logprobs) {
  const int row = blockIdx.x;
  const T* z = logits + static_cast<long long>(row) * row_stride;
  const float t = temps[row];
  const bool greedy = (t == 0.f);
  const float inv_t = greedy ? 1.f : 1.f / t;
  const unsigned long long seed = static_cast<unsigned long long>(seeds[row]);
  Acc a{-INFINITY, 0.f, -INFINITY, 0x7fffffff, 0.f};
  auto visit = [&](float v, int i) {
    v *= inv_t;
    if (v > a.m) { a.s = a.s * __expf(a.m - v) + 1.f; a.m = v; }
    else if (v > -INFINITY) a.s += __expf(v - a.m);
    const float score = greedy ? v : v + gumbel(seed, i);
    if (score > a.best) { a.best = score; a.best_idx = i; a.zbest = v; }
  };
  int done = 0;
  if constexpr (sizeof(T) == 2) {
    // 16-byte loads (8 logits) when the row starts on a 16-byte boundary
    if ((reinterpret_cast<uintptr_t>(z) & 15) == 0) {
      const int nvec = vocab / 8;
      const uint4* zv = reinterpret_cast<const uint4*>(z);
      for (int c = threadIdx.x; c < nvec; c += kThreads) {
        const uint4 w = zv[c];
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&u[j]);
          visit(__low2float(h), c * 8 + 2 * j);
          visit(__high2float(h), c * 8 + 2 * j + 1);
        }
      }
      done = nvec * 8;
    }
  }
  for (int i = done + threadIdx.x; i < vocab; i += kThreads) {
    float v;
    if constexpr (sizeof(T) == 2) v = __bfloat162float(z[i]); else v = z[i];
    visit(v, i);
  }
  __shared__ Acc sm[kThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Acc b;
    b.m = __shfl_xor_sync(0xffffffffu, a.m, o);
    b.s = __shfl_xor_sync(0xffffffffu, a.s, o);
    b.best = __shfl_xor_sync(0xffffffffu, a.best, o);
    b.best_idx = __shfl_xor_sync(0xffffffffu, a.best_idx, o);
    b.zbest = __shfl_xor_sync(0xffffffffu, a.zbest, o);
    merge(a, b);
  }
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    Acc r = sm[0];
    for (int w = 1; w < kThreads / 32; ++w) merge(r, sm[w]);
    tokens[row] = r.best_idx;
    logprobs[row] = r.zbest - (r.m + __logf(r.s));
  }
}

}  // namespace sampler
}  // namespace lvb

// logits: [rows, vocab] fp32 (is_bf16 = 0) or bf16 with row stride `row_stride` elements; temps fp32 [rows];
// seeds int64 [rows]; tokens int32 [rows]; logprobs fp32 [rows].
extern "C" int lvb_sample(const void* logits, int is_bf16, long long row_stride, int rows, int vocab, const float* temps,
                          const long long* seeds, int* tokens, float* logprobs, void* stream) {
  using namespace lvb;
  using namespace lvb::sampler;
  if (rows <= 0 || vocab <= 0) return kErrBadArg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<rows, kThreads, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), row_stride, vocab,
                                                           temps, seeds, tokens, logprobs);
  else
    sample_kernel<float><<<rows, kThreads, 0, s>>>(reinterpret_cast<const float*>(logits), row_stride, vocab, temps, seeds,
                                                   tokens, logprobs);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
