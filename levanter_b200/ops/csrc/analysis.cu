// One-pass kernels behind the logging and analysis hooks.
//
//  * tensor_summary + histogram: min, max, sum, sum of squares and element count of a tensor in one read, then equal-width
//    bin counts in a second read whose range comes from the first kernel's result in device memory (the host reads one small
//    record at the end).  The reference bins by comparing every element with every edge and sums the counts over the mesh
//    (src/levanter/tracker/histogram.py:92-142).
//  * entropy_top2: per row of logits, the predictive entropy H = lse - sum(p * z) and the gap between the two largest logits
//    in a single streaming pass with online rescaling (the reference materialises softmax and runs two argmax passes,
//    src/levanter/analysis/entropy.py:31-63,101-106).
// Sums are reduced per block and then in block order, so results do not depend on scheduling; bin counts are integers.
#include "common.cuh"
#include <cuda_bf16.h>

namespace lvb {
namespace analysis {

constexpr int kBlock = 256;
constexpr int kMaxBlocks = 1024;
constexpr int kMaxBins = 256;

template <bool BF16>
__device__ __forceinline__ float load_elem(const void* x, long long i) {
  if (BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(x)[i]);
  return static_cast<const float*>(x)[i];
}

// partial[b] = {min, max, sum, sumsq} of block b's elements
template <bool BF16>
__global__ void __launch_bounds__(kBlock) summary_partial_kernel(const void* __restrict__ x, long long n, float4* __restrict__ partial) {
  float mn = INFINITY, mx = -INFINITY, s = 0.f, ss = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * kBlock) {
    const float v = load_elem<BF16>(x, i);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
    s += v;
    ss = fmaf(v, v, ss);
  }
  __shared__ float4 red[kBlock / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    s += __shfl_xor_sync(0xffffffffu, s, o);
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = make_float4(mn, mx, s, ss);
  __syncthreads();
  if (threadIdx.x == 0) {
    float4 r = red[0];
    for (int w = 1; w < kBlock / 32; ++w) {
      r.x = fminf(r.x, red[w].x);
      r.y = fmaxf(r.y, red[w].y);
      r.z += red[w].z;
      r.w += red[w].w;
    }
    partial[blockIdx.x] = r;
  }
}

// out = {min, max, sum, sumsq}; blocks are folded in order by one thread (at most kMaxBlocks of them)
__global__ void summary_final_kernel(const float4* __restrict__ partial, int blocks, float* __restrict__ out) {
  float4 r = partial[0];
  for (int b = 1; b < blocks; ++b) {
    r.x = fminf(r.x, partial[b].x);
    r.y = fmaxf(r.y, partial[b].y);
    r.z += partial[b].z;
    r.w += partial[b].w;
  }
  out[0] = r.x;
  out[1] = r.y;
  out[2] = r.z;
  out[3] = r.w;
}

// counts[bin] += #elements with lo <= v <= hi falling in the bin; range = {lo, hi} in device memory (hi <= lo means width 1)
template <bool BF16>
__global__ void __launch_bounds__(kBlock)
histogram_kernel(const void* __restrict__ x, long long n, const float* __restrict__ range, int bins, int* __restrict__ counts) {
  __shared__ int s_cnt[kMaxBins];
  for (int b = threadIdx.x; b < bins; b += kBlock) s_cnt[b] = 0;
  __syncthreads();
  const float lo = range[0];
  const float hi = range[1] > lo ? range[1] : lo + 1.f;
  const float width = hi - lo;
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * kBlock) {
    const float v = load_elem<BF16>(x, i);
    if (v >= lo && v <= hi) {
      int b = static_cast<int>(floorf(__fmul_rn(__fdiv_rn(v - lo, width), static_cast<float>(bins))));  // same rounding as the host formula
      b = b < 0 ? 0 : (b >= bins ? bins - 1 : b);
      atomicAdd(&s_cnt[b], 1);
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < bins; b += kBlock)
    if (s_cnt[b]) atomicAdd(&counts[b], s_cnt[b]);
}

struct RowStat {
  float m, z, s;  // running max, sum exp(v - m), sum exp(v - m) * v
  float a, b;     // largest and second largest value
};

__device__ __forceinline__ void stat_add(RowStat& r, float v) {
  if (v == -INFINITY) {  // a masked logit: probability zero, and it can only ever be the second largest of a masked row
  } else if (v > r.m) {
    const float c = __expf(r.m - v);  // 0 on the first element (m = -inf)
    r.z = r.z * c + 1.f;
    r.s = r.s * c + v;
    r.m = v;
  } else {
    const float e = __expf(v - r.m);
    r.z += e;
    r.s = fmaf(e, v, r.s);
  }
  if (v > r.a) {
    r.b = r.a;
    r.a = v;
  } else if (v > r.b) {
    r.b = v;
  }
}

__device__ __forceinline__ RowStat stat_merge(const RowStat& x, const RowStat& y) {
  RowStat r;
  r.m = fmaxf(x.m, y.m);
  const float cx = x.m == -INFINITY ? 0.f : __expf(x.m - r.m);
  const float cy = y.m == -INFINITY ? 0.f : __expf(y.m - r.m);
  r.z = x.z * cx + y.z * cy;
  r.s = x.s * cx + y.s * cy;
  r.a = fmaxf(x.a, y.a);
  r.b = fmaxf(fminf(x.a, y.a), fmaxf(x.b, y.b));
  return r;
}

__device__ __forceinline__ RowStat stat_shfl_xor(const RowStat& x, int o) {
  RowStat y;
  y.m = __shfl_xor_sync(0xffffffffu, x.m, o);
  y.z = __shfl_xor_sync(0xffffffffu, x.z, o);
  y.s = __shfl_xor_sync(0xffffffffu, x.s, o);
  y.a = __shfl_xor_sync(0xffffffffu, x.a, o);
  y.b = __shfl_xor_sync(0xffffffffu, x.b, o);
  return y;
}

// one block per row: entropy[row] = lse - sum(p z), gap[row] = top1 - top2, lse_out[row] (each may be null)
template <bool BF16>
__global__ void __launch_bounds__(kBlock)
entropy_top2_kernel(const void* __restrict__ logits, int V, long long ld, float* __restrict__ entropy, float* __restrict__ gap,
                    float* __restrict__ lse_out) {
  const long long row = blockIdx.x;
  RowStat r{-INFINITY, 0.f, 0.f, -INFINITY, -INFINITY};
  if (BF16 && (V % 8 == 0) && (ld % 8 == 0)) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(logits) + row * ld);
    for (int i = threadIdx.x; i < V / 8; i += kBlock) {
      const uint4 q = __ldg(p + i);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      float v[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
      // eight values at once: one rescale of the running sums to the new maximum, then branch-free accumulation
      float m8 = v[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) m8 = fmaxf(m8, v[j]);
      if (m8 > r.m) {
        const float c = __expf(r.m - m8);  // 0 while the running maximum is still -inf
        r.z *= c;
        r.s *= c;
        r.m = m8;
      }
      if (r.m != -INFINITY) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float e = __expf(v[j] - r.m);  // exp(-inf) = 0 for masked logits
          r.z += e;
          r.s = fmaf(e, v[j] == -INFINITY ? 0.f : v[j], r.s);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {  // top two without branches
        r.b = fmaxf(r.b, fminf(r.a, v[j]));
        r.a = fmaxf(r.a, v[j]);
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += kBlock) stat_add(r, load_elem<BF16>(logits, row * ld + i));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = stat_merge(r, stat_shfl_xor(r, o));
  __shared__ RowStat red[kBlock / 32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = r;
  __syncthreads();
  if (threadIdx.x == 0) {
    RowStat t = red[0];
    for (int w = 1; w < kBlock / 32; ++w) t = stat_merge(t, red[w]);
    const float lse = t.m + __logf(t.z);
    if (entropy) entropy[row] = lse - t.s / t.z;
    if (gap) gap[row] = t.a - t.b;
    if (lse_out) lse_out[row] = lse;
  }
}

}  // namespace analysis
}  // namespace lvb

using namespace lvb;

// summary[4] = {min, max, sum, sum of squares} of x[n] (fp32 or bf16); scratch: 16 KB (1024 float4) on the same device.
extern "C" int lvb_tensor_summary(const void* x, long long n, int is_bf16, void* scratch, float* summary, void* stream) {
  if (n <= 0) return kErrBadArg;
  auto s = static_cast<cudaStream_t>(stream);
  long long want = (n + analysis::kBlock * 8 - 1) / (analysis::kBlock * 8);
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > analysis::kMaxBlocks ? analysis::kMaxBlocks : want));
  if (is_bf16)
    analysis::summary_partial_kernel<true><<<blocks, analysis::kBlock, 0, s>>>(x, n, static_cast<float4*>(scratch));
  else
    analysis::summary_partial_kernel<false><<<blocks, analysis::kBlock, 0, s>>>(x, n, static_cast<float4*>(scratch));
  analysis::summary_final_kernel<<<1, 1, 0, s>>>(static_cast<const float4*>(scratch), blocks, summary);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// counts[bins] (int32, zeroed by the caller) += bin counts of x over range[2] = {lo, hi} read on the device; bins <= 256.
extern "C" int lvb_histogram(const void* x, long long n, int is_bf16, const float* range, int bins, int* counts, void* stream) {
  if (n <= 0 || bins < 1 || bins > analysis::kMaxBins) return kErrBadArg;
  auto s = static_cast<cudaStream_t>(stream);
  long long want = (n + analysis::kBlock * 8 - 1) / (analysis::kBlock * 8);
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want));
  if (is_bf16)
    analysis::histogram_kernel<true><<<blocks, analysis::kBlock, 0, s>>>(x, n, range, bins, counts);
  else
    analysis::histogram_kernel<false><<<blocks, analysis::kBlock, 0, s>>>(x, n, range, bins, counts);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// logits [rows, V] with row stride ld (elements), fp32 or bf16; every output [rows] fp32 or null.
extern "C" int lvb_entropy_top2(const void* logits, int rows, int V, long long ld, int is_bf16, float* entropy, float* gap, float* lse,
                                void* stream) {
  if (rows <= 0 || V < 2 || ld < V) return kErrBadArg;
  auto s = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    analysis::entropy_top2_kernel<true><<<rows, analysis::kBlock, 0, s>>>(logits, V, ld, entropy, gap, lse);
  else
    analysis::entropy_top2_kernel<false><<<rows, analysis::kBlock, 0, s>>>(logits, V, ld, entropy, gap, lse);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
