// Causal long convolution along the sequence, one filter per channel (the Hyena operator's long filter):
//
//   y[n, t, c] = sum_{s <= t} k[s, c] * u[n, t - s, c]  (+ bias[c])
//
// The reference computes it with zero-padded FFTs of size 2L in fp32 (src/levanter/models/hyena.py:326-339).  For the
// sequence lengths that fit in shared memory (L <= 4096) the direct sum costs L^2 / 2 multiply-adds per (sequence, channel),
// which a B200 does faster than three FFT passes move the data, and it is exact in fp32: one CTA holds a tile of channels
// of one sequence (u and k as bf16 in shared memory, channel-minor), every thread owns one channel and every
// (256 / channels)-th output position, so the triangular work is balanced across the threads.
// The same loop gives the gradients: with kRevIn / kRevOut the input and output are indexed from the end of the sequence
// (du = reverse(conv(reverse(dy), k))), and with kCorr it correlates two sequences (dk[s] = sum_t u[t - s] dy[t]) and writes
// one partial per sequence, which the caller sums over the batch in a fixed order.
#include "common.cuh"

namespace lvb {
namespace lconv {

constexpr int kThreads = 256;

// MODE 0: out[t] = sum_{s<=t} b[s] a[t-s]           (a = u or reversed dy, b = k)
// MODE 1: out[s] = sum_{t>=s} a[t-s] b[t]            (a = u, b = dy; correlation, fp32 partial per sequence)
template <int CT, int MODE>
__global__ void __launch_bounds__(kThreads) long_conv_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                                             const float* __restrict__ bias, void* __restrict__ out, int L, int C,
                                                             int rev_in, int rev_out, int b_per_seq, int out_f32) {
  extern __shared__ __nv_bfloat16 sm[];
  __nv_bfloat16* sa = sm;           // [L][CT]
  __nv_bfloat16* sb = sm + L * CT;  // [L][CT]
  const int n = blockIdx.y;
  const int c0 = blockIdx.x * CT;
  const int cl = threadIdx.x % CT;
  const int tg = threadIdx.x / CT;
  constexpr int TG = kThreads / CT;
  const size_t seq_off = static_cast<size_t>(n) * L * C;
  for (int i = threadIdx.x; i < L * CT; i += kThreads) {
    const int t = i / CT, c = i % CT;
    const bool ok = c0 + c < C;
    const int ta = rev_in ? (L - 1 - t) : t;
    sa[i] = ok ? a[seq_off + static_cast<size_t>(ta) * C + c0 + c] : __float2bfloat16(0.f);
    const int tb = (rev_in && b_per_seq) ? (L - 1 - t) : t;
    sb[i] = ok ? b[(b_per_seq ? seq_off : 0) + static_cast<size_t>(tb) * C + c0 + c] : __float2bfloat16(0.f);
  }
  __syncthreads();
  if (c0 + cl >= C) return;
  const float bv = (bias != nullptr) ? bias[c0 + cl] : 0.f;
  for (int t = tg; t < L; t += TG) {
    float acc0 = 0.f, acc1 = 0.f;
    if constexpr (MODE == 0) {
      int s = 0;
      for (; s + 1 <= t; s += 2) {
        acc0 = fmaf(__bfloat162float(sb[s * CT + cl]), __bfloat162float(sa[(t - s) * CT + cl]), acc0);
        acc1 = fmaf(__bfloat162float(sb[(s + 1) * CT + cl]), __bfloat162float(sa[(t - s - 1) * CT + cl]), acc1);
      }
      if (s <= t) acc0 = fmaf(__bfloat162float(sb[s * CT + cl]), __bfloat162float(sa[(t - s) * CT + cl]), acc0);
    } else {
      // here `t` plays the role of the lag s: out[s] = sum_{j >= s} a[j - s] b[j]
      int j = t;
      for (; j + 1 < L; j += 2) {
        acc0 = fmaf(__bfloat162float(sa[(j - t) * CT + cl]), __bfloat162float(sb[j * CT + cl]), acc0);
        acc1 = fmaf(__bfloat162float(sa[(j + 1 - t) * CT + cl]), __bfloat162float(sb[(j + 1) * CT + cl]), acc1);
      }
      if (j < L) acc0 = fmaf(__bfloat162float(sa[(j - t) * CT + cl]), __bfloat162float(sb[j * CT + cl]), acc0);
    }
    const float r = acc0 + acc1 + bv;
    const int to = rev_out ? (L - 1 - t) : t;
    const size_t o = seq_off + static_cast<size_t>(to) * C + c0 + cl;
    if (out_f32) reinterpret_cast<float*>(out)[o] = r;
    else reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16(r);
  }
}

template <int MODE>
int launch(const void* a, const void* b, const float* bias, void* out, int N, int L, int C, int rev_in, int rev_out, int b_per_seq,
           int out_f32, cudaStream_t stream) {
  const int ct = L <= 1024 ? 32 : (L <= 2048 ? 16 : 8);
  const int smem = 2 * L * ct * 2;
  dim3 grid((C + ct - 1) / ct, N);
#define LVB_LC(CT)                                                                                                        \
  do {                                                                                                                    \
    auto kern = long_conv_kernel<CT, MODE>;                                                                               \
    static bool attr_set = false;                                                                                         \
    if (!attr_set) {                                                                                                      \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 4096 * 8 * 2) != cudaSuccess)       \
        return kErrCuda;                                                                                                  \
      attr_set = true;                                                                                                    \
    }                                                                                                                     \
    kern<<<grid, kThreads, smem, stream>>>(reinterpret_cast<const __nv_bfloat16*>(a), reinterpret_cast<const __nv_bfloat16*>(b), bias, out, L, \
                                           C, rev_in, rev_out, b_per_seq, out_f32);                                        \
  } while (0)
  if (ct == 32) LVB_LC(32);
  else if (ct == 16) LVB_LC(16);
  else LVB_LC(8);
#undef LVB_LC
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace lconv
}  // namespace lvb

// y[N, L, C] = causal_conv(u[N, L, C], k[L, C]) (+ bias[C], fp32, may be null); bf16 in, bf16 or fp32 out; L <= 4096.
// reverse != 0 computes reverse(conv(reverse(u), k)) along L instead: the input gradient of the forward form.
extern "C" int lvb_long_conv(const void* u, const void* k, const float* bias, void* y, int N, int L, int C, int reverse, int out_f32,
                             void* stream) {
  using namespace lvb;
  if (N <= 0 || L <= 0 || L > 4096 || C <= 0) return kErrBadArg;
  return lconv::launch<0>(u, k, bias, y, N, L, C, reverse ? 1 : 0, reverse ? 1 : 0, 0, out_f32, reinterpret_cast<cudaStream_t>(stream));
}

// dk_partial[N, L, C] (fp32): dk_partial[n, s, c] = sum_{t >= s} u[n, t - s, c] * dy[n, t, c]; the filter gradient is its sum over n.
extern "C" int lvb_long_conv_filter_grad(const void* u, const void* dy, float* dk_partial, int N, int L, int C, void* stream) {
  using namespace lvb;
  if (N <= 0 || L <= 0 || L > 4096 || C <= 0) return kErrBadArg;
  return lconv::launch<1>(u, dy, nullptr, dk_partial, N, L, C, 0, 0, 1, 1, reinterpret_cast<cudaStream_t>(stream));
}
