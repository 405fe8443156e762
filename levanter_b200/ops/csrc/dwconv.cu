// Depthwise causal 1-D convolution over channel-last activations, y[b, l, c] = act(bias[c] + sum_j w[c, j] x[b, l-(K-1)+j, c]),
// with K in {2, 3, 4}: the short input filter of the Hyena operator (src/levanter/models/hyena.py:474-482,514-518: k = 3,
// padded by k-1 and truncated, i.e. causal) and the q/k/v convolutions (k = 4, SiLU) of the gated delta-rule layer.
//
// The library path is transpose -> conv1d -> slice -> transpose (-> SiLU): four passes over the activations.  Here a thread
// owns 16 bytes of channels (8 bf16 or 4 fp32) and walks a run of positions with the last K-1 inputs in registers, so x is
// read once (plus a K-1 halo per run) and y written once, fully coalesced across channels.  The same kernel run over the
// flipped sequence gives the input gradient.  The weight/bias gradients are accumulated per run in registers, written as
// partial sums and folded in a fixed order by a second kernel (bitwise reproducible).
#include "common.cuh"
#include <cuda_bf16.h>

namespace lvb {
namespace dwconv {

constexpr int kBlock = 128;
constexpr int kRun = 64;     // positions per thread, gradient prologue (its partial sums are written once per run)
constexpr int kRunFwd = 32;  // positions per thread, convolution: shorter runs put more loads in flight

template <bool BF16>
struct Vec {
  static constexpr int N = BF16 ? 8 : 4;
  __device__ static __forceinline__ void load(const void* base, size_t elem, float (&v)[N]) {
    if (BF16) {
      const uint4 q = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + elem);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    } else {
      const float4 q = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem);
      v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
  }
  __device__ static __forceinline__ void store(void* base, size_t elem, const float (&v)[N]) {
    if (BF16) {
      uint4 q;
      q.x = pack_bf16x2(v[0], v[1]); q.y = pack_bf16x2(v[2], v[3]); q.z = pack_bf16x2(v[4], v[5]); q.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + elem) = q;
    } else {
      *reinterpret_cast<float4*>(static_cast<float*>(base) + elem) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
};

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_grad(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// flip != 0 walks the sequence backwards (position l stands for L-1-l), which turns the causal filter into the
// anti-causal one of the input gradient.  grid: (channel vectors / kBlock, runs, batch)
template <bool BF16, int K>
__global__ void __launch_bounds__(kBlock)
conv_kernel(const void* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, void* __restrict__ y, int L, int C,
            int act, int flip) {
  constexpr int N = Vec<BF16>::N;
  const int cv = blockIdx.x * kBlock + threadIdx.x;
  if (cv * N >= C) return;
  const int c0 = cv * N;
  const int l0 = blockIdx.y * kRunFwd;
  const size_t row0 = static_cast<size_t>(blockIdx.z) * L;
  float wr[N][K], br[N], win[K - 1][N];
#pragma unroll
  for (int i = 0; i < N; ++i) {
    br[i] = bias ? bias[c0 + i] : 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) wr[i][j] = w[(c0 + i) * K + j];
  }
  auto pos = [&](int l) { return (row0 + (flip ? L - 1 - l : l)) * C + c0; };
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {  // win[j] = input at l0 - (K-1) + j
    const int l = l0 - (K - 1) + j;
    if (l >= 0) Vec<BF16>::load(x, pos(l), win[j]);
    else
#pragma unroll
      for (int i = 0; i < N; ++i) win[j][i] = 0.f;
  }
  const int l_end = min(l0 + kRunFwd, L);
#pragma unroll 4
  for (int l = l0; l < l_end; ++l) {
    float cur[N], out[N];
    Vec<BF16>::load(x, pos(l), cur);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      float a = fmaf(wr[i][K - 1], cur[i], br[i]);
#pragma unroll
      for (int j = 0; j < K - 1; ++j) a = fmaf(wr[i][j], win[j][i], a);
      out[i] = act ? silu(a) : a;
    }
    Vec<BF16>::store(y, pos(l), out);
#pragma unroll
    for (int j = 0; j + 1 < K - 1; ++j)
#pragma unroll
      for (int i = 0; i < N; ++i) win[j][i] = win[j + 1][i];
#pragma unroll
    for (int i = 0; i < N; ++i) win[K - 2][i] = cur[i];
  }
}

// dpre = dy * act'(pre) (pre recomputed from x) and this run's contribution to dw[c, j] = sum dpre[l] x[l-(K-1)+j] and
// dbias[c] = sum dpre[l], written to partial[(batch * runs + run), c, 0..K] (K weights then the bias).
template <bool BF16, int K>
__global__ void __launch_bounds__(kBlock)
bwd_prep_kernel(const void* __restrict__ x, const void* __restrict__ dy, const float* __restrict__ w, const float* __restrict__ bias,
                void* __restrict__ dpre, float* __restrict__ partial, int L, int C, int act) {
  constexpr int N = Vec<BF16>::N;
  const int cv = blockIdx.x * kBlock + threadIdx.x;
  if (cv * N >= C) return;
  const int c0 = cv * N;
  const int l0 = blockIdx.y * kRun;
  const size_t row0 = static_cast<size_t>(blockIdx.z) * L;
  float wr[N][K], br[N], win[K - 1][N], gw[N][K + 1];
#pragma unroll
  for (int i = 0; i < N; ++i) {
    br[i] = bias ? bias[c0 + i] : 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) wr[i][j] = w[(c0 + i) * K + j];
#pragma unroll
    for (int j = 0; j <= K; ++j) gw[i][j] = 0.f;
  }
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int l = l0 - (K - 1) + j;
    if (l >= 0) Vec<BF16>::load(x, (row0 + l) * C + c0, win[j]);
    else
#pragma unroll
      for (int i = 0; i < N; ++i) win[j][i] = 0.f;
  }
  const int l_end = min(l0 + kRun, L);
#pragma unroll 2
  for (int l = l0; l < l_end; ++l) {
    float cur[N], g[N];
    const size_t at = (row0 + l) * C + c0;
    Vec<BF16>::load(x, at, cur);
    Vec<BF16>::load(dy, at, g);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if (act) {
        float a = fmaf(wr[i][K - 1], cur[i], br[i]);
#pragma unroll
        for (int j = 0; j < K - 1; ++j) a = fmaf(wr[i][j], win[j][i], a);
        g[i] *= silu_grad(a);
      }
      gw[i][K - 1] = fmaf(g[i], cur[i], gw[i][K - 1]);
#pragma unroll
      for (int j = 0; j < K - 1; ++j) gw[i][j] = fmaf(g[i], win[j][i], gw[i][j]);
      gw[i][K] += g[i];
    }
    if (dpre != nullptr) Vec<BF16>::store(dpre, at, g);
#pragma unroll
    for (int j = 0; j + 1 < K - 1; ++j)
#pragma unroll
      for (int i = 0; i < N; ++i) win[j][i] = win[j + 1][i];
#pragma unroll
    for (int i = 0; i < N; ++i) win[K - 2][i] = cur[i];
  }
  float* out = partial + (static_cast<size_t>(blockIdx.z) * gridDim.y + blockIdx.y) * C * (K + 1);
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int j = 0; j <= K; ++j) out[(c0 + i) * (K + 1) + j] = gw[i][j];
}

// dw[c, j] and dbias[c] from the partial sums, folded in order of (batch, run)
__global__ void bwd_reduce_kernel(const float* __restrict__ partial, int parts, int C, int K, float* __restrict__ dw, float* __restrict__ dbias) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;  // over C * (K + 1)
  if (i >= C * (K + 1)) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<size_t>(p) * C * (K + 1) + i];
  const int c = i / (K + 1), j = i - c * (K + 1);
  if (j < K) dw[c * K + j] = s;
  else if (dbias != nullptr) dbias[c] = s;
}

template <bool BF16, int K>
int launch_conv(const void* x, const float* w, const float* bias, void* y, int B, int L, int C, int act, int flip, cudaStream_t s) {
  constexpr int N = Vec<BF16>::N;
  dim3 grid((C / N + kBlock - 1) / kBlock, (L + kRunFwd - 1) / kRunFwd, B);
  conv_kernel<BF16, K><<<grid, kBlock, 0, s>>>(x, w, bias, y, L, C, act, flip);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

template <bool BF16, int K>
int launch_prep(const void* x, const void* dy, const float* w, const float* bias, void* dpre, float* partial, float* dw, float* dbias,
                int B, int L, int C, int act, cudaStream_t s) {
  constexpr int N = Vec<BF16>::N;
  dim3 grid((C / N + kBlock - 1) / kBlock, (L + kRun - 1) / kRun, B);
  bwd_prep_kernel<BF16, K><<<grid, kBlock, 0, s>>>(x, dy, w, bias, dpre, partial, L, C, act);
  const int total = C * (K + 1);
  bwd_reduce_kernel<<<(total + 255) / 256, 256, 0, s>>>(partial, static_cast<int>(grid.y * grid.z), C, K, dw, dbias);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace dwconv
}  // namespace lvb

using namespace lvb;

#define LVB_DWCONV_DISPATCH(CALL)                                              \
  if (is_bf16) {                                                               \
    if (K == 2) return dwconv::CALL(true, 2);                                  \
    if (K == 3) return dwconv::CALL(true, 3);                                  \
    if (K == 4) return dwconv::CALL(true, 4);                                  \
  } else {                                                                     \
    if (K == 2) return dwconv::CALL(false, 2);                                 \
    if (K == 3) return dwconv::CALL(false, 3);                                 \
    if (K == 4) return dwconv::CALL(false, 4);                                 \
  }                                                                            \
  return kErrBadArg;

static bool dwconv_args_ok(int B, int L, int C, int is_bf16) { return B > 0 && B <= 65535 && L > 0 && C > 0 && C % (is_bf16 ? 8 : 4) == 0; }

// x, y: [B, L, C] contiguous (bf16 or fp32); w: fp32 [C, K]; bias: fp32 [C] or null.  flip != 0: anti-causal (input gradient).
extern "C" int lvb_dwconv_fwd(const void* x, const float* w, const float* bias, void* y, int B, int L, int C, int K, int is_bf16, int act,
                              int flip, void* stream) {
  if (!dwconv_args_ok(B, L, C, is_bf16)) return kErrBadArg;
  auto s = static_cast<cudaStream_t>(stream);
#define FWD(BF, KK) launch_conv<BF, KK>(x, w, bias, y, B, L, C, act, flip, s)
  LVB_DWCONV_DISPATCH(FWD)
#undef FWD
}

extern "C" long long lvb_dwconv_partial_floats(int B, int L, int C, int K) {
  return static_cast<long long>(B) * ((L + dwconv::kRun - 1) / dwconv::kRun) * C * (K + 1);
}

// dpre [B, L, C] (same dtype as x; may be null when act == 0, where it equals dy), partial: lvb_dwconv_partial_floats fp32,
// dw fp32 [C, K], dbias fp32 [C] or null.
extern "C" int lvb_dwconv_bwd_prep(const void* x, const void* dy, const float* w, const float* bias, void* dpre, float* partial, float* dw,
                                   float* dbias, int B, int L, int C, int K, int is_bf16, int act, void* stream) {
  if (!dwconv_args_ok(B, L, C, is_bf16)) return kErrBadArg;
  auto s = static_cast<cudaStream_t>(stream);
#define PREP(BF, KK) launch_prep<BF, KK>(x, dy, w, bias, dpre, partial, dw, dbias, B, L, C, act, s)
  LVB_DWCONV_DISPATCH(PREP)
#undef PREP
}
