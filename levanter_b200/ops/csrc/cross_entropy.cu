// Row-wise cross-entropy statistics and logit gradients over a chunk of fp32 logits.
//
// The LM head is applied chunk by chunk (tokens x vocab never exists in full): the GEMM writes a
// chunk of fp32 logits, ce_stats reduces each row to (logsumexp, target logit), and in the
// backward pass the chunk is recomputed and ce_grad turns it into bf16 dlogits for the dX / dW
// GEMMs.  Semantics follow the reference's blockwise loss (src/levanter/models/loss.py:251-507):
// optional tanh soft-cap on the logits, loss = logZ - logit[target], z-loss = w * logZ^2 with
// gradient (g_loss + g_logz) * p - g_loss * onehot.
#include "common.cuh"

namespace lvb {
namespace ce {

constexpr int kBlock = 256;

__device__ __forceinline__ float capped(float l, float cap) { return cap > 0.f ? cap * tanhf(l / cap) : l; }

// one block per row
__global__ void __launch_bounds__(kBlock) ce_stats_kernel(const float* __restrict__ logits, long long ld,
                                                          const int* __restrict__ targets, float* __restrict__ lse_out,
                                                          float* __restrict__ tgt_out, int rows, int vocab, float cap,
                                                          int* status) {
  const int row = blockIdx.x;
  const float* p = logits + static_cast<long long>(row) * ld;
  float m = -INFINITY, s = 0.f;
  const int nvec = vocab >> 2;
  for (int i = threadIdx.x; i < nvec; i += kBlock) {
    float4 v = reinterpret_cast<const float4*>(p)[i];
    float a[4] = {capped(v.x, cap), capped(v.y, cap), capped(v.z, cap), capped(v.w, cap)};
    float lm = fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
    s += __expf(a[0] - m) + __expf(a[1] - m) + __expf(a[2] - m) + __expf(a[3] - m);
  }
  for (int i = (nvec << 2) + threadIdx.x; i < vocab; i += kBlock) {
    float a = capped(p[i], cap);
    if (a > m) {
      s *= __expf(m - a);
      m = a;
    }
    s += __expf(a - m);
  }
  // combine (m, s) across the block
  __shared__ float sm[kBlock / 32], ss[kBlock / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float om = __shfl_xor_sync(0xffffffffu, m, o);
    float os = __shfl_xor_sync(0xffffffffu, s, o);
    float nm = fmaxf(m, om);
    s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) {
    sm[threadIdx.x >> 5] = m;
    ss[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = sm[0], S = ss[0];
    for (int w = 1; w < kBlock / 32; ++w) {
      float nm = fmaxf(M, sm[w]);
      S = (nm == -INFINITY) ? 0.f : S * __expf(M - nm) + ss[w] * __expf(sm[w] - nm);
      M = nm;
    }
    lse_out[row] = M + __logf(S);
    int t = targets[row];
    if (t < 0 || t >= vocab) {
      // out-of-range targets (padding / ignore ids) contribute a zero target logit; their loss
      // weight is expected to be zero.  Record it so real indexing bugs are visible.
      if (t >= vocab) record_status(status, kBoundsCheck, 500, t);
      tgt_out[row] = 0.f;
    } else {
      tgt_out[row] = capped(p[t], cap);
    }
  }
}

// dlogits[row, j] = d(cap)/d(raw) * ( (g_loss[row] + g_logz[row]) * p_j - g_loss[row] * [j == target] )
// g_logz already contains 2 * z_weight * lse * g when z-loss is on.
__global__ void __launch_bounds__(kBlock) ce_grad_kernel(const float* __restrict__ logits, long long ld,
                                                         const int* __restrict__ targets, const float* __restrict__ lse,
                                                         const float* __restrict__ g_loss,
                                                         const float* __restrict__ g_logz,
                                                         __nv_bfloat16* __restrict__ dlogits, long long ldd, int rows,
                                                         int vocab, float cap) {
  const int row = blockIdx.x;
  const float* p = logits + static_cast<long long>(row) * ld;
  __nv_bfloat16* d = dlogits + static_cast<long long>(row) * ldd;
  const float L = lse[row];
  const float gl = g_loss[row];
  const float gp = gl + (g_logz != nullptr ? g_logz[row] : 0.f);
  const int t = targets[row];
  const int nvec = vocab >> 2;
  for (int i = threadIdx.x; i < nvec; i += kBlock) {
    float4 v = reinterpret_cast<const float4*>(p)[i];
    float raw[4] = {v.x, v.y, v.z, v.w};
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a = raw[j], dcap = 1.f;
      if (cap > 0.f) {
        float th = tanhf(raw[j] / cap);
        a = cap * th;
        dcap = 1.f - th * th;
      }
      float g = gp * __expf(a - L);
      if (4 * i + j == t) g -= gl;
      o[j] = g * dcap;
    }
    uint2 w;
    w.x = pack_bf16x2(o[0], o[1]);
    w.y = pack_bf16x2(o[2], o[3]);
    reinterpret_cast<uint2*>(d)[i] = w;
  }
  for (int i = (nvec << 2) + threadIdx.x; i < vocab; i += kBlock) {
    float a = p[i], dcap = 1.f;
    if (cap > 0.f) {
      float th = tanhf(a / cap);
      a = cap * th;
      dcap = 1.f - th * th;
    }
    float g = gp * __expf(a - L);
    if (i == t) g -= gl;
    d[i] = __float2bfloat16(g * dcap);
  }
}

}  // namespace ce
}  // namespace lvb

// logits: fp32 [rows, vocab] with row stride ld (multiple of 4); targets: int32 [rows].
extern "C" int lvb_ce_stats(const float* logits, long long ld, const int* targets, float* lse, float* tgt, int rows,
                            int vocab, float soft_cap, int* status, void* stream) {
  using namespace lvb;
  if (rows <= 0 || vocab <= 0 || (ld & 3)) return kErrBadArg;
  ce::ce_stats_kernel<<<rows, ce::kBlock, 0, reinterpret_cast<cudaStream_t>(stream)>>>(logits, ld, targets, lse, tgt,
                                                                                     rows, vocab, soft_cap, status);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// dlogits: bf16 [rows, vocab] with row stride ldd (multiple of 4).
extern "C" int lvb_ce_grad(const float* logits, long long ld, const int* targets, const float* lse,
                           const float* g_loss, const float* g_logz, void* dlogits, long long ldd, int rows, int vocab,
                           float soft_cap, void* stream) {
  using namespace lvb;
  if (rows <= 0 || vocab <= 0 || (ld & 3) || (ldd & 3)) return kErrBadArg;
  ce::ce_grad_kernel<<<rows, ce::kBlock, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, ld, targets, lse, g_loss, g_logz, reinterpret_cast<__nv_bfloat16*>(dlogits), ldd, rows, vocab, soft_cap);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
