// Data-parallel collectives fused with the math around them, over peer-mapped memory (NVLink / NVSwitch).
//
// The sharded engine keeps, on every rank, a flat fp32 gradient buffer and a flat bf16 weight buffer with identical
// layout, allocated as symmetric memory so that each rank holds device pointers to every peer's copy.  One optimizer step
// then needs two kernels per owned range instead of reduce-scatter -> optimizer -> all-gather library calls:
//
//  * p2p_reduce_scatter: out[i] = scale * sum_r grad_r[off + i].  Each rank pulls its own range from every peer with
//    16-byte loads (starting at a different peer per CTA so that the links are loaded evenly) and writes the reduced range
//    locally; the per-block sum of squares of the result is produced in the same pass for the global gradient norm.
//  * p2p_adamw_allgather: the AdamW update of the owned range (fp32 master weights and moments), whose bf16 result is
//    stored straight into every peer's weight buffer (16-byte stores), i.e. the all-gather is the epilogue of the update.
//
// Ordering between ranks (all gradients complete before the pull, all weights stored before the next forward pass) is done
// by the caller with barriers on the symmetric-memory signal pads; the kernels themselves never wait on another rank.
// No load here carries a multicast qualifier; peers are addressed with plain global loads and stores.
#include "common.cuh"

namespace lvb {
namespace p2p {

constexpr int kBlock = 256;
constexpr int kMaxWorld = 16;

struct PeerPtrs {
  void* p[kMaxWorld];
};

__global__ void __launch_bounds__(kBlock)
reduce_scatter_kernel(PeerPtrs peers, int world, int rank, long long off, long long n4, float scale, float4* __restrict__ out,
                      float* __restrict__ partial_sumsq) {
  float acc_sq = 0.f;
  const int first = (rank + 1 + blockIdx.x) % world;  // spread the first access over the peers
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * kBlock) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int k = 0; k < world; ++k) {
      int r = first + k;
      if (r >= world) r -= world;
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peers.p[r]) + off)[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    out[i] = s;
    acc_sq += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc_sq = warp_sum(acc_sq);
  __shared__ float sm[kBlock / 32];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc_sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kBlock / 32; ++w) t += sm[w];
    partial_sumsq[blockIdx.x] = t;
  }
}

__global__ void sumsq_accumulate_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out) {
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 32) acc += partial[i];
  acc = warp_sum(acc);
  if (threadIdx.x == 0) out[0] += acc;
}

// 8 elements per thread: fp32 state in two float4, bf16 result in one 16-byte store per peer.
__global__ void __launch_bounds__(kBlock)
adamw_allgather_kernel(float4* __restrict__ p, float4* __restrict__ m, float4* __restrict__ v, const float4* __restrict__ g,
                       PeerPtrs peers, int world, int rank, long long off, long long n8, float lr, float b1, float b2, float eps,
                       float wd, float bc1, float bc2, const float* __restrict__ grad_scale, int nesterov) {
  const float gs = grad_scale != nullptr ? grad_scale[0] : 1.f;
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * kBlock) {
    float out[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long j = 2 * i + h;
      const float4 gq = g[j];
      float4 pq = p[j], mq = m[j], vq = v[j];
      const float gv[4] = {gq.x * gs, gq.y * gs, gq.z * gs, gq.w * gs};
      float* pv = reinterpret_cast<float*>(&pq);
      float* mv = reinterpret_cast<float*>(&mq);
      float* vv = reinterpret_cast<float*>(&vq);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mi = b1 * mv[e] + (1.f - b1) * gv[e];
        const float vi = b2 * vv[e] + (1.f - b2) * gv[e] * gv[e];
        mv[e] = mi;
        vv[e] = vi;
        float mhat = mi / bc1;
        if (nesterov) mhat = b1 * (mi / (1.f - (1.f - bc1) * b1)) + (1.f - b1) * gv[e] / bc1;
        const float u = mhat / (sqrtf(vi / bc2) + eps) + wd * pv[e];
        pv[e] -= lr * u;
        out[4 * h + e] = pv[e];
      }
      p[j] = pq; m[j] = mq; v[j] = vq;
    }
    uint4 w;
    w.x = pack_bf16x2(out[0], out[1]); w.y = pack_bf16x2(out[2], out[3]);
    w.z = pack_bf16x2(out[4], out[5]); w.w = pack_bf16x2(out[6], out[7]);
    const int first = (rank + blockIdx.x) % world;
#pragma unroll 4
    for (int k = 0; k < world; ++k) {
      int r = first + k;
      if (r >= world) r -= world;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peers.p[r]) + off)[i] = w;
    }
  }
}


// ---- the same two kernels through the NVSwitch multicast mapping of the buffers: one `multimem.ld_reduce` returns the sum
// over all ranks (the reduction happens in the switch), one `multimem.st` stores to every rank's copy, so each element
// crosses this GPU's links once instead of once per peer.
__device__ __forceinline__ float4 multimem_ld_reduce_add(const float* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

__device__ __forceinline__ void multimem_st_16(void* mc_addr, uint4 w) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(w.x)),
               "f"(__uint_as_float(w.y)), "f"(__uint_as_float(w.z)), "f"(__uint_as_float(w.w))
               : "memory");
}

__global__ void __launch_bounds__(kBlock)
mm_reduce_scatter_kernel(const float* __restrict__ mc_grad, long long off, long long n4, float scale, float4* __restrict__ out,
                         float* __restrict__ partial_sumsq) {
  float acc_sq = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * kBlock) {
    float4 s = multimem_ld_reduce_add(mc_grad + off + 4 * i);
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    out[i] = s;
    acc_sq += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc_sq = warp_sum(acc_sq);
  __shared__ float sm[kBlock / 32];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc_sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kBlock / 32; ++w) t += sm[w];
    partial_sumsq[blockIdx.x] = t;
  }
}

__global__ void __launch_bounds__(kBlock)
mm_adamw_allgather_kernel(float4* __restrict__ p, float4* __restrict__ m, float4* __restrict__ v, const float4* __restrict__ g,
                          __nv_bfloat16* __restrict__ mc_param, long long off, long long n8, float lr, float b1, float b2, float eps,
                          float wd, float bc1, float bc2, const float* __restrict__ grad_scale, int nesterov) {
  const float gs = grad_scale != nullptr ? grad_scale[0] : 1.f;
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * kBlock) {
    float out[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long j = 2 * i + h;
      const float4 gq = g[j];
      float4 pq = p[j], mq = m[j], vq = v[j];
      const float gv[4] = {gq.x * gs, gq.y * gs, gq.z * gs, gq.w * gs};
      float* pv = reinterpret_cast<float*>(&pq);
      float* mv = reinterpret_cast<float*>(&mq);
      float* vv = reinterpret_cast<float*>(&vq);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mi = b1 * mv[e] + (1.f - b1) * gv[e];
        const float vi = b2 * vv[e] + (1.f - b2) * gv[e] * gv[e];
        mv[e] = mi;
        vv[e] = vi;
        float mhat = mi / bc1;
        if (nesterov) mhat = b1 * (mi / (1.f - (1.f - bc1) * b1)) + (1.f - b1) * gv[e] / bc1;
        const float u = mhat / (sqrtf(vi / bc2) + eps) + wd * pv[e];
        pv[e] -= lr * u;
        out[4 * h + e] = pv[e];
      }
      p[j] = pq; m[j] = mq; v[j] = vq;
    }
    uint4 w;
    w.x = pack_bf16x2(out[0], out[1]); w.y = pack_bf16x2(out[2], out[3]);
    w.z = pack_bf16x2(out[4], out[5]); w.w = pack_bf16x2(out[6], out[7]);
    multimem_st_16(mc_param + off + 8 * i, w);
  }
}

inline int grid_for(long long work) {
  long long g = (work + kBlock - 1) / kBlock;
  long long cap = static_cast<long long>(num_sms()) * 4;
  if (cap > 1024) cap = 1024;
  return static_cast<int>(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace p2p
}  // namespace lvb

// out[0 .. n) = scale * sum over ranks of grad_r[off .. off + n); sumsq[0] += sum(out^2).
//   peer_grads : host array of `world` device pointers (fp32 bases of every rank's gradient buffer, own rank included)
//   off, n     : elements; both multiples of 4, and the bases 16-byte aligned
//   scratch    : fp32 [1024] device scratch for the block partials
extern "C" int lvb_p2p_reduce_scatter(const void* const* peer_grads, int world, int rank, long long off, long long n, float scale,
                                      float* out, float* sumsq, float* scratch, void* stream) {
  using namespace lvb;
  using namespace lvb::p2p;
  if (world <= 0 || world > kMaxWorld || rank < 0 || rank >= world || n <= 0) return kErrBadArg;
  if ((off & 3) || (n & 3) || (reinterpret_cast<uintptr_t>(out) & 15)) return kErrBadArg;
  PeerPtrs pp;
  for (int r = 0; r < world; ++r) {
    if (peer_grads[r] == nullptr || (reinterpret_cast<uintptr_t>(peer_grads[r]) & 15)) return kErrBadArg;
    pp.p[r] = const_cast<void*>(peer_grads[r]);
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(n / 4);
  reduce_scatter_kernel<<<grid, kBlock, 0, s>>>(pp, world, rank, off, n / 4, scale, reinterpret_cast<float4*>(out), scratch);
  if (sumsq != nullptr) sumsq_accumulate_kernel<<<1, 32, 0, s>>>(scratch, grid, sumsq);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// AdamW on the owned range [0, n) of p/m/v (fp32) with gradients g (fp32), then the bf16 weights are stored to
// peer_params[r][off .. off + n) for every rank r (own rank included).  off and n multiples of 8; all bases 16-byte aligned.
extern "C" int lvb_p2p_adamw_allgather(float* p, float* m, float* v, const float* g, const void* const* peer_params, int world,
                                       int rank, long long off, long long n, float lr, float b1, float b2, float eps, float wd,
                                       float bc1, float bc2, const float* grad_scale, int nesterov, void* stream) {
  using namespace lvb;
  using namespace lvb::p2p;
  if (world <= 0 || world > kMaxWorld || rank < 0 || rank >= world || n <= 0) return kErrBadArg;
  if ((off & 7) || (n & 7)) return kErrBadArg;
  for (const void* q : {static_cast<const void*>(p), static_cast<const void*>(m), static_cast<const void*>(v), static_cast<const void*>(g)})
    if (reinterpret_cast<uintptr_t>(q) & 15) return kErrBadArg;
  PeerPtrs pp;
  for (int r = 0; r < world; ++r) {
    if (peer_params[r] == nullptr || (reinterpret_cast<uintptr_t>(peer_params[r]) & 15)) return kErrBadArg;
    pp.p[r] = const_cast<void*>(peer_params[r]);
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  adamw_allgather_kernel<<<grid_for(n / 8), kBlock, 0, s>>>(reinterpret_cast<float4*>(p), reinterpret_cast<float4*>(m),
                                                          reinterpret_cast<float4*>(v), reinterpret_cast<const float4*>(g), pp,
                                                          world, rank, off, n / 8, lr, b1, b2, eps, wd, bc1, bc2, grad_scale,
                                                          nesterov);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// Multicast variants: mc_grad / mc_param are this rank's multicast addresses of the gradient / weight buffers (one address
// that reaches every rank's copy through the switch).  Same contract as the peer-pointer entry points above.
extern "C" int lvb_mm_reduce_scatter(const void* mc_grad, long long off, long long n, float scale, float* out, float* sumsq,
                                     float* scratch, void* stream) {
  using namespace lvb;
  using namespace lvb::p2p;
  if (mc_grad == nullptr || n <= 0 || (off & 3) || (n & 3) || (reinterpret_cast<uintptr_t>(mc_grad) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return kErrBadArg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(n / 4);
  mm_reduce_scatter_kernel<<<grid, kBlock, 0, s>>>(reinterpret_cast<const float*>(mc_grad), off, n / 4, scale,
                                                  reinterpret_cast<float4*>(out), scratch);
  if (sumsq != nullptr) sumsq_accumulate_kernel<<<1, 32, 0, s>>>(scratch, grid, sumsq);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

extern "C" int lvb_mm_adamw_allgather(float* p, float* m, float* v, const float* g, void* mc_param, long long off, long long n,
                                      float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                                      const float* grad_scale, int nesterov, void* stream) {
  using namespace lvb;
  using namespace lvb::p2p;
  if (mc_param == nullptr || n <= 0 || (off & 7) || (n & 7) || (reinterpret_cast<uintptr_t>(mc_param) & 15)) return kErrBadArg;
  for (const void* q : {static_cast<const void*>(p), static_cast<const void*>(m), static_cast<const void*>(v), static_cast<const void*>(g)})
    if (reinterpret_cast<uintptr_t>(q) & 15) return kErrBadArg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  mm_adamw_allgather_kernel<<<grid_for(n / 8), kBlock, 0, s>>>(reinterpret_cast<float4*>(p), reinterpret_cast<float4*>(m),
                                                             reinterpret_cast<float4*>(v), reinterpret_cast<const float4*>(g),
                                                             reinterpret_cast<__nv_bfloat16*>(mc_param), off, n / 8, lr, b1, b2,
                                                             eps, wd, bc1, bc2, grad_scale, nesterov);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// ---------------------------------------------------------------------------------------------------------------------
// Bounded wait on a flag, as a kernel of its own: one thread waits until *flag >= target or until limit_ns of the global
// timer have passed, then records the outcome and returns (the context stays usable either way).
//   result[0] = 1 reached / 2 gave up, result[1] = last value seen, result[2..3] = waited nanoseconds (lo, hi).
// A give-up also records kTimeoutFlag in `status` like every other wait in this library.  Used by hosts that want to
// learn whether a peer ever signalled without committing a full collective to it, and by the tests of the time-out path
// (a flag that nothing sets).
namespace lvb {
__global__ void flag_wait_probe_kernel(const int* flag, int target, unsigned long long limit_ns, int sys_scope, int* result,
                                       int* status) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  const unsigned long long t0 = globaltimer_ns();
  int v = 0;
  int outcome = 2;
  unsigned long long waited = 0;
  while (true) {
    v = sys_scope ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    waited = globaltimer_ns() - t0;
    if (v >= target) { outcome = 1; break; }
    if (waited > limit_ns) break;
    __nanosleep(200);
  }
  result[0] = outcome;
  result[1] = v;
  result[2] = static_cast<int>(waited & 0xffffffffull);
  result[3] = static_cast<int>(waited >> 32);
  if (outcome == 2) record_status(status, kTimeoutFlag, 900, target);
}
}  // namespace lvb

extern "C" int lvb_flag_wait_probe(const int* flag, int target, unsigned long long limit_ns, int sys_scope, int* result, int* status,
                                   void* stream) {
  using namespace lvb;
  if (flag == nullptr || result == nullptr) return kErrBadArg;
  if (limit_ns > 5000000000ull) limit_ns = 5000000000ull;  // never more than 5 s
  flag_wait_probe_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, target, limit_ns, sys_scope, result, status);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// ---------------------------------------------------------------------------------------------------------------------
// All-reduce of a symmetric buffer in place (tensor-parallel activations): rank r reduces elements [r * n / world, ...) and
// publishes them to every rank.  The caller orders the ranks around the launch (inputs complete before, results read after).
//   multicast: one multimem.ld_reduce (the switch adds the copies) and one multimem.st (the switch writes every copy).
//   peer pointers: loads from every rank's copy, stores to every rank's copy.
namespace lvb {
namespace p2p {

__global__ void __launch_bounds__(kBlock)
mm_all_reduce_bf16_kernel(__nv_bfloat16* mc, long long off8, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n8; i += static_cast<long long>(gridDim.x) * kBlock) {
    __nv_bfloat16* a = mc + (off8 + i) * 8;
    uint32_t r0, r1, r2, r3;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "l"(a)
                 : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(a), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
                 : "memory");
  }
}

__global__ void __launch_bounds__(kBlock)
mm_all_reduce_f32_kernel(float* mc, long long off4, long long n4) {
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n4; i += static_cast<long long>(gridDim.x) * kBlock) {
    float* a = mc + (off4 + i) * 4;
    const float4 s = multimem_ld_reduce_add(a);
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a), "f"(s.x), "f"(s.y), "f"(s.z), "f"(s.w) : "memory");
  }
}

struct PeerBufs {
  void* p[8];
};

__global__ void __launch_bounds__(kBlock)
p2p_all_reduce_bf16_kernel(PeerBufs bufs, int world, long long off8, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n8; i += static_cast<long long>(gridDim.x) * kBlock) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 w = reinterpret_cast<const uint4*>(bufs.p[r])[off8 + i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    for (int r = 0; r < world; ++r) reinterpret_cast<uint4*>(bufs.p[r])[off8 + i] = o;
  }
}

__global__ void __launch_bounds__(kBlock)
p2p_all_reduce_f32_kernel(PeerBufs bufs, int world, long long off4, long long n4) {
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n4; i += static_cast<long long>(gridDim.x) * kBlock) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = reinterpret_cast<const float4*>(bufs.p[r])[off4 + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    for (int r = 0; r < world; ++r) reinterpret_cast<float4*>(bufs.p[r])[off4 + i] = acc;
  }
}

}  // namespace p2p
}  // namespace lvb

// n elements (bf16: is_f32 = 0, a multiple of 8 * world; fp32: a multiple of 4 * world) at the start of the symmetric buffer.
// mc: this rank's multicast address of the buffer, or null to use the peer pointers.
extern "C" int lvb_all_reduce_symmetric(void* mc, void* const* peers, int rank, int world, long long n, int is_f32, void* stream) {
  using namespace lvb;
  using namespace lvb::p2p;
  const int vec = is_f32 ? 4 : 8;
  if (world <= 0 || world > 8 || rank < 0 || rank >= world || n <= 0 || (n % (static_cast<long long>(vec) * world)) != 0) return kErrBadArg;
  if (mc == nullptr && peers == nullptr) return kErrBadArg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long per = n / world / vec;  // vectors in this rank's slice
  const long long off = per * rank;
  const int grid = grid_for(per);
  if (mc != nullptr) {
    if (reinterpret_cast<uintptr_t>(mc) & 15) return kErrBadArg;
    if (is_f32) mm_all_reduce_f32_kernel<<<grid, kBlock, 0, s>>>(reinterpret_cast<float*>(mc), off, per);
    else mm_all_reduce_bf16_kernel<<<grid, kBlock, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(mc), off, per);
  } else {
    PeerBufs b;
    for (int r = 0; r < 8; ++r) b.p[r] = peers[r < world ? r : 0];
    if (is_f32) p2p_all_reduce_f32_kernel<<<grid, kBlock, 0, s>>>(b, world, off, per);
    else p2p_all_reduce_bf16_kernel<<<grid, kBlock, 0, s>>>(b, world, off, per);
  }
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// ---------------------------------------------------------------------------------------------------------------------
// One-shot all-reduce for small tensors (decode-size activations) in ONE launch: every rank pushes its input into slot
// `rank` of every rank's staging area, bumps an arrival counter there, waits (bounded) until all `world` slots of its own
// area have arrived and sums them.  Two areas used alternately and counters that only grow make a barrier between calls
// unnecessary: a rank can be at most one call ahead of its slowest peer, because its own call completes only when every
// peer's push of that call has arrived.  Latency is one NVLink round trip instead of several launches.
namespace lvb {
namespace p2p {

struct OneShotArgs {
  unsigned char* stage[8];  // rank r's staging area for this call's parity: [world][cap_bytes]
  int* flags[8];            // rank r's arrival counters for this call's parity: [world]
};


__global__ void __launch_bounds__(kBlock)
one_shot_all_reduce_kernel(OneShotArgs a, const uint4* __restrict__ in, uint4* __restrict__ out, long long n16, long long cap16,
                           int rank, int world, int target, int is_f32, int* status) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  // push: this block's share of the input into slot `rank` of every rank's area
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n16; i += static_cast<long long>(gridDim.x) * kBlock) {
    const uint4 v = in[i];
    for (int r = 0; r < world; ++r) reinterpret_cast<uint4*>(a.stage[r])[rank * cap16 + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int r = 0; r < world; ++r) red_release_sys_add(a.flags[r] + rank, 1);
    // wait until every rank's blocks have all pushed into this rank's area
    for (int r = 0; r < world && !s_abort; ++r)
      flag_wait_ge(a.flags[rank] + r, target, true, &s_abort, status, 700, r);
  }
  __syncthreads();
  if (s_abort) return;
  const uint4* mine = reinterpret_cast<const uint4*>(a.stage[rank]);
  for (long long i = blockIdx.x * static_cast<long long>(kBlock) + threadIdx.x; i < n16; i += static_cast<long long>(gridDim.x) * kBlock) {
    if (is_f32) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const uint4 w = __ldcg(mine + r * cap16 + i);
        acc.x += __uint_as_float(w.x); acc.y += __uint_as_float(w.y); acc.z += __uint_as_float(w.z); acc.w += __uint_as_float(w.w);
      }
      out[i] = make_uint4(__float_as_uint(acc.x), __float_as_uint(acc.y), __float_as_uint(acc.z), __float_as_uint(acc.w));
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < world; ++r) {
        const uint4 w = __ldcg(mine + r * cap16 + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      out[i] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
  }
}

}  // namespace p2p
}  // namespace lvb

// in/out: local tensors of `bytes` bytes (a multiple of 16, at most cap_bytes); may be the same tensor.
// stage[r] / flags[r]: rank r's staging area ([world][cap_bytes]) and arrival counters ([world] ints) of this call's parity.
// blocks: the grid size, equal on every rank for a given call.  target: the sum of `blocks` over all calls, this one included,
// that have used this parity (every block of a pusher adds one arrival to each counter).
extern "C" int lvb_all_reduce_one_shot(const void* in, void* out, void* const* stage, int* const* flags, int rank, int world,
                                       long long bytes, long long cap_bytes, int blocks, int target, int is_f32, int* status,
                                       void* stream) {
  using namespace lvb;
  using namespace lvb::p2p;
  if (world <= 0 || world > 8 || rank < 0 || rank >= world || bytes <= 0 || (bytes & 15) || bytes > cap_bytes || (cap_bytes & 15) ||
      blocks <= 0 || blocks > num_sms())
    return kErrBadArg;
  OneShotArgs a;
  for (int r = 0; r < 8; ++r) {
    a.stage[r] = reinterpret_cast<unsigned char*>(stage[r < world ? r : 0]);
    a.flags[r] = flags[r < world ? r : 0];
  }
  one_shot_all_reduce_kernel<<<blocks, kBlock, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      a, reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(out), bytes / 16, cap_bytes / 16, rank, world, target, is_f32, status);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
