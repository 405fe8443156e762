// Token embedding: row gather (forward) and a deterministic scatter-add of the output gradient into the fp32 gradient
// accumulator (backward).
//
// Replaces hnn.Embedding's gather and its transpose (src/levanter/models/llama.py:460-468): the reference lowers both to
// XLA gather / scatter.  Backward takes the token positions sorted by token id: the CTA at the first position of a run of
// equal ids sums the run's gradient rows in position order (fp32) and adds the sum to that row of the accumulator, so each
// row has one writer and the result does not depend on scheduling.
#include "common.cuh"

namespace lvb {
namespace emb {

// out[t, :] = weight[ids[t], :]; 16 bytes per thread and step.  Ids outside [0, vocab) leave a bounds code and a zero row.
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out,
                                     int tokens, int dim, int vocab, int* status) {
  const int vec = dim >> 3;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) record_status(status, kBoundsCheck, 600, id);
    const uint4* src = reinterpret_cast<const uint4*>(weight + static_cast<size_t>(ok ? id : 0) * dim);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * dim);
    for (int v = threadIdx.x; v < vec; v += blockDim.x) dst[v] = ok ? __ldg(src + v) : make_uint4(0, 0, 0, 0);
  }
}

// sorted_ids[i] ascending, order[i] = position in dy of the i-th entry.  grad[id, :] += scale * sum_{run} dy[order[j], :].
__global__ void embedding_bwd_kernel(const int* __restrict__ sorted_ids, const int* __restrict__ order, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ grad, int tokens, int dim, int vocab, float scale, int* status) {
  const int vec = dim >> 3;
  for (int i = blockIdx.x; i < tokens; i += gridDim.x) {
    const int id = sorted_ids[i];
    if (i > 0 && sorted_ids[i - 1] == id) continue;  // not the start of a run (uniform over the CTA)
    if (id < 0 || id >= vocab) {
      if (threadIdx.x == 0) record_status(status, kBoundsCheck, 601, id);
      continue;
    }
    int end = i + 1;
    while (end < tokens && sorted_ids[end] == id) ++end;
    float* g = grad + static_cast<size_t>(id) * dim;
    for (int v = threadIdx.x; v < vec; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = i; j < end; ++j) {
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(dy + static_cast<size_t>(order[j]) * dim) + v);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(h[q]);
          acc[2 * q] += f.x;
          acc[2 * q + 1] += f.y;
        }
      }
      float4* o = reinterpret_cast<float4*>(g + v * 8);
      float4 a = o[0], b = o[1];
      a.x += scale * acc[0]; a.y += scale * acc[1]; a.z += scale * acc[2]; a.w += scale * acc[3];
      b.x += scale * acc[4]; b.y += scale * acc[5]; b.z += scale * acc[6]; b.w += scale * acc[7];
      o[0] = a;
      o[1] = b;
    }
  }
}

}  // namespace emb
}  // namespace lvb

// out[tokens, dim] (bf16) = weight[ids]; dim a multiple of 8, rows 16-byte aligned.
extern "C" int lvb_embedding_fwd(const int* ids, const void* weight, void* out, int tokens, int dim, int vocab, int* status, void* stream) {
  using namespace lvb;
  if (tokens <= 0 || dim <= 0 || (dim & 7) || vocab <= 0) return kErrBadArg;
  const int threads = dim >= 2048 ? 256 : 128;
  int grid = tokens < 8 * num_sms() ? tokens : 8 * num_sms();
  emb::embedding_fwd_kernel<<<grid, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ids, reinterpret_cast<const __nv_bfloat16*>(weight), reinterpret_cast<__nv_bfloat16*>(out), tokens, dim, vocab, status);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// grad[vocab, dim] (fp32) += scale * scatter(dy[tokens, dim] (bf16)) with the positions sorted by id (see the kernel).
extern "C" int lvb_embedding_bwd(const int* sorted_ids, const int* order, const void* dy, float* grad, int tokens, int dim, int vocab,
                                 float scale, int* status, void* stream) {
  using namespace lvb;
  if (tokens <= 0 || dim <= 0 || (dim & 7) || vocab <= 0) return kErrBadArg;
  const int threads = dim >= 2048 ? 256 : 128;
  int grid = tokens < 16 * num_sms() ? tokens : 16 * num_sms();
  emb::embedding_bwd_kernel<<<grid, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      sorted_ids, order, reinterpret_cast<const __nv_bfloat16*>(dy), grad, tokens, dim, vocab, scale, status);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
