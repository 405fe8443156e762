// Rotary embedding and gated-activation kernels (bf16 in/out, fp32 math).
//
// RoPE uses the half-split convention (first half pairs with second half) and a precomputed
// fp32 cos/sin table [max_pos, head_dim] that already includes any YaRN temperature
// (src/levanter/layers/rotary.py:17-46,186-229).  The backward pass is the same rotation with
// sin negated, so one kernel serves both directions.
//
// The gated activation computes h = act(gate) * up for SwiGLU / GeGLU MLPs
// (src/levanter/models/llama.py:273-280, src/levanter/models/gemma.py) and its backward.
#include "common.cuh"

namespace lvb {
namespace ew {

// x: [tokens, heads, head_dim] with token stride `tok_stride` elements (heads contiguous).
// One thread handles 8 consecutive dims of the first half and the matching 8 of the second half.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos_ids, int tokens, int heads,
                            int head_dim, long long tok_stride, int seq_len, int max_pos, float sin_sign,
                            int* status) {
  const int half = head_dim >> 1;
  const int vec_per_head = half >> 3;
  const long long total = static_cast<long long>(tokens) * heads * vec_per_head;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(idx % vec_per_head);
    const long long th = idx / vec_per_head;
    const int h = static_cast<int>(th % heads);
    const int t = static_cast<int>(th / heads);
    int pos = pos_ids != nullptr ? pos_ids[t] : (t % seq_len);
    if (pos < 0 || pos >= max_pos) {
      record_status(status, kBoundsCheck, 400, pos);
      continue;
    }
    __nv_bfloat16* p = x + t * tok_stride + static_cast<long long>(h) * head_dim + v * 8;
    const float* c = cos_t + static_cast<long long>(pos) * head_dim + v * 8;
    const float* s = sin_t + static_cast<long long>(pos) * head_dim + v * 8;
    uint4 w1 = *reinterpret_cast<const uint4*>(p);
    uint4 w2 = *reinterpret_cast<const uint4*>(p + half);
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&w1);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&w2);
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x1 = __bfloat1622float2(a[j]);
      float2 x2 = __bfloat1622float2(b[j]);
      const float c0 = c[2 * j], c1 = c[2 * j + 1];
      const float s0 = s[2 * j] * sin_sign, s1 = s[2 * j + 1] * sin_sign;
      // the table's second half equals its first half
      o1[j] = pack_bf16x2(x1.x * c0 - x2.x * s0, x1.y * c1 - x2.y * s1);
      o2[j] = pack_bf16x2(x2.x * c0 + x1.x * s0, x2.y * c1 + x1.y * s1);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4*>(p + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

enum Act : int { kSilu = 0, kGeluTanh = 1, kGelu = 2, kRelu = 3, kQuickGelu = 4 };

__device__ __forceinline__ float act_fwd(float g, int act) {
  switch (act) {
    case kSilu: return g / (1.f + __expf(-g));
    case kGeluTanh: {
      const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      return 0.5f * g * (1.f + tanhf(u));
    }
    case kGelu: return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
    case kRelu: return fmaxf(g, 0.f);
    default: return g / (1.f + __expf(-1.702f * g));
  }
}
__device__ __forceinline__ float act_bwd(float g, int act) {
  switch (act) {
    case kSilu: {
      const float sg = 1.f / (1.f + __expf(-g));
      return sg * (1.f + g * (1.f - sg));
    }
    case kGeluTanh: {
      const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      const float th = tanhf(u);
      const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * g * g);
      return 0.5f * (1.f + th) + 0.5f * g * (1.f - th * th) * du;
    }
    case kGelu: return 0.5f * (1.f + erff(g * 0.7071067811865476f)) + g * 0.3989422804014327f * __expf(-0.5f * g * g);
    case kRelu: return g > 0.f ? 1.f : 0.f;
    default: {
      const float sg = 1.f / (1.f + __expf(-1.702f * g));
      return sg * (1.f + 1.702f * g * (1.f - sg));
    }
  }
}

// gate/up: [rows, cols] with row strides ldg/ldu (so both may be halves of one fused [rows, 2*cols] buffer).
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                               __nv_bfloat16* __restrict__ out, int rows, int cols, long long ldg, long long ldu,
                               long long ldo, int act) {
  const int vec_per_row = cols >> 3;
  const long long total = static_cast<long long>(rows) * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(idx % vec_per_row);
    const long long r = idx / vec_per_row;
    uint4 wg = *reinterpret_cast<const uint4*>(gate + r * ldg + v * 8);
    uint4 wu = *reinterpret_cast<const uint4*>(up + r * ldu + v * 8);
    const __nv_bfloat162* g = reinterpret_cast<const __nv_bfloat162*>(&wg);
    const __nv_bfloat162* u = reinterpret_cast<const __nv_bfloat162*>(&wu);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gf = __bfloat1622float2(g[j]);
      float2 uf = __bfloat1622float2(u[j]);
      o[j] = pack_bf16x2(act_fwd(gf.x, act) * uf.x, act_fwd(gf.y, act) * uf.y);
    }
    *reinterpret_cast<uint4*>(out + r * ldo + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gate,
                               const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ dgate,
                               __nv_bfloat16* __restrict__ dup, int rows, int cols, long long ldd, long long ldg,
                               long long ldu, long long lddg, long long lddu, int act) {
  const int vec_per_row = cols >> 3;
  const long long total = static_cast<long long>(rows) * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(idx % vec_per_row);
    const long long r = idx / vec_per_row;
    uint4 wd = *reinterpret_cast<const uint4*>(dout + r * ldd + v * 8);
    uint4 wg = *reinterpret_cast<const uint4*>(gate + r * ldg + v * 8);
    uint4 wu = *reinterpret_cast<const uint4*>(up + r * ldu + v * 8);
    const __nv_bfloat162* d = reinterpret_cast<const __nv_bfloat162*>(&wd);
    const __nv_bfloat162* g = reinterpret_cast<const __nv_bfloat162*>(&wg);
    const __nv_bfloat162* u = reinterpret_cast<const __nv_bfloat162*>(&wu);
    uint32_t og[4], ou[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 df = __bfloat1622float2(d[j]);
      float2 gf = __bfloat1622float2(g[j]);
      float2 uf = __bfloat1622float2(u[j]);
      og[j] = pack_bf16x2(df.x * uf.x * act_bwd(gf.x, act), df.y * uf.y * act_bwd(gf.y, act));
      ou[j] = pack_bf16x2(df.x * act_fwd(gf.x, act), df.y * act_fwd(gf.y, act));
    }
    *reinterpret_cast<uint4*>(dgate + r * lddg + v * 8) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dup + r * lddu + v * 8) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

inline int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  long long cap = static_cast<long long>(num_sms()) * 16;
  return static_cast<int>(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace ew
}  // namespace lvb

// In-place rotation of x[tokens, heads, head_dim] (token stride tok_stride elements).
// pos_ids: int32 [tokens] or null (then position = token index mod seq_len).
// sin_sign: +1 forward, -1 backward.  head_dim must be a multiple of 16.
extern "C" int lvb_rope(void* x, const float* cos_t, const float* sin_t, const int* pos_ids, int tokens, int heads,
                        int head_dim, long long tok_stride, int seq_len, int max_pos, float sin_sign, int* status,
                        void* stream) {
  using namespace lvb;
  if (tokens <= 0 || heads <= 0 || (head_dim & 15) || (tok_stride & 7)) return kErrBadArg;
  const long long total = static_cast<long long>(tokens) * heads * (head_dim >> 4);
  const int block = 256;
  ew::rope_kernel<<<ew::grid_for(total, block), block, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(x), cos_t, sin_t, pos_ids, tokens, heads, head_dim, tok_stride, seq_len, max_pos,
      sin_sign, status);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

extern "C" int lvb_glu_fwd(const void* gate, const void* up, void* out, int rows, int cols, long long ldg,
                           long long ldu, long long ldo, int act, void* stream) {
  using namespace lvb;
  if (rows <= 0 || cols <= 0 || (cols & 7) || (ldg & 7) || (ldu & 7) || (ldo & 7)) return kErrBadArg;
  const long long total = static_cast<long long>(rows) * (cols >> 3);
  const int block = 256;
  ew::glu_fwd_kernel<<<ew::grid_for(total, block), block, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gate), reinterpret_cast<const __nv_bfloat16*>(up),
      reinterpret_cast<__nv_bfloat16*>(out), rows, cols, ldg, ldu, ldo, act);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

extern "C" int lvb_glu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup, int rows,
                           int cols, long long ldd, long long ldg, long long ldu, long long lddg, long long lddu,
                           int act, void* stream) {
  using namespace lvb;
  if (rows <= 0 || cols <= 0 || (cols & 7) || (ldd & 7) || (ldg & 7) || (ldu & 7) || (lddg & 7) || (lddu & 7))
    return kErrBadArg;
  const long long total = static_cast<long long>(rows) * (cols >> 3);
  const int block = 256;
  ew::glu_bwd_kernel<<<ew::grid_for(total, block), block, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dout), reinterpret_cast<const __nv_bfloat16*>(gate),
      reinterpret_cast<const __nv_bfloat16*>(up), reinterpret_cast<__nv_bfloat16*>(dgate),
      reinterpret_cast<__nv_bfloat16*>(dup), rows, cols, ldd, ldg, ldu, lddg, lddu, act);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
