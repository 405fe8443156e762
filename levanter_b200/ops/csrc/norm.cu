// RMSNorm / LayerNorm forward and backward (bf16 activations, fp32 math).
//
// Covers hnn.RmsNorm / hnn.LayerNorm and Gemma's (1 + w) variant
// (src/levanter/layers/normalization.py:38-48, src/levanter/models/gemma.py:279-291), per-head
// qk-norm (rows = tokens*heads, dim = head_size) and the residual-add that precedes every
// pre-norm block: h = x + residual is written once and normalised in the same pass.
//
// Launch shape: blockDim = (TX, TY): TX threads cooperate on one row, TY rows per block.
// Every thread moves 16-byte vectors (8 bf16).  dim must be a multiple of 8.
#include "common.cuh"

namespace lvb {
namespace norm {

constexpr int kMaxVecPerThread = 8;  // backward keeps dw partials in registers: dim <= TX*8*8

struct Vec8 {
  float v[8];
};

__device__ __forceinline__ Vec8 load8(const __nv_bfloat16* p) {
  uint4 w = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
  Vec8 o;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = __bfloat1622float2(h[j]);
    o.v[2 * j] = f.x;
    o.v[2 * j + 1] = f.y;
  }
  return o;
}
__device__ __forceinline__ Vec8 unpack8(const uint4& w) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
  Vec8 o;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = __bfloat1622float2(h[j]);
    o.v[2 * j] = f.x;
    o.v[2 * j + 1] = f.y;
  }
  return o;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Vec8& a) {
  uint4 o;
  o.x = pack_bf16x2(a.v[0], a.v[1]);
  o.y = pack_bf16x2(a.v[2], a.v[3]);
  o.z = pack_bf16x2(a.v[4], a.v[5]);
  o.w = pack_bf16x2(a.v[6], a.v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ Vec8 loadw8(const void* w, int wf32, int col, float offset) {
  Vec8 o;
  if (w == nullptr) {
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = 1.f;
    return o;
  }
  if (wf32) {
    // two 16-byte loads (col is a multiple of 8 and the array 16-byte aligned): eight scalar loads per vector made the
    // weight reads, not the activations, the busiest traffic of the load/store unit
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + col);
    const float4 lo = __ldg(p), hi = __ldg(p + 1);
    o.v[0] = lo.x + offset; o.v[1] = lo.y + offset; o.v[2] = lo.z + offset; o.v[3] = lo.w + offset;
    o.v[4] = hi.x + offset; o.v[5] = hi.y + offset; o.v[6] = hi.z + offset; o.v[7] = hi.w + offset;
  } else {
    o = load8(reinterpret_cast<const __nv_bfloat16*>(w) + col);
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] += offset;
  }
  return o;
}

// Sum over the TX threads of a row.  TX is a power of two; rows never straddle
// warps when TX <= 32, otherwise TX is a multiple of 32 and shared memory joins the warps.
template <int N>
__device__ __forceinline__ void row_reduce(float (&val)[N], float* scratch, int TX) {
  const int tx = threadIdx.x;
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float v = val[i];
    for (int o = min(TX, 32) >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    val[i] = v;
  }
  if (TX > 32) {
    const int nw = TX >> 5;
    float* s = scratch + threadIdx.y * (nw * N);
    if ((tx & 31) == 0) {
#pragma unroll
      for (int i = 0; i < N; ++i) s[(tx >> 5) * N + i] = val[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < N; ++i) {
      float v = 0.f;
      for (int w = 0; w < nw; ++w) v += s[w * N + i];
      val[i] = v;
    }
    __syncthreads();
  }
}

template <bool LN>
__global__ void norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                const void* __restrict__ w, const void* __restrict__ b, int wf32,
                                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
                                float* __restrict__ rstd_out, float* __restrict__ mean_out, int rows, int dim,
                                float eps, float w_offset) {
  extern __shared__ float scratch[];
  const int TX = blockDim.x;
  const int row0 = blockIdx.x * blockDim.y + threadIdx.y;
  const int nvec = dim >> 3;
  // rows beyond the end still take part in the block-wide barriers of row_reduce
  const bool active = row0 < rows;
  const size_t base = static_cast<size_t>(active ? row0 : 0) * dim;
  float acc[2] = {0.f, 0.f};
  if (active) {
    for (int i = threadIdx.x; i < nvec; i += TX) {
      Vec8 a = load8(x + base + i * 8);
      if (residual != nullptr) {
        Vec8 r = load8(residual + base + i * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) a.v[j] += r.v[j];
        if (h_out != nullptr) {
          store8(h_out + base + i * 8, a);
          a = load8(h_out + base + i * 8);  // normalise exactly what later layers will read
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[0] += a.v[j];
        acc[1] += a.v[j] * a.v[j];
      }
    }
  }
  row_reduce<2>(acc, scratch, TX);
  const float mean = LN ? acc[0] / dim : 0.f;
  const float var = LN ? fmaxf(acc[1] / dim - mean * mean, 0.f) : acc[1] / dim;
  const float rstd = rsqrtf(var + eps);
  if (!active) return;
  if (threadIdx.x == 0) {
    if (rstd_out != nullptr) rstd_out[row0] = rstd;
    if (LN && mean_out != nullptr) mean_out[row0] = mean;
  }
  const __nv_bfloat16* src = (residual != nullptr && h_out != nullptr) ? h_out : x;
  for (int i = threadIdx.x; i < nvec; i += TX) {
    Vec8 a = load8(src + base + i * 8);
    if (residual != nullptr && h_out == nullptr) {
      Vec8 r = load8(residual + base + i * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) a.v[j] += r.v[j];
    }
    Vec8 ww = loadw8(w, wf32, i * 8, w_offset);
    Vec8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = (a.v[j] - mean) * rstd * ww.v[j];
    if (b != nullptr) {
      Vec8 bb = loadw8(b, wf32, i * 8, 0.f);
#pragma unroll
      for (int j = 0; j < 8; ++j) o.v[j] += bb.v[j];
    }
    store8(y + base + i * 8, o);
  }
}

// Forward with one warp per row and the row held in registers (packed bf16: VPL 16-byte vectors per lane): every load of the
// row is issued before anything waits, the row is read from memory once, and the reduction is five shuffles with no
// block-wide barrier.  For dim = 256 * VPL, VPL in {1, 2, 4, 8, 16} (256 ... 4096).
template <bool LN, int VPL, bool RES>
__global__ void __launch_bounds__(128, 3)
norm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual, const void* __restrict__ w,
                     const void* __restrict__ b, int wf32, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
                     float* __restrict__ rstd_out, float* __restrict__ mean_out, int rows, float eps, float w_offset) {
  constexpr int dim = 256 * VPL;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t base = static_cast<size_t>(row) * dim;
  uint4 v[VPL];
#pragma unroll
  for (int s = 0; s < VPL; ++s) v[s] = *reinterpret_cast<const uint4*>(x + base + (lane + 32 * s) * 8);
  if constexpr (RES) {
    uint4 r[VPL];
#pragma unroll
    for (int s = 0; s < VPL; ++s) r[s] = *reinterpret_cast<const uint4*>(residual + base + (lane + 32 * s) * 8);
#pragma unroll
    for (int s = 0; s < VPL; ++s) {
      const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&v[s]);
      const __nv_bfloat162* c = reinterpret_cast<const __nv_bfloat162*>(&r[s]);
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = __bfloat1622float2(a[j]), fc = __bfloat1622float2(c[j]);
        ow[j] = pack_bf16x2(fa.x + fc.x, fa.y + fc.y);  // normalise exactly what later layers will read
      }
      v[s] = o;
      if (h_out != nullptr) *reinterpret_cast<uint4*>(h_out + base + (lane + 32 * s) * 8) = o;
    }
  }
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int s = 0; s < VPL; ++s) {
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&v[s]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a[j]);
      s1 += f.x + f.y;
      s2 += f.x * f.x + f.y * f.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  const float mean = LN ? s1 / dim : 0.f;
  const float var = LN ? fmaxf(s2 / dim - mean * mean, 0.f) : s2 / dim;
  const float rstd = rsqrtf(var + eps);
  if (lane == 0) {
    if (rstd_out != nullptr) rstd_out[row] = rstd;
    if (LN && mean_out != nullptr) mean_out[row] = mean;
  }
#pragma unroll
  for (int s = 0; s < VPL; ++s) {
    const int col = (lane + 32 * s) * 8;
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&v[s]);
    const Vec8 ww = loadw8(w, wf32, col, w_offset);
    Vec8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a[j]);
      o.v[2 * j] = (f.x - mean) * rstd * ww.v[2 * j];
      o.v[2 * j + 1] = (f.y - mean) * rstd * ww.v[2 * j + 1];
    }
    if (b != nullptr) {
      const Vec8 bb = loadw8(b, wf32, col, 0.f);
#pragma unroll
      for (int j = 0; j < 8; ++j) o.v[j] += bb.v[j];
    }
    store8(y + base + col, o);
  }
}

// Backward.  Each block walks rows blockIdx.x*TY + ty, += gridDim.x*TY and keeps its
// share of dw (and db) in registers; partials go to dw_part[gridDim.x*TY, dim] and are
// summed by norm_bwd_reduce_kernel, so the result is deterministic.
//   dx = rstd * (g - mean(g) - xhat * mean(g * xhat))        (LN)
//   dx = rstd * (g - xhat * mean(g * xhat))                   (RMS)      with g = dy * w
// If dres_in is given it is added to dx (gradient arriving through the residual stream).
template <bool LN, int VPT>
__global__ void norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                const void* __restrict__ w, int wf32, const float* __restrict__ rstd_in,
                                const float* __restrict__ mean_in, const __nv_bfloat16* __restrict__ dres_in,
                                __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part,
                                float* __restrict__ db_part, int rows, int dim, float w_offset) {
  extern __shared__ float scratch[];
  const int TX = blockDim.x;
  const int nvec = dim >> 3;
  float dw_acc[VPT][8];
  float db_acc[VPT][8];
#pragma unroll
  for (int s = 0; s < VPT; ++s)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw_acc[s][j] = 0.f; db_acc[s][j] = 0.f; }
  const int row_stride = gridDim.x * blockDim.y;
  const int first = blockIdx.x * blockDim.y + threadIdx.y;
  const int iters = (rows + row_stride - 1) / row_stride;
  for (int it = 0; it < iters; ++it) {
    const int row = first + it * row_stride;
    const bool active = row < rows;
    const size_t base = static_cast<size_t>(active ? row : 0) * dim;
    const float rstd = active ? rstd_in[row] : 0.f;
    const float mean = (LN && active) ? mean_in[row] : 0.f;
    float acc[2] = {0.f, 0.f};
    if (active) {
#pragma unroll
      for (int s = 0; s < VPT; ++s) {
        const int i = threadIdx.x + s * TX;
        if (i < nvec) {
          Vec8 g = load8(dy + base + i * 8);
          Vec8 a = load8(x + base + i * 8);
          Vec8 ww = loadw8(w, wf32, i * 8, w_offset);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xh = (a.v[j] - mean) * rstd;
            const float gw = g.v[j] * ww.v[j];
            acc[0] += gw;
            acc[1] += gw * xh;
            dw_acc[s][j] += g.v[j] * xh;
            db_acc[s][j] += g.v[j];
          }
        }
      }
    }
    row_reduce<2>(acc, scratch, TX);
    const float m1 = LN ? acc[0] / dim : 0.f;
    const float m2 = acc[1] / dim;
    if (active) {
#pragma unroll
      for (int s = 0; s < VPT; ++s) {
        const int i = threadIdx.x + s * TX;
        if (i < nvec) {
          Vec8 g = load8(dy + base + i * 8);
          Vec8 a = load8(x + base + i * 8);
          Vec8 ww = loadw8(w, wf32, i * 8, w_offset);
          Vec8 o;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xh = (a.v[j] - mean) * rstd;
            o.v[j] = rstd * (g.v[j] * ww.v[j] - m1 - xh * m2);
          }
          if (dres_in != nullptr) {
            Vec8 r = load8(dres_in + base + i * 8);
#pragma unroll
            for (int j = 0; j < 8; ++j) o.v[j] += r.v[j];
          }
          store8(dx + base + i * 8, o);
        }
      }
    }
  }
  const int prow = blockIdx.x * blockDim.y + threadIdx.y;
#pragma unroll
  for (int s = 0; s < VPT; ++s) {
    const int i = threadIdx.x + s * TX;
    if (i < nvec) {
      if (dw_part != nullptr) {
        float* p = dw_part + static_cast<size_t>(prow) * dim + i * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) p[j] = dw_acc[s][j];
      }
      if (db_part != nullptr) {
        float* p = db_part + static_cast<size_t>(prow) * dim + i * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) p[j] = db_acc[s][j];
      }
    }
  }
}

// out[c] (+)= sum over the partial rows.  A block owns 32 columns; its 8 thread rows each sum every 8th partial row (four
// independent accumulators, so the loads overlap) and are then added in a fixed order: deterministic, and a few hundred
// partial rows cost tens of loads per thread instead of one dependent chain of all of them.
__global__ void __launch_bounds__(256)
norm_bwd_reduce_kernel(const float* __restrict__ part, float* __restrict__ out, int nparts, int dim, int accumulate) {
  __shared__ float sm[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if (c < dim) {
    int r = ty;
    for (; r + 24 < nparts; r += 32) {
      a0 += part[static_cast<size_t>(r) * dim + c];
      a1 += part[static_cast<size_t>(r + 8) * dim + c];
      a2 += part[static_cast<size_t>(r + 16) * dim + c];
      a3 += part[static_cast<size_t>(r + 24) * dim + c];
    }
    for (; r < nparts; r += 8) a0 += part[static_cast<size_t>(r) * dim + c];
  }
  sm[ty][tx] = (a0 + a1) + (a2 + a3);
  __syncthreads();
  if (ty == 0 && c < dim) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += sm[j][tx];
    out[c] = accumulate ? out[c] + s : s;
  }
}

inline void pick_block(int dim, int& TX, int& TY) {
  const int nvec = dim >> 3;
  TX = 8;
  while (TX < nvec && TX < 256) TX <<= 1;  // one vector per thread when possible
  if (nvec >= 512) TX = 256;
  TY = 256 / TX;
  if (TY < 1) TY = 1;
}

}  // namespace norm
}  // namespace lvb

// y = norm(x (+ residual)) * (w + w_offset) (+ b).  layer_norm: 0 = RMS, 1 = LayerNorm.
// h_out (optional) receives x + residual.  rstd_out / mean_out are fp32 [rows] (saved for backward).
extern "C" int lvb_norm_fwd(const void* x, const void* residual, const void* w, const void* b, int w_is_f32, void* y,
                            void* h_out, float* rstd_out, float* mean_out, int rows, int dim, float eps,
                            float w_offset, int layer_norm, void* stream) {
  using namespace lvb;
  using namespace lvb::norm;
  if (rows <= 0 || dim <= 0 || (dim & 7)) return kErrBadArg;
  int TX, TY;
  pick_block(dim, TX, TY);
  dim3 block(TX, TY);
  dim3 grid((rows + TY - 1) / TY);
  size_t smem = sizeof(float) * TY * (TX > 32 ? (TX / 32) * 2 : 0);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<const __nv_bfloat16*>(residual);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  auto H = reinterpret_cast<__nv_bfloat16*>(h_out);
  {
    const int vpl = dim / 256;
    if (dim % 256 == 0 && (vpl == 1 || vpl == 2 || vpl == 4 || vpl == 8 || vpl == 16)) {
      const dim3 wgrid((rows + 3) / 4);
#define LVB_NORM_WARP(LNV, V)                                                                                                  \
  if (R != nullptr)                                                                                                            \
    norm_fwd_warp_kernel<LNV, V, true><<<wgrid, 128, 0, s>>>(X, R, w, b, w_is_f32, Y, H, rstd_out, mean_out, rows, eps, w_offset); \
  else                                                                                                                         \
    norm_fwd_warp_kernel<LNV, V, false><<<wgrid, 128, 0, s>>>(X, R, w, b, w_is_f32, Y, H, rstd_out, mean_out, rows, eps, w_offset)
#define LVB_NORM_WARP_V(LNV)                                                                                                   \
  switch (vpl) {                                                                                                               \
    case 1: LVB_NORM_WARP(LNV, 1); break;                                                                                      \
    case 2: LVB_NORM_WARP(LNV, 2); break;                                                                                      \
    case 4: LVB_NORM_WARP(LNV, 4); break;                                                                                      \
    case 8: LVB_NORM_WARP(LNV, 8); break;                                                                                      \
    default: LVB_NORM_WARP(LNV, 16); break;                                                                                    \
  }
      if (layer_norm) { LVB_NORM_WARP_V(true) } else { LVB_NORM_WARP_V(false) }
#undef LVB_NORM_WARP_V
#undef LVB_NORM_WARP
      return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
    }
  }
  if (layer_norm)
    norm_fwd_kernel<true><<<grid, block, smem, s>>>(X, R, w, b, w_is_f32, Y, H, rstd_out, mean_out, rows, dim, eps, w_offset);
  else
    norm_fwd_kernel<false><<<grid, block, smem, s>>>(X, R, w, b, w_is_f32, Y, H, rstd_out, mean_out, rows, dim, eps, w_offset);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// Backward of lvb_norm_fwd.  x is the normalised input (x + residual if a residual was added).
// scratch: fp32 [2 * nparts * dim] where nparts = lvb_norm_bwd_parts(rows, dim); dw/db are fp32 [dim]
// (either may be null).  accumulate != 0 adds into dw/db.
extern "C" int lvb_norm_bwd_parts(int rows, int dim) {
  using namespace lvb::norm;
  int TX, TY;
  pick_block(dim, TX, TY);
  int blocks = (rows + TY - 1) / TY;
  int cap = lvb::num_sms() * 3;  // three CTAs of 256 threads fit an SM at this kernel's register count; two left its warps 25 % active
  if (blocks > cap) blocks = cap;
  return blocks * TY;
}

extern "C" int lvb_norm_bwd(const void* dy, const void* x, const void* w, int w_is_f32, const float* rstd,
                            const float* mean, const void* dres_in, void* dx, float* dw, float* db, float* scratch,
                            int rows, int dim, float w_offset, int layer_norm, int accumulate, void* stream) {
  using namespace lvb;
  using namespace lvb::norm;
  if (rows <= 0 || dim <= 0 || (dim & 7)) return kErrBadArg;
  int TX, TY;
  pick_block(dim, TX, TY);
  if ((dim >> 3) > TX * kMaxVecPerThread) return kErrTooLarge;
  const int nparts = lvb_norm_bwd_parts(rows, dim);
  dim3 block(TX, TY);
  dim3 grid(nparts / TY);
  size_t smem = sizeof(float) * TY * (TX > 32 ? (TX / 32) * 2 : 0);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float* dw_part = dw != nullptr ? scratch : nullptr;
  float* db_part = db != nullptr ? scratch + static_cast<size_t>(nparts) * dim : nullptr;
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto DR = reinterpret_cast<const __nv_bfloat16*>(dres_in);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  const int vpt = ((dim >> 3) + TX - 1) / TX;
#define LVB_NORM_BWD(LN, V) \
  norm_bwd_kernel<LN, V><<<grid, block, smem, s>>>(DY, X, w, w_is_f32, rstd, mean, DR, DX, dw_part, db_part, rows, dim, w_offset)
  if (layer_norm) {
    if (vpt <= 1) LVB_NORM_BWD(true, 1); else if (vpt <= 2) LVB_NORM_BWD(true, 2);
    else if (vpt <= 4) LVB_NORM_BWD(true, 4); else LVB_NORM_BWD(true, 8);
  } else {
    if (vpt <= 1) LVB_NORM_BWD(false, 1); else if (vpt <= 2) LVB_NORM_BWD(false, 2);
    else if (vpt <= 4) LVB_NORM_BWD(false, 4); else LVB_NORM_BWD(false, 8);
  }
#undef LVB_NORM_BWD
  if (dw != nullptr) norm_bwd_reduce_kernel<<<(dim + 31) / 32, 256, 0, s>>>(dw_part, dw, nparts, dim, accumulate);
  if (db != nullptr) norm_bwd_reduce_kernel<<<(dim + 31) / 32, 256, 0, s>>>(db_part, db, nparts, dim, accumulate);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
