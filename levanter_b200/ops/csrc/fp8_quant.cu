// Quantisation to fp8 for delayed per-tensor scaling: ONE pass over a bf16 matrix produces its fp8 copy, optionally the
// transposed fp8 copy (the weight-gradient and input-gradient GEMMs want K-contiguous operands), and the absolute maximum
// of the tensor for the scaling history.  The scale used comes from the history (a device scalar written by earlier steps),
// so no pass over the tensor precedes the quantisation; values beyond the scale's range saturate.
//
// Semantics of the reference's fp8 path (haliax.quantization Fp8DotGeneralOp reached through trainer.quantization,
// src/levanter/trainer.py:648): e4m3 for forward operands, e5m2 for gradients, per-tensor delayed scaling.
#include <cuda_fp8.h>

#include "common.cuh"

namespace lvb {
namespace f8 {

constexpr int TILE = 64;

template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3));
}

// x [rows, cols] (row stride ld) -> q [rows, cols], qt [cols, rows] (may be null); amax_out gets max |x| (atomic on the bit
// pattern of a non-negative float); inv_scale_out[0] = amax_in / fmax (what the GEMM epilogue multiplies by).
template <bool E5M2>
__global__ void quantize_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int rows, int cols, const float* __restrict__ amax_in,
                                float fmax, uint8_t* __restrict__ q, uint8_t* __restrict__ qt, float* __restrict__ inv_scale_out,
                                unsigned int* __restrict__ amax_out) {
  __shared__ uint8_t tile[TILE][TILE + 4];
  __shared__ float wmax[8];
  const float amax = fmaxf(amax_in[0], 1e-12f);
  const float scale = fmax / amax;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && inv_scale_out != nullptr) inv_scale_out[0] = amax / fmax;
  const int r0 = blockIdx.y * TILE, c0 = blockIdx.x * TILE;
  // 256 threads: thread t handles row (t / 8) + 32 * pass, 8 consecutive columns (t % 8) * 8
  float local_max = 0.f;
  const int cc = (threadIdx.x & 7) * 8;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int rr = (threadIdx.x >> 3) + 32 * pass;
    const int r = r0 + rr, c = c0 + cc;
    uint8_t b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (r < rows && c < cols) {
      const __nv_bfloat16* src = x + static_cast<long long>(r) * ld + c;
      float v[8];
      if (c + 8 <= cols && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(src));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          v[2 * j] = f.x;
          v[2 * j + 1] = f.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (c + j < cols) ? __bfloat162float(src[j]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        local_max = fmaxf(local_max, fabsf(v[j]));
        b[j] = to_fp8<E5M2>(v[j] * scale);
      }
      uint8_t* dst = q + static_cast<long long>(r) * cols + c;
      if (c + 8 <= cols && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
        *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(b);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (c + j < cols) dst[j] = b[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[rr][cc + j] = b[j];
  }
  local_max = lvb::warp_max(local_max);
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = local_max;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int w = 0; w < 8; ++w) m = fmaxf(m, wmax[w]);
    if (amax_out != nullptr) atomicMax(amax_out, __float_as_uint(m));
  }
  if (qt != nullptr) {
    // transposed store: thread t writes column (t / 8) + 32 * pass of the tile as 8 consecutive bytes of a row of qt
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int tc = (threadIdx.x >> 3) + 32 * pass;  // column of x = row of qt
      const int tr = (threadIdx.x & 7) * 8;           // first of 8 rows of x = columns of qt
      const int c = c0 + tc, r = r0 + tr;
      if (c < cols && r < rows) {
        uint8_t b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) b[j] = tile[tr + j][tc];
        uint8_t* dst = qt + static_cast<long long>(c) * rows + r;
        if (r + 8 <= rows && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
          *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(b);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (r + j < rows) dst[j] = b[j];
        }
      }
    }
  }
}

}  // namespace f8
}  // namespace lvb

// x [rows, cols] bf16 (row stride ld elements) -> q [rows, cols] and, if qt != null, qt [cols, rows], as e4m3 (fmt 0) or
// e5m2 (fmt 1) of x * fmax / amax_in[0].  inv_scale_out[0] = amax_in[0] / fmax (may be null).  amax_out (may be null) is a
// device uint32 that the caller zeroes beforehand; afterwards its bits are the float max |x|.
extern "C" int lvb_fp8_quantize(const void* x, long long ld, int rows, int cols, const float* amax_in, int fmt, void* q, void* qt,
                                float* inv_scale_out, void* amax_out, void* stream) {
  using namespace lvb;
  if (rows <= 0 || cols <= 0 || fmt < 0 || fmt > 1 || amax_in == nullptr || q == nullptr) return kErrBadArg;
  dim3 grid((cols + f8::TILE - 1) / f8::TILE, (rows + f8::TILE - 1) / f8::TILE);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (fmt == 0)
    f8::quantize_kernel<false><<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), ld, rows, cols, amax_in, 448.f,
                                                     reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(qt), inv_scale_out,
                                                     reinterpret_cast<unsigned int*>(amax_out));
  else
    f8::quantize_kernel<true><<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), ld, rows, cols, amax_in, 57344.f,
                                                    reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(qt), inv_scale_out,
                                                    reinterpret_cast<unsigned int*>(amax_out));
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
