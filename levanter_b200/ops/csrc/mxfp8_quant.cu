// bf16 -> block-scaled fp8 ("MX": one power-of-two scale per 32 values) in one pass, for gemm_mxfp8.cu.
//
// From x[R, C] (bf16, row-major) the kernel writes, as asked,
//   q_row [R, C] fp8 with blocks of 32 along C and their scales  (x as a K-major operand contracted over C), and/or
//   q_col [C, R] fp8 -- the transpose -- with blocks of 32 along R and their scales  (x^T as an operand contracted over R).
// A training step needs both of an activation or a weight: the forward product contracts over one dimension, a backward
// product over the other, and a block's scale belongs to the contraction direction, so the transposed copy is a different
// quantisation, not a byte shuffle of the first.  One CTA reads a 128 x 128 tile once into shared memory and serves both.
//
// scale = 2^e with e = ceil(log2(amax / fmax)) (fmax = 448 for e4m3, 57344 for e5m2): the smallest power of two that brings
// the block's largest magnitude into range, so nothing saturates.  An all-zero block gets e = -127.  The byte stored is e + 127.  Scales go to the chunked layout the tensor core
// wants: for every (128 operand rows, 128 values of K) 512 bytes, byte (r % 32) * 16 + (r / 32) * 4 + j for row r and block j;
// rows past the end of the operand get 127 (scale 1) so that the zero rows TMA fills in stay zero.
#include <cuda_fp8.h>

#include "common.cuh"

namespace lvb {
namespace mxq {

constexpr int kTile = 128;
constexpr int kPitch = kTile + 8;  // bf16 per shared-memory row: 272 bytes keep rows 16-byte aligned and put row i at bank 4 i

// ceil(log2(amax / fmax)), exactly: the exponent field of the correctly rounded quotient, plus one unless it is a power of two
__device__ __forceinline__ int block_exponent(float amax, float fmax) {
  if (!(amax > 0.f)) return -127;
  const int bits = __float_as_int(__fdiv_rn(amax, fmax));
  const int e = ((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) != 0 ? 1 : 0);
  return e < -127 ? -127 : (e > 126 ? 126 : e);
}
__device__ __forceinline__ float exp2_int(int e) {  // 2^e for e in [-126, 127]; 2^-127 for the all-zero block does not matter
  e = e < -126 ? -126 : e;
  return __int_as_float((e + 127) << 23);
}
__device__ __forceinline__ uint32_t cvt4(float a, float b, float c, float d, int fmt) {
  const __nv_fp8_interpretation_t k = fmt ? __NV_E5M2 : __NV_E4M3;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, k);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, k);
  return lo | (hi << 16);
}
__device__ __forceinline__ float amax8(uint4 w, float m) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 f = __bfloat1622float2(h[t]);
    m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
  return m;
}
__device__ __forceinline__ uint2 cvt8(uint4 w, float inv, int fmt) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
  return make_uint2(cvt4(a.x * inv, a.y * inv, b.x * inv, b.y * inv, fmt), cvt4(c.x * inv, c.y * inv, d.x * inv, d.y * inv, fmt));
}

// Five CTAs per SM (35 KB of shared memory and at most 48 registers each): the tile is brought in by 16-byte asynchronous copies,
// and each block of 32 is read from shared memory twice (maximum, then conversion) rather than held in registers, so that
// enough CTAs are resident for their load phases to keep DRAM busy while others compute.
__global__ void __launch_bounds__(256, 5)
mxfp8_quant_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int R, int C, int fmt, uint8_t* __restrict__ q_row,
                   uint8_t* __restrict__ sf_row, uint8_t* __restrict__ q_col, uint8_t* __restrict__ sf_col) {
  __shared__ __align__(16) __nv_bfloat16 tile[kTile * kPitch];
  const int c0 = blockIdx.x * kTile, r0 = blockIdx.y * kTile;
  const int tid = threadIdx.x;
  const float fmax = fmt ? 57344.f : 448.f;
  // ---- load: 128 rows x 16 chunks of 16 bytes, 8 chunks per thread; outside the matrix the tile is zero (C % 8 == 0)
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = it * 256 + tid;
    const int r = idx >> 4, c = (idx & 15) * 8;
    const uint32_t dst = smem_u32(tile + r * kPitch + c);
    const bool in = r0 + r < R && c0 + c < C;
    const void* src = in ? static_cast<const void*>(x + static_cast<size_t>(r0 + r) * ldx + c0 + c) : static_cast<const void*>(x);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0) : "memory");
  }
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  const int cblocks = (C + kTile - 1) / kTile, rblocks = (R + kTile - 1) / kTile;
  const int i = tid & 127, half = tid >> 7;  // a row (or column) of the tile -- consecutive over a warp -- and two of its four blocks
  if (q_row != nullptr) {
    uint8_t* sf = sf_row + (static_cast<size_t>(blockIdx.y) * cblocks + blockIdx.x) * 512 + (i & 31) * 16 + (i >> 5) * 4;
#pragma unroll
    for (int bb = 0; bb < 2; ++bb) {
      const int j = half * 2 + bb;
      const uint4* src = reinterpret_cast<const uint4*>(tile + i * kPitch + j * 32);
      float amax = 0.f;
#pragma unroll
      for (int t = 0; t < 4; ++t) amax = amax8(src[t], amax);
      const bool live = r0 + i < R && c0 + j * 32 < C;
      const int e = live ? block_exponent(amax, fmax) : 0;
      sf[j] = static_cast<uint8_t>(e + 127);
      if (live) {
        const float inv = exp2_int(-e);
        const uint2 a = cvt8(src[0], inv, fmt), b = cvt8(src[1], inv, fmt), c = cvt8(src[2], inv, fmt), d = cvt8(src[3], inv, fmt);
        uint4* dst = reinterpret_cast<uint4*>(q_row + static_cast<size_t>(r0 + i) * C + c0 + j * 32);  // C % 32 == 0
        dst[0] = make_uint4(a.x, a.y, b.x, b.y);
        dst[1] = make_uint4(c.x, c.y, d.x, d.y);
      }
    }
  }
  if (q_col != nullptr) {
    // operand rows are the columns of x; K runs over the rows of x.  A warp reads 32 consecutive columns of one row at a time.
    uint8_t* sf = sf_col + (static_cast<size_t>(blockIdx.x) * rblocks + blockIdx.y) * 512 + (i & 31) * 16 + (i >> 5) * 4;
#pragma unroll
    for (int bb = 0; bb < 2; ++bb) {
      const int j = half * 2 + bb;
      const __nv_bfloat16* src = tile + (j * 32) * kPitch + i;
      float amax = 0.f;
#pragma unroll
      for (int t = 0; t < 32; ++t) amax = fmaxf(amax, fabsf(__bfloat162float(src[t * kPitch])));
      const bool live = c0 + i < C && r0 + j * 32 < R;
      const int e = live ? block_exponent(amax, fmax) : 0;
      sf[j] = static_cast<uint8_t>(e + 127);
      if (live) {
        const float inv = exp2_int(-e);
        uint32_t w[8];
#pragma unroll
        for (int t = 0; t < 8; ++t)
          w[t] = cvt4(__bfloat162float(src[(4 * t) * kPitch]) * inv, __bfloat162float(src[(4 * t + 1) * kPitch]) * inv,
                      __bfloat162float(src[(4 * t + 2) * kPitch]) * inv, __bfloat162float(src[(4 * t + 3) * kPitch]) * inv, fmt);
        uint4* dst = reinterpret_cast<uint4*>(q_col + static_cast<size_t>(c0 + i) * R + r0 + j * 32);  // R % 32 == 0
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
  }
}

}  // namespace mxq
}  // namespace lvb

// x [R, C] bf16 (C and the row stride ldx multiples of 8 elements; 16-byte aligned) -> q_row [R, C] + sf_row and / or q_col [C, R] + sf_col
// (either pair may be null).  fmt: 0 = e4m3, 1 = e5m2.  q_row needs C % 32 == 0, q_col needs R % 32 == 0; the scale arrays have
// lvb_mxfp8_sf_bytes(R, round_up(C, 128)) and lvb_mxfp8_sf_bytes(C, round_up(R, 128)) bytes and are written completely.
extern "C" int lvb_mxfp8_quantize(const void* x, long long ldx, int R, int C, int fmt, void* q_row, void* sf_row, void* q_col,
                                  void* sf_col, void* stream) {
  using namespace lvb;
  if (R <= 0 || C <= 0 || (ldx & 7) || (C & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || fmt < 0 || fmt > 1) return kErrBadArg;
  if ((q_row == nullptr) != (sf_row == nullptr) || (q_col == nullptr) != (sf_col == nullptr)) return kErrBadArg;
  if ((q_row != nullptr && (C & 31)) || (q_col != nullptr && (R & 31))) return kErrBadArg;
  if ((reinterpret_cast<uintptr_t>(q_row) & 15) || (reinterpret_cast<uintptr_t>(q_col) & 15)) return kErrBadArg;
  dim3 grid((C + 127) / 128, (R + 127) / 128);
  mxq::mxfp8_quant_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, R, C, fmt, reinterpret_cast<uint8_t*>(q_row), reinterpret_cast<uint8_t*>(sf_row),
      reinterpret_cast<uint8_t*>(q_col), reinterpret_cast<uint8_t*>(sf_col));
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
