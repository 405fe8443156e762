// Block-scaled fp8 GEMM on sm_100a (tcgen05.mma kind::mxf8f6f4 with block_scale).
//
//   C[M,N] = alpha * sum_k (A[m,k] * 2^(sfa[m, k/32] - 127)) * (B[n,k] * 2^(sfb[n, k/32] - 127))   (+ bias[N]) (+ C)
//
// A [M,K] and B [N,K] are one-byte floats (e4m3 or e5m2), K contiguous; every run of 32 values along K of every row has its
// own power-of-two scale (one byte, the exponent biased by 127: the OCP "MX" format).  The tensor core applies the scales
// itself: they sit in tensor memory beside the accumulator, one byte per (row, 32 values), and each K = 32 instruction names
// which byte to use.  Against per-tensor scaling (gemm_bf16.cu, kind::f8f6f4) nothing is pre- or post-multiplied on CUDA
// cores and an outlier costs precision only inside its own block of 32.
//
// Scale factors in global memory are stored the way the hardware wants them copied: for every (128 rows, 128 values of K)
// a chunk of 512 bytes, byte (r % 32) * 16 + (r / 32) * 4 + j for row r and the j-th block of 32; chunks ordered
// [row block][K block].  One untiled bulk copy brings a chunk into shared memory and one tcgen05.cp (32 lanes x 128 bits,
// replicated to the four lane quarters) puts it into four TMEM columns: column c holds rows 32c..32c+31, byte j of the column
// the scale of K block j.  mxfp8_quant.cu writes this layout.
//
// Structure as the other GEMMs here: warp 0 TMA producer, warp 1 MMA issuer (one elected thread: per 128-wide K block it
// issues the scale copies and four K = 32 MMAs, then commits the stage), warps 2-5 epilogue; persistent over 128 x BN tiles.
// BN = 128 keeps two accumulators so the epilogue of a tile overlaps the next tile's main loop; BN = 256 has one (the 512
// TMEM columns also hold the scales).  Every wait is bounded (common.cuh).
#include "common.cuh"

namespace lvb {
namespace mx {

constexpr int BM = 128;
constexpr int BK = 128;  // fp8 values (= bytes) of K per stage: one 128-byte swizzle row
constexpr int kThreads = 192;
constexpr int kSfChunk = 512;

enum Flags : int { kOutF32 = 1, kAccumulate = 2, kBias = 4, kBiasF32 = 16 };

struct Params {
  void* C;
  const void* bias;
  const uint8_t* sfa;  // [ceil(M/128)][K/128][512]
  const uint8_t* sfb;  // [ceil(N/128)][K/128][512]
  int M, N, K;
  int ldc;
  int flags;
  float alpha;
  int a_fmt, b_fmt;  // 0 = e4m3, 1 = e5m2
  int tiles_m, tiles_n;
  int* status;
};

template <int BN>
struct Cfg {
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = BN * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSfBytes = kSfChunk * (1 + BN / 128);
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kAccBufs = BN == 256 ? 1 : 2;
  static constexpr int kSfCol0 = 256;  // scale columns start behind the accumulators
  static constexpr int kSfColsPerStage = 16;
  static constexpr int kTiles = kStages * kStageBytes;
  static constexpr int kSf = kTiles;
  static constexpr int kBars = kSf + kStages * kSfBytes;
  static constexpr int kTotal = kBars + 256 + 1024;
};

// Instruction descriptor of the block-scaled fp8 MMA: both operands K-major, scales E8M0, fp32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_mx(int m, int n, int a_fmt, int b_fmt) {
  return (static_cast<uint32_t>(a_fmt) << 7) | (static_cast<uint32_t>(b_fmt) << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24);
}
// which byte of the scale columns this instruction uses (the j-th block of 32 inside the 128-wide K block), for A and B
__device__ __forceinline__ uint32_t idesc_with_sf(uint32_t idesc, uint32_t j) { return idesc | (j << 29) | (j << 4); }

__device__ __forceinline__ void umma_mxf8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                             uint32_t tmem_sfa, uint32_t tmem_sfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
// 32 rows x 16 bytes of shared memory (512 contiguous bytes, no swizzle) -> 4 TMEM columns, replicated to every lane quarter
__device__ __forceinline__ void tmem_cp_sf(uint32_t tmem_dst, uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(128 >> 4) << 32;  // 8-row groups of 16-byte rows are 128 bytes apart
  d |= static_cast<uint64_t>(1) << 46;         // descriptor version for sm_100; no swizzle
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(d) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  using L = Cfg<BN>;
  constexpr int kStages = L::kStages;
  constexpr int kAccBufs = L::kAccBufs;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int k_blocks = p.K / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<512>(tmem_holder);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int mb = t % p.tiles_m, nb = t / p.tiles_m;  // row blocks fastest: the CTAs running together share B tiles
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 100, stage);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* ssf = smem + L::kSf + stage * L::kSfBytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes + L::kSfBytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, mb * BM);
          tma_load_2d(sa + L::kABytes, &tmB, &full_bar[stage], kb * BK, nb * BN);
          bulk_load(ssf, p.sfa + (static_cast<size_t>(mb) * k_blocks + kb) * kSfChunk, kSfChunk, &full_bar[stage]);
#pragma unroll
          for (int j = 0; j < BN / 128; ++j)
            bulk_load(ssf + (1 + j) * kSfChunk, p.sfb + (static_cast<size_t>(nb * (BN / 128) + j) * k_blocks + kb) * kSfChunk, kSfChunk,
                      &full_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_mx(BM, BN, p.a_fmt, p.b_fmt);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t tphase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        ok = mbar_wait(&tempty_bar[buf], tphase ^ 1, abort_flag, p.status, 200, buf);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 201, stage);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t ssf = smem_u32(smem + L::kSf + stage * L::kSfBytes);
          const uint32_t tsfa = tmem_base + L::kSfCol0 + stage * L::kSfColsPerStage;
          const uint32_t tsfb = tsfa + 4;
          tmem_cp_sf(tsfa, ssf);
#pragma unroll
          for (int j = 0; j < BN / 128; ++j) tmem_cp_sf(tsfb + 4 * j, ssf + (1 + j) * kSfChunk);
          const uint64_t adesc = make_smem_desc(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc(sa + L::kABytes, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_mxf8_ss(tmem_acc, adesc + k * 2, bdesc + k * 2, idesc_with_sf(idesc, k), (kb > 0 || k > 0) ? 1u : 0u, tsfa, tsfb);
          umma_commit(&empty_bar[stage]);  // frees the stage (tiles and scale chunks) once the copies and MMAs retired
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[buf]);
        if (++buf == kAccBufs) { buf = 0; tphase ^= 1; }
      }
    }
  } else {
    const int quad = warp & 3;
    int buf = 0;
    uint32_t tphase = 0;
    bool ok = true;
    const bool out_f32 = (p.flags & kOutF32) != 0;
    const bool accum = (p.flags & kAccumulate) != 0;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int mb = t % p.tiles_m, nb = t / p.tiles_m;
      ok = mbar_wait(&tfull_bar[buf], tphase, abort_flag, p.status, 300, buf);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = mb * BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        const int col0 = nb * BN + c;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          const bool full = (col0 + 32 <= p.N);
          if (p.flags & kBias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N)
                v[j] += (p.flags & kBiasF32) ? reinterpret_cast<const float*>(p.bias)[col0 + j]
                                             : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + j]);
          }
          if (out_f32) {
            float* cp = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            if (full && (p.ldc & 3) == 0) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                if (accum) {
                  const float4 old = reinterpret_cast<const float4*>(cp)[q];
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                reinterpret_cast<float4*>(cp)[q] = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) cp[j] = accum ? cp[j] + v[j] : v[j];
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            if (full && (p.ldc & 7) == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
                o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
                o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
                o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
                reinterpret_cast<uint4*>(cp)[q] = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) cp[j] = __float2bfloat16(v[j]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      if (++buf == kAccBufs) { buf = 0; tphase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

template <int BN>
int launch(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream) {
  using L = Cfg<BN>;
  static_assert(L::kTotal <= 232448, "exceeds the shared memory of an SM");
  static_assert(L::kSfCol0 + L::kStages * L::kSfColsPerStage <= 512 && L::kAccBufs * BN <= L::kSfCol0, "TMEM columns");
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d_u8(&tmA, A, p.M, p.K, lda, BM);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_u8(&tmB, B, p.N, p.K, ldb, BN);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_mxfp8_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  int grid = p.tiles_m * p.tiles_n;
  if (grid > num_sms()) grid = num_sms();
  kern<<<grid, kThreads, L::kTotal, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace mx
}  // namespace lvb

// Bytes of the scale-factor array of an operand with `rows` rows and K values per row (K a multiple of 128).
extern "C" long long lvb_mxfp8_sf_bytes(int rows, int K) { return static_cast<long long>((rows + 127) / 128) * (K / 128) * 512; }

// C[M,N] = alpha * A B^T with block scales (see the head of this file).  K % 128 == 0; lda / ldb in bytes, multiples of 16;
// sfa / sfb in the chunked layout (lvb_mxfp8_sf_bytes bytes each, 16-byte aligned), rows beyond M / N of the last chunk must
// hold finite scales (the quantiser writes 127).  flags: 1 = fp32 C, 2 = C += (fp32 C only), 4 = bias, 16 = bias is fp32.
// bn: tile width 128 or 256, 0 = chosen here.
extern "C" int lvb_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, int lda,
                              int ldb, int ldc, int a_fmt, int b_fmt, int flags, float alpha, const void* bias, int bn, int* status,
                              void* stream) {
  using namespace lvb;
  using namespace lvb::mx;
  if (M <= 0 || N <= 0 || K <= 0 || (K % BK) != 0 || (lda & 15) || (ldb & 15) || a_fmt < 0 || a_fmt > 1 || b_fmt < 0 || b_fmt > 1)
    return kErrBadArg;
  if (sfa == nullptr || sfb == nullptr || (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15)) return kErrBadArg;
  if ((flags & kAccumulate) && !(flags & kOutF32)) return kErrBadArg;
  Params p;
  p.C = C; p.bias = bias;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa); p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.flags = flags; p.alpha = alpha;
  p.a_fmt = a_fmt; p.b_fmt = b_fmt; p.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 0) bn = (N > 128 && ((M + 127) / 128) * ((N + 255) / 256) >= num_sms()) ? 256 : 128;
  if (bn == 256) return mx::launch<256>(A, B, p, lda, ldb, s);
  if (bn == 128) return mx::launch<128>(A, B, p, lda, ldb, s);
  return kErrBadArg;
}
