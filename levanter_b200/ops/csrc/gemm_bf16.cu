// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] = alpha * op(A) * op(B)^T (+ bias[N]) (+ residual[M,N]) (+ C if accumulate)
//
//   * operands arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a
//     kStages-deep shared-memory ring,
//   * one thread issues tcgen05.mma (M=128, N=BN, K=16) with the fp32
//     accumulator in tensor memory; two accumulators (2*BN TMEM columns) let the
//     epilogue of tile i overlap the main loop of tile i+1,
//   * four epilogue warps read the accumulator with tcgen05.ld (one row per
//     thread), apply the epilogue and store 64-byte row segments.
//
// Operand majorness.  "K-major" means the reduction index is contiguous in
// memory, "MN-major" that the row (A) / column (B) index is contiguous:
//   forward      Y[T,N]  = X[T,K]  W[N,K]^T      A K-major,  B K-major
//   grad input   dX[T,K] = dY[T,N] W[N,K]        A K-major,  B MN-major
//   grad weight  dW[N,K] = dY[T,N]^T X[T,K]      A MN-major, B MN-major
// so no operand is ever transposed in memory.
//
// This GEMM covers the dense projections that the reference lowers through
// XLA dots (hnn.Linear -> hax.dot; src/levanter/layers/attention.py:1606-1635,
// src/levanter/models/llama.py:273-280).
#include "common.cuh"

namespace lvb {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;     // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kNumThreads = 192;  // warp0 TMA, warp1 MMA, warps2-5 epilogue
constexpr int kMaxPeers = 8;

enum EpiFlags : int {
  kOutF32 = 1,       // C is float (else bf16)
  kAccumulate = 2,   // C += result
  kBias = 4,         // + bias[N] (bf16)
  kResidual = 8,     // + residual[M,N] (bf16, row stride ldr)
  kBiasF32 = 16,     // bias is float
};

struct Params {
  void* C;
  const void* bias;
  const __nv_bfloat16* residual;
  int M, N, K;
  int ldc, ldr;
  int flags;
  float alpha;
  int tiles_m, tiles_n;
  int* status;
  const float* alpha_dev;  // optional device scalar multiplied into alpha (fp8: product of the two operand scales)
  int a_fmt, b_fmt;        // fp8 only: 0 = e4m3, 1 = e5m2
  // fused collectives (0 = off).  a_rows_per_map: rows [r * a_rows_per_map, (r + 1) * a_rows_per_map) of A live in rank r's
  // memory and are fetched through tensor map r (all-gather fused into the operand loads).  c_rows_per_rank: rows of C in
  // that range are stored to c_peer[r] (this rank's slot in rank r's staging buffer: the scatter half of a reduce-scatter).
  int a_rows_per_map;
  int c_rows_per_rank;
  void* c_peer[kMaxPeers];
};

struct PeerMaps {
  CUtensorMap maps[kMaxPeers];
};

template <int BN>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kTileBytes = kStages * kStageBytes;
  // barriers: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kTotal = kTileBytes + kBarBytes + 1024;  // +1024 for manual alignment
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  constexpr int GM = 8;
  int group_size = GM * tiles_n;
  int g = t / group_size;
  int first_m = g * GM;
  int gm = min(GM, tiles_m - first_m);
  int r = t - g * group_size;
  mb = first_m + (r % gm);
  nb = r / gm;
}

// kF8: one-byte operands (both K-major); a stage row is still 128 bytes, i.e. 128 elements of K instead of 64.
template <int BN, bool A_MN, bool B_MN, bool kF8 = false>
__device__ __forceinline__ void gemm_body(const CUtensorMap* tmA_maps, const CUtensorMap& tmB, const Params& p) {
  const CUtensorMap& tmA = tmA_maps[0];
  using L = SmemLayout<BN>;
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kTileBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  constexpr int BKE = kF8 ? 2 * BK : BK;  // elements of K per stage
  const int k_blocks = (p.K + BKE - 1) / BKE;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);  // one arrival per epilogue warp
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<2 * BN>(tmem_holder);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 100, stage);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          const int k0 = kb * BKE;
          if constexpr (!A_MN) {
            if (p.a_rows_per_map > 0) {
              const int r = m0 / p.a_rows_per_map;  // the rank whose memory holds these rows
              tma_load_2d(sa, tmA_maps + r, &full_bar[stage], k0, m0 - r * p.a_rows_per_map);
            } else {
              tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (64 * BK * 2), &tmA, &full_bar[stage], m0 + 64 * c, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &tmB, &full_bar[stage], n0 + 64 * c, k0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = kF8 ? make_idesc_f8(BM, BN, p.a_fmt, p.b_fmt) : make_idesc_bf16(BM, BN, A_MN, B_MN);
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
          const uint32_t sb = sa + L::kABytes;
          // K-major: 8-row groups are 1024 B apart (SBO); a K step of 16
          // elements moves 32 B inside the swizzle row.
          // MN-major: 64-element chunks are 64*BK*2 B apart (LBO), 8-k groups
          // 1024 B apart (SBO); a K step of 16 moves two groups (2048 B).
          const uint64_t adesc = A_MN ? make_smem_desc(sa, 64 * BK * 2, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t bdesc = B_MN ? make_smem_desc(sb, 64 * BK * 2, 1024) : make_smem_desc(sb, 16, 1024);
          constexpr uint32_t a_step = (A_MN ? 2048 : 32) >> 4;
          constexpr uint32_t b_step = (B_MN ? 2048 : 32) >> 4;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if constexpr (kF8) umma_f8_ss(tmem_acc, adesc + k * a_step, bdesc + k * b_step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma_bf16_ss(tmem_acc, adesc + k * a_step, bdesc + k * b_step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage when the MMAs retire
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[buf]);  // accumulator complete
        if (++buf == 2) { buf = 0; tphase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    int buf = 0;
    uint32_t tphase = 0;
    bool ok = true;
    const bool out_f32 = (p.flags & kOutF32) != 0;
    const bool accum = (p.flags & kAccumulate) != 0;
    const float alpha = p.alpha_dev != nullptr ? p.alpha * p.alpha_dev[0] : p.alpha;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      ok = mbar_wait(&tfull_bar[buf], tphase, abort_flag, p.status, 300, buf);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = mb * BM + quad * 32 + lane;
      const int n0 = nb * BN;
      void* c_base = p.C;
      size_t c_row = static_cast<size_t>(row);
      if (p.c_rows_per_rank > 0 && row < p.M) {
        const int d = row / p.c_rows_per_rank;
        c_base = p.c_peer[d];
        c_row = static_cast<size_t>(row - d * p.c_rows_per_rank);
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        const int col0 = n0 + c;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
          const bool full = (col0 + 32 <= p.N);
          if (p.flags & kBias) {
            if (p.flags & kBiasF32) {
              const float* b = reinterpret_cast<const float*>(p.bias) + col0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (full || col0 + j < p.N) v[j] += b[j];
            } else {
              const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (full || col0 + j < p.N) v[j] += __bfloat162float(b[j]);
            }
          }
          if (p.flags & kResidual) {
            const __nv_bfloat16* rr = p.residual + static_cast<size_t>(row) * p.ldr + col0;
            if (full && (p.ldr & 7) == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 w = reinterpret_cast<const uint4*>(rr)[q];
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 f = __bfloat1622float2(h[j]);
                  v[q * 8 + 2 * j] += f.x;
                  v[q * 8 + 2 * j + 1] += f.y;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(rr[j]);
            }
          }
          if (out_f32) {
            float* cp = reinterpret_cast<float*>(c_base) + c_row * p.ldc + col0;
            if (full && (p.ldc & 3) == 0) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                if (accum) {
                  float4 old = reinterpret_cast<float4*>(cp)[q];
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
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(c_base) + c_row * p.ldc + col0;
            if (full && (p.ldc & 7) == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if (accum) {
                  uint4 w = reinterpret_cast<const uint4*>(cp)[q];
                  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float2 f = __bfloat1622float2(h[j]);
                    v[q * 8 + 2 * j] += f.x;
                    v[q * 8 + 2 * j + 1] += f.y;
                  }
                }
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
                if (col0 + j < p.N)
                  cp[j] = __float2bfloat16(accum ? __bfloat162float(cp[j]) + v[j] : v[j]);
            }
          }
        }
      }
      // all TMEM reads of this warp are complete (tmem_ld_wait above)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      if (++buf == 2) { buf = 0; tphase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2 * BN>(tmem_base);
  }
}

template <int BN, bool A_MN, bool B_MN, bool kF8 = false>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_body<BN, A_MN, B_MN, kF8>(&tmA, tmB, p);
}

// A's row blocks come from different ranks' memories: one tensor map per rank (plain TMA loads, no cluster qualifier).
template <int BN>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_gathered_a_kernel(const __grid_constant__ PeerMaps tmAs, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_body<BN, false, false, false>(tmAs.maps, tmB, p);
}

template <int BN, bool A_MN, bool B_MN>
int launch(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream, int max_ctas) {
  using L = SmemLayout<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(&tmA, A, p.M, p.K, lda, BM, BK);   // [M,K] rows=M
  else       rc = make_tmap_2d_bf16(&tmA, A, p.K, p.M, lda, BK, 64);   // [K,M] rows=K, box 64 k x 64 m
  if (rc != kErrOk) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tmB, B, p.N, p.K, ldb, BN, BK);
  else       rc = make_tmap_2d_bf16(&tmB, B, p.K, p.N, ldb, BK, 64);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess)
      return kErrCuda;
    attr_set = true;
  }
  int grid = p.tiles_m * p.tiles_n;
  int cap = num_sms();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  kern<<<grid, kNumThreads, L::kTotal, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace gemm
}  // namespace lvb

// C[M,N] = alpha * op(A) op(B)^T ...   (see the header of this file)
//   a_mn / b_mn : 0 = K-major operand ([M,K] / [N,K] row-major, row stride lda / ldb),
//                 1 = MN-major operand ([K,M] / [K,N] row-major).
//   flags       : lvb::gemm::EpiFlags
//   max_ctas    : 0 = one CTA per SM; otherwise an upper bound on the grid (leaves
//                 SMs free for a concurrent communication kernel).
//   status      : device int32[8], may be null.
extern "C" int lvb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                             int ldc, int a_mn, int b_mn, int flags, float alpha, const void* bias,
                             const void* residual, int ldr, int max_ctas, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return kErrBadArg;
  if ((lda & 7) || (ldb & 7)) return kErrBadArg;
  Params p;
  p.C = C;
  p.bias = bias;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.flags = flags;
  p.alpha = alpha;
  p.status = status;
  p.alpha_dev = nullptr;
  p.a_fmt = p.b_fmt = 0;
  p.a_rows_per_map = 0;
  p.c_rows_per_rank = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool wide = (N > 128);
  if (wide) {
    if (!a_mn && !b_mn) return launch<256, false, false>(A, B, p, lda, ldb, s, max_ctas);
    if (!a_mn && b_mn) return launch<256, false, true>(A, B, p, lda, ldb, s, max_ctas);
    if (a_mn && b_mn) return launch<256, true, true>(A, B, p, lda, ldb, s, max_ctas);
    return launch<256, true, false>(A, B, p, lda, ldb, s, max_ctas);
  } else {
    if (!a_mn && !b_mn) return launch<128, false, false>(A, B, p, lda, ldb, s, max_ctas);
    if (!a_mn && b_mn) return launch<128, false, true>(A, B, p, lda, ldb, s, max_ctas);
    if (a_mn && b_mn) return launch<128, true, true>(A, B, p, lda, ldb, s, max_ctas);
    return launch<128, true, false>(A, B, p, lda, ldb, s, max_ctas);
  }
}


namespace lvb {
namespace gemm {

template <int BN>
int launch_f8(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream, int max_ctas) {
  using L = SmemLayout<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d_u8(&tmA, A, p.M, p.K, lda, BM);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_u8(&tmB, B, p.N, p.K, ldb, BN);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_kernel<BN, false, false, true>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  int grid = p.tiles_m * p.tiles_n;
  int cap = num_sms();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  kern<<<grid, kNumThreads, L::kTotal, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace gemm
}  // namespace lvb

// fp8 GEMM with per-tensor scales: C[M,N] = alpha * scale[0] * A[M,K] B[N,K]^T (+ C if accumulate).
//   A, B   : one-byte floats, K contiguous (row strides lda / ldb bytes, multiples of 16); a_fmt / b_fmt: 0 = e4m3, 1 = e5m2
//   scale  : optional device fp32 scalar (the product of the operands' de-quantisation scales), so no host sync is needed
//   flags  : kOutF32 / kAccumulate / kBias / kBiasF32 / kResidual as for lvb_gemm_bf16; C is bf16 unless kOutF32
extern "C" int lvb_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_fmt,
                            int b_fmt, int flags, float alpha, const float* scale, const void* bias, const void* residual,
                            int ldr, int max_ctas, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 15) || (ldb & 15) || a_fmt < 0 || a_fmt > 1 || b_fmt < 0 || b_fmt > 1) return kErrBadArg;
  Params p;
  p.C = C;
  p.bias = bias;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.flags = flags;
  p.alpha = alpha;
  p.status = status;
  p.alpha_dev = scale;
  p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.a_rows_per_map = 0;
  p.c_rows_per_rank = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return N > 128 ? launch_f8<256>(A, B, p, lda, ldb, s, max_ctas) : launch_f8<128>(A, B, p, lda, ldb, s, max_ctas);
}


// ---------------------------------------------------------------------------------------------------------------------
// Tensor-parallel GEMMs with the collective fused in (sequence-parallel layout: activations are split by rows over ranks).
namespace lvb {
namespace gemm {

template <int BN>
int launch_gathered_a(const void* const* a_peers, const void* B, Params p, int world, int lda, int ldb, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  PeerMaps maps;
  CUtensorMap tmB;
  for (int r = 0; r < world; ++r) {
    int rc = make_tmap_2d_bf16(&maps.maps[r], a_peers[r], p.a_rows_per_map, p.K, lda, BM, BK);
    if (rc != kErrOk) return rc;
  }
  for (int r = world; r < kMaxPeers; ++r) maps.maps[r] = maps.maps[0];
  int rc = make_tmap_2d_bf16(&tmB, B, p.N, p.K, ldb, BN, BK);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_gathered_a_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  int grid = p.tiles_m * p.tiles_n;
  if (grid > num_sms()) grid = num_sms();
  kern<<<grid, kNumThreads, L::kTotal, stream>>>(maps, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace gemm
}  // namespace lvb

// All-gather fused into a GEMM: C[M, N] = concat_r(A_r)[M, K] B[N, K]^T where A_r [M / world, K] (bf16, row stride lda)
// is rank r's shard, read in place from rank r's memory by TMA (a_peers[r]: device pointer valid on this GPU; own rank
// included).  M / world must be a multiple of 128.  The caller orders the ranks (every A_r complete before the launch).
extern "C" int lvb_gemm_allgather_a(const void* const* a_peers, int world, const void* B, void* C, int M, int N, int K, int lda,
                                    int ldb, int ldc, int flags, float alpha, const void* bias, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (world <= 0 || world > kMaxPeers || M <= 0 || N <= 0 || K <= 0 || M % world != 0 || (M / world) % BM != 0) return kErrBadArg;
  if ((lda & 7) || (ldb & 7)) return kErrBadArg;
  Params p;
  p.C = C; p.bias = bias; p.residual = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = 0;
  p.flags = flags; p.alpha = alpha; p.status = status; p.alpha_dev = nullptr;
  p.a_fmt = p.b_fmt = 0;
  p.a_rows_per_map = M / world;
  p.c_rows_per_rank = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return N > 128 ? launch_gathered_a<256>(a_peers, B, p, world, lda, ldb, s) : launch_gathered_a<128>(a_peers, B, p, world, lda, ldb, s);
}

// The scatter half of a reduce-scatter fused into a GEMM epilogue: this rank's partial product P[M, N] = A[M, K] B[N, K]^T
// (K is the sharded dimension) is stored, rows [r * M / world, (r + 1) * M / world) to c_peers[r], which the caller points at
// this rank's slot of rank r's staging buffer [world, M / world, ldc].  Every rank then sums its own staging buffer over the
// slots (lvb_sum_slots).  Output dtype per flags (fp32 with kOutF32, else bf16).
extern "C" int lvb_gemm_scatter_c(const void* A, const void* B, void* const* c_peers, int world, int M, int N, int K, int lda,
                                  int ldb, int ldc, int flags, float alpha, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (world <= 0 || world > kMaxPeers || M <= 0 || N <= 0 || K <= 0 || M % world != 0) return kErrBadArg;
  if ((lda & 7) || (ldb & 7)) return kErrBadArg;
  Params p;
  p.C = c_peers[0]; p.bias = nullptr; p.residual = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = 0;
  p.flags = flags & kOutF32; p.alpha = alpha; p.status = status; p.alpha_dev = nullptr;
  p.a_fmt = p.b_fmt = 0;
  p.a_rows_per_map = 0;
  p.c_rows_per_rank = M / world;
  for (int r = 0; r < kMaxPeers; ++r) p.c_peer[r] = c_peers[r < world ? r : 0];
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return N > 128 ? launch<256, false, false>(A, B, p, lda, ldb, s, 0) : launch<128, false, false>(A, B, p, lda, ldb, s, 0);
}

namespace lvb {
namespace gemm {
__global__ void sum_slots_kernel(const float4* __restrict__ staging, long long slot4, int world, float4* __restrict__ out_f32,
                                 uint2* __restrict__ out_bf16, long long n4) {
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n4; i += gridDim.x * 256LL) {
    float4 s = staging[i];
    for (int r = 1; r < world; ++r) {
      const float4 v = staging[r * slot4 + i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    if (out_f32 != nullptr) out_f32[i] = s;
    if (out_bf16 != nullptr) out_bf16[i] = make_uint2(pack_bf16x2(s.x, s.y), pack_bf16x2(s.z, s.w));
  }
}
}  // namespace gemm
}  // namespace lvb

// out[n] = sum over slots of staging[slot][n] (fp32 staging, n a multiple of 4); bf16 and/or fp32 output.
extern "C" int lvb_sum_slots(const float* staging, long long slot_elems, int world, float* out_f32, void* out_bf16, long long n,
                             void* stream) {
  using namespace lvb;
  if (world <= 0 || n <= 0 || (n & 3) || (slot_elems & 3)) return kErrBadArg;
  long long blocks = (n / 4 + 255) / 256;
  long long cap = static_cast<long long>(num_sms()) * 8;
  gemm::sum_slots_kernel<<<static_cast<int>(blocks < cap ? blocks : cap), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(staging), slot_elems / 4, world, reinterpret_cast<float4*>(out_f32),
      reinterpret_cast<uint2*>(out_bf16), n / 4);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
