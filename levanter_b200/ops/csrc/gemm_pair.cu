// bf16 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
//   C[M,N] = alpha * op(A) * op(B)^T (+ bias[N]) (+ residual[M,N]) (+ C if accumulate)
//
// Two CTAs of a cluster work on one 256 x BN tile.  CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and
// columns [BN/2 r, BN/2 r + BN/2) of the B tile into its own shared memory (TMA, no multicast: every byte is loaded once
// by exactly one CTA); ONE thread of the leader CTA issues tcgen05.mma.cta_group::2 (M = 256, N = BN, K = 16), which reads
// both halves of both operands and accumulates rows [128 r, ...) of the tile in CTA r's tensor memory.  Compared with a
// 128 x 256 tile per CTA this halves the shared-memory traffic of the B operand per flop (the limit of the single-CTA
// kernel in gemm_bf16.cu) and leaves room for a six-stage ring.
//
// Synchronisation (all waits bounded, see common.cuh):
//   full[s]   in the LEADER's shared memory: the leader's producer posts the expected bytes of both CTAs' loads, and both
//             CTAs' TMA loads complete on it (the follower addresses it by clearing the CTA-rank bit of its own barrier's
//             shared-memory address);
//   empty[s]  in each CTA: the leader's tcgen05.commit arrives on both CTAs' copies once the MMAs reading stage s retired;
//   tfull[b]  in each CTA: same mechanism, accumulator b complete;
//   tempty[b] in the leader: the four epilogue warps of each CTA arrive on it (remote arrive from the follower).
// Operand majorness as in gemm_bf16.cu (K-major / MN-major through the UMMA descriptors).
//
// Replaces the dense projections that the reference lowers through XLA dots (hnn.Linear -> hax.dot;
// src/levanter/layers/attention.py:1606-1635, src/levanter/models/llama.py:273-280).
#include "common.cuh"

namespace lvb {
namespace gemm2 {

constexpr int BMC = 128;  // rows of C per CTA
constexpr int BMP = 256;  // rows of C per CTA pair
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kNumThreads = 192;  // warp0 TMA, warp1 MMA (leader) / TMEM allocation, warps2-5 epilogue
constexpr uint32_t kLeaderMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared-memory address: the leader's copy

enum EpiFlags : int { kOutF32 = 1, kAccumulate = 2, kBias = 4, kResidual = 8, kBiasF32 = 16 };

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
};

template <int BN>
struct Smem {
  static constexpr int kABytes = BMC * BK * 2;
  static constexpr int kBBytes = (BN / 2) * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = 196608 / kStageBytes;
  static constexpr int kTileBytes = kStages * kStageBytes;
  static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kTotal = kTileBytes + kBarBytes + 1024;
};

// ---------------------------------------------------------------- cluster / pair helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t n_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the leader CTA's copy of a barrier (the barrier sits at the same offset in both CTAs).
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(0));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// 2-D tiled load into this CTA's shared memory, completion on the LEADER's barrier (no multicast).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & kLeaderMask), "r"(x), "r"(y)
      : "memory");
}
template <int kCols>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_holder) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)), "r"(kCols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int kCols>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(kCols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of both CTAs] * B[smem of both CTAs]; issued by ONE thread of the leader CTA.
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this offset in BOTH CTAs of the pair once all MMAs issued so far by this thread completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  constexpr int GM = 4;  // 4 pair-tiles = 1024 rows of A stay hot in L2 while the raster sweeps N
  int group_size = GM * tiles_n;
  int g = t / group_size;
  int first_m = g * GM;
  int gm = min(GM, tiles_m - first_m);
  int r = t - g * group_size;
  mb = first_m + (r % gm);
  nb = r / gm;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  using L = Smem<BN>;
  constexpr int kStages = L::kStages;
  constexpr int BNH = BN / 2;  // columns of the B tile held by one CTA
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
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int first_tile = static_cast<int>(cluster_id_x());
  const int tile_step = static_cast<int>(n_clusters_x());

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8);  // one arrival per epilogue warp of either CTA
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair<2 * BN>(tmem_holder);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
        int mb, nb;
        tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
        const int m0 = mb * BMP + static_cast<int>(cta) * BMC;  // this CTA's rows of the tile
        const int n0 = nb * BN + static_cast<int>(cta) * BNH;   // this CTA's columns of the B tile
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 100, stage);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);  // both CTAs' loads of this stage
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BMC / 64; ++c) tma_load_2d_pair(sa + c * (64 * BK * 2), &tmA, &full_bar[stage], m0 + 64 * c, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmB, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c) tma_load_2d_pair(sb + c * (64 * BK * 2), &tmB, &full_bar[stage], n0 + 64 * c, k0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta == 0) {
      const uint32_t idesc = make_idesc_bf16(BMP, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t tphase = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
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
          const uint64_t adesc = A_MN ? make_smem_desc(sa, 64 * BK * 2, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t bdesc = B_MN ? make_smem_desc(sb, 64 * BK * 2, 1024) : make_smem_desc(sb, 16, 1024);
          constexpr uint32_t a_step = (A_MN ? 2048 : 32) >> 4;
          constexpr uint32_t b_step = (B_MN ? 2048 : 32) >> 4;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_ss_pair(tmem_acc, adesc + k * a_step, bdesc + k * b_step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);  // frees the stage in both CTAs when the MMAs retire
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[buf]);  // accumulator complete, in both CTAs
        if (++buf == 2) { buf = 0; tphase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (four warps per CTA, this CTA's 128 rows)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    int buf = 0;
    uint32_t tphase = 0;
    bool ok = true;
    const bool out_f32 = (p.flags & kOutF32) != 0;
    const bool accum = (p.flags & kAccumulate) != 0;
    const float alpha = p.alpha;
    for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
      int mb, nb;
      tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      ok = mbar_wait(&tfull_bar[buf], tphase, abort_flag, p.status, 300, buf);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = mb * BMP + static_cast<int>(cta) * BMC + quad * 32 + lane;
      const int n0 = nb * BN;
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
            float* cp = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            if (full && (p.ldc & 3) == 0) {
              if (accum) {
                // C += tile as vector reductions resolved in L2; every element has exactly one adder per launch, so the
                // sum stays deterministic
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + 4 * q), "f"(v[4 * q]), "f"(v[4 * q + 1]),
                               "f"(v[4 * q + 2]), "f"(v[4 * q + 3])
                               : "memory");
              } else {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  reinterpret_cast<float4*>(cp)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
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
                if (col0 + j < p.N) cp[j] = __float2bfloat16(accum ? __bfloat162float(cp[j]) + v[j] : v[j]);
            }
          }
        }
      }
      // all TMEM reads of this warp are complete (tmem_ld_wait above)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty_bar[buf]);
      if (++buf == 2) { buf = 0; tphase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA releases tensor memory or leaves while its peer may still signal or accumulate into it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair<2 * BN>(tmem_base);
  }
}

template <int BN, bool A_MN, bool B_MN>
int launch(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream, int max_ctas) {
  using L = Smem<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(&tmA, A, p.M, p.K, lda, BMC, BK);  // [M,K] rows=M
  else       rc = make_tmap_2d_bf16(&tmA, A, p.K, p.M, lda, BK, 64);   // [K,M] rows=K, box 64 k x 64 m
  if (rc != kErrOk) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tmB, B, p.N, p.K, ldb, BN / 2, BK);
  else       rc = make_tmap_2d_bf16(&tmB, B, p.K, p.N, ldb, BK, 64);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BMP - 1) / BMP;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_pair_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  int pairs = p.tiles_m * p.tiles_n;
  // as many pairs as can be resident at once (a GPC with an odd number of free SMs cannot host a pair on the last one)
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (num_sms() / 2));
    cfg.blockDim = dim3(kNumThreads);
    cfg.dynamicSmemBytes = L::kTotal;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = num_sms() / 2;
    }
    max_pairs = n;
  }
  int cap = max_pairs;
  if (max_ctas > 0 && max_ctas / 2 < cap) cap = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (pairs > cap) pairs = cap;
  kern<<<2 * pairs, kNumThreads, L::kTotal, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace gemm2
}  // namespace lvb

// The CTA-pair form of lvb_gemm_bf16 (same arguments and semantics).  N must exceed 128; lda / ldb multiples of 8.
extern "C" int lvb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                                  int b_mn, int flags, float alpha, const void* bias, const void* residual, int ldr, int max_ctas,
                                  int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm2;
  if (M <= 0 || N <= 128 || K <= 0) return kErrBadArg;
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
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch<256, false, false>(A, B, p, lda, ldb, s, max_ctas);
  if (!a_mn && b_mn) return launch<256, false, true>(A, B, p, lda, ldb, s, max_ctas);
  if (a_mn && b_mn) return launch<256, true, true>(A, B, p, lda, ldb, s, max_ctas);
  return launch<256, true, false>(A, B, p, lda, ldb, s, max_ctas);
}
