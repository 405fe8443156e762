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
// kScatter mode fuses a reduce-scatter over GPUs into the epilogue (the weight-gradient product of fully sharded training,
// or a row-parallel tensor-parallel output): every epilogue warp stores its 32 rows into the staging slot of the rank that
// owns them (peer stores over NVLink, row-contiguous 128-byte segments) and bumps that rank's arrival counter of the
// (32-row group, column tile) unit; four more warps per CTA sum this rank's own units over the slots as they fill.  The
// protocol (two alternating staging areas, counters that only grow, an ordered raster) is that of lvb_gemm_reduce_scatter
// in gemm_bf16.cu.
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
constexpr int kMaxPeers = 8;

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
  // ---- K split (kPlain): a piece of work is (tile, split); each split stores its raw fp32 partial tile to ws[split, M, N]
  // and a second kernel sums the slabs in order.  For products with far fewer tiles than SM pairs (decode-size M).
  int splits = 1;
  int kb_per_split = 0;
  float* ws = nullptr;
  // ---- reduce-scatter epilogue (kScatter)
  int rank, world;
  int c_rows_per_rank;       // rows [r * c_rows_per_rank, ...) of C belong to rank r (a multiple of 32)
  void* c_peer[kMaxPeers];   // this rank's slot in rank r's staging area
  int* c_cnt[kMaxPeers];     // rank r's arrival counters, one per (32-row group, column tile); they only ever grow
  int c_target;              // value of a counter once all `world` parts of this call's unit have arrived
  const int* c_m_order;      // the raster's i-th 256-row block is block c_m_order[i]
  const float* rs_staging;   // this rank's own staging area [world, slot]
  long long rs_slot;         // elements per slot
  void* rs_out;              // this rank's reduced rows [c_rows_per_rank, N] (fp32 or bf16), row stride rs_ldo
  int rs_ldo;
  int rs_out_f32;
  int rs_accumulate;         // add to rs_out (fp32 only) instead of storing
  // ---- copy job (kCopyJob): units [cj_u0, cj_u1) of a table of {source rank, source offset / 16, destination offset / 16,
  // bytes / 16}; a seventh warp of every CTA moves them (peer or local memory -> shared memory -> cj_dst) beside the GEMM
  const int4* cj_table;
  int cj_u0, cj_u1;
  const uint8_t* cj_src[kMaxPeers];
  uint8_t* cj_dst;
};

constexpr int kPlain = 0;
constexpr int kScatter = 1;
constexpr int kCopyJob = 2;
constexpr int kCopyUnit = 16384;                  // bytes per bulk copy of a copy job
constexpr int kCopyExtra = 256 + 2 * kCopyUnit;  // extra dynamic shared memory of the copy-job kernel
constexpr int kCopyThreads = kNumThreads + 32;
constexpr int kReduceThreads = 128;
constexpr int kScatterThreads = kNumThreads + kReduceThreads;
constexpr int kEpiStride = 36;  // floats per staged row (144 B: 16-byte aligned, conflict-free for float4 rows)
constexpr int kEpiExtra = 256 + 4 * 32 * kEpiStride * 4;

__device__ __forceinline__ void reduce_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kReduceThreads) : "memory"); }

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

template <int BN, bool A_MN, bool B_MN, int MODE>
__device__ __forceinline__ void gemm_pair_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p) {
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
  // scatter mode only: a 32 x 32 fp32 transposition buffer per epilogue warp behind the barriers
  float* epi_buf = reinterpret_cast<float*>(smem + ((L::kTileBytes + L::kBarBytes + 127) & ~127));
  // copy-job mode only: two copy barriers and two staging buffers in the same place
  uint64_t* copy_bar = reinterpret_cast<uint64_t*>(epi_buf);
  uint8_t* copy_buf = reinterpret_cast<uint8_t*>(copy_bar) + 128;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int splits = p.splits;
  const int kbps = splits > 1 ? p.kb_per_split : k_blocks;
  const int num_work = num_tiles * splits;  // the split index runs fastest
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
    if constexpr (MODE == kCopyJob) {
      mbar_init(&copy_bar[0], 1);
      mbar_init(&copy_bar[1], 1);
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
      for (int t = first_tile; t < num_work && ok; t += tile_step) {
        int mb, nb;
        tile_coords(t / splits, p.tiles_m, p.tiles_n, mb, nb);
        if constexpr (MODE == kScatter) mb = __ldg(p.c_m_order + mb);
        const int m0 = mb * BMP + static_cast<int>(cta) * BMC;  // this CTA's rows of the tile
        const int n0 = nb * BN + static_cast<int>(cta) * BNH;   // this CTA's columns of the B tile
        const int kb0 = (t % splits) * kbps;
        const int kb1 = min(k_blocks, kb0 + kbps);
        for (int kb = kb0; kb < kb1; ++kb) {
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
      for (int t = first_tile; t < num_work && ok; t += tile_step) {
        ok = mbar_wait(&tempty_bar[buf], tphase ^ 1, abort_flag, p.status, 200, buf);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        const int kb0 = (t % splits) * kbps;
        const int n_kb = min(k_blocks, kb0 + kbps) - kb0;
        for (int kb = 0; kb < n_kb; ++kb) {
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
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (four warps per CTA, this CTA's 128 rows)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    int buf = 0;
    uint32_t tphase = 0;
    bool ok = true;
    const bool out_f32 = (p.flags & kOutF32) != 0;
    const bool accum = (p.flags & kAccumulate) != 0;
    const float alpha = p.alpha;
    for (int t = first_tile; t < num_work && ok; t += tile_step) {
      int mb, nb;
      tile_coords(t / splits, p.tiles_m, p.tiles_n, mb, nb);
      if constexpr (MODE == kScatter) mb = __ldg(p.c_m_order + mb);
      ok = mbar_wait(&tfull_bar[buf], tphase, abort_flag, p.status, 300, buf);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = mb * BMP + static_cast<int>(cta) * BMC + quad * 32 + lane;
      const int n0 = nb * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
      // scatter mode: this warp's 32 rows belong to one rank (rows per rank and M are multiples of 32)
      const int row0w = row - lane;
      const bool c_live = row0w < p.M;
      int c_dest = 0;
      float* c_dst_row0 = nullptr;
      if constexpr (MODE == kScatter) {
        c_dest = c_live ? row0w / p.c_rows_per_rank : 0;
        c_dst_row0 = reinterpret_cast<float*>(p.c_peer[c_dest]) + static_cast<size_t>(row0w - c_dest * p.c_rows_per_rank) * p.ldc;
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        const int col0 = n0 + c;
        if constexpr (MODE == kScatter) {
          // Peer stores: turn the row-per-lane fragment into row-contiguous 128-byte segments through shared memory, so a
          // store instruction covers 4 rows x 128 B instead of 32 rows x 16 B (NVLink moves short writes poorly).
          if (col0 < p.N && c_live) {  // warp-uniform
            float* eb = epi_buf + (warp - 2) * (32 * kEpiStride);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<float4*>(eb + lane * kEpiStride + 4 * q) =
                  make_float4(__uint_as_float(r[4 * q]) * alpha, __uint_as_float(r[4 * q + 1]) * alpha,
                              __uint_as_float(r[4 * q + 2]) * alpha, __uint_as_float(r[4 * q + 3]) * alpha);
            __syncwarp();
            const int col = col0 + 4 * (lane & 7);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rl = (lane >> 3) + 4 * i;
              const float4 val = *reinterpret_cast<const float4*>(eb + rl * kEpiStride + 4 * (lane & 7));
              if (col < p.N) *reinterpret_cast<float4*>(c_dst_row0 + static_cast<size_t>(rl) * p.ldc + col) = val;
            }
            __syncwarp();
          }
          continue;
        }
        if constexpr (MODE == kPlain) {
          if (splits > 1) {
            // partial sum of this K split: raw fp32 to the workspace slab (N is a multiple of 4 on this path)
            if (row < p.M && col0 < p.N) {
              float* wp = p.ws + (static_cast<size_t>(t % splits) * p.M + row) * p.N + col0;
#pragma unroll
              for (int q = 0; q < 8; ++q)
                if (col0 + 4 * q < p.N)
                  reinterpret_cast<float4*>(wp)[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                                 __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
            }
            continue;
          }
        }
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
      if constexpr (MODE == kScatter) __threadfence_system();  // this lane's stores before the arrival below
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_leader(&tempty_bar[buf]);
        if constexpr (MODE == kScatter) {
          if (c_live) {  // one arrival per rank and (32-row group, column tile) of the owner's rows
            const int grp = (row0w - c_dest * p.c_rows_per_rank) >> 5;
            red_release_sys_add(p.c_cnt[c_dest] + grp * p.tiles_n + nb, 1);
          }
        }
      }
      if (++buf == 2) { buf = 0; tphase ^= 1; }
    }
  } else if constexpr (MODE == kCopyJob) {
    // ------------------------------------------------------------ copy-job warp (warp 6 of every CTA)
    // CTA b moves units cj_u0 + b, cj_u0 + b + grid, ...: source (a peer's or this GPU's memory) -> shared memory -> cj_dst,
    // both legs as bulk copies without any cluster qualifier, one load in flight while the previous unit is stored.  The
    // consumer of the copied data is a later kernel on the same stream, so completion of the stores before this kernel ends
    // is the only ordering needed.
    if (lane == 0 && p.cj_u1 > p.cj_u0) {
      auto issue = [&](int u, int b) {
        const int4 e = __ldg(p.cj_table + u);
        const uint32_t bytes = static_cast<uint32_t>(e.w) << 4;
        mbar_expect_tx(&copy_bar[b], bytes);
        bulk_load(copy_buf + b * kCopyUnit, p.cj_src[e.x] + (static_cast<size_t>(static_cast<uint32_t>(e.y)) << 4), bytes, &copy_bar[b]);
      };
      int u = p.cj_u0 + static_cast<int>(blockIdx.x);
      uint32_t ph0 = 0, ph1 = 0;
      int j = 0;
      bool ok = true, pending_load = false;
      if (u < p.cj_u1) issue(u, 0);
      while (u < p.cj_u1) {
        const int un = u + static_cast<int>(gridDim.x);
        const int b = j & 1;
        pending_load = false;
        if (un < p.cj_u1) {
          bulk_wait_read<0>();  // the store that last read the other buffer has drained it
          issue(un, b ^ 1);
          pending_load = true;
        }
        ok = mbar_wait(&copy_bar[b], b ? ph1 : ph0, abort_flag, p.status, 410, b);
        if (!ok) break;
        if (b) ph1 ^= 1; else ph0 ^= 1;
        const int4 e = __ldg(p.cj_table + u);
        bulk_store(p.cj_dst + (static_cast<size_t>(static_cast<uint32_t>(e.z)) << 4), copy_buf + b * kCopyUnit, static_cast<uint32_t>(e.w) << 4);
        bulk_commit();
        u = un;
        ++j;
      }
      bulk_wait<0>();
      if (!ok && pending_load) mbar_wait_quiet(&copy_bar[(j & 1) ^ 1], (j & 1) ? ph0 : ph1);  // let the load in flight land
    }
  } else if constexpr (MODE == kScatter) {
    // ------------------------------------------------------------ reduce warps (warps 6-9 of every CTA)
    // This rank's rows, concurrently with the main loop, in units of 32 rows x BN columns in the order the raster produces
    // them: wait until all `world` ranks (this one included) have delivered the unit, then sum the slots.
    const int rtid = threadIdx.x - kNumThreads;
    const int own_units = (p.c_rows_per_rank >> 5) * p.tiles_n;
    const bool out_f32 = p.rs_out_f32 != 0;
    const bool acc_out = p.rs_accumulate != 0;
    constexpr int RU = 32;
    constexpr int kVecPerRow = BN / 4;
    constexpr int kUnroll = 4;  // independent 16-byte loads in flight per thread and slot
    for (int t = blockIdx.x; t < own_units; t += gridDim.x) {
      if (rtid == 0 && !*abort_flag) flag_wait_ge(p.c_cnt[p.rank] + t, p.c_target, true, abort_flag, p.status, 500, t);
      reduce_bar_sync();
      if (*abort_flag) break;
      const int grp = t / p.tiles_n, nb = t - grp * p.tiles_n;
      for (int i0 = rtid; i0 < RU * kVecPerRow; i0 += kUnroll * kReduceThreads) {
        float4 acc[kUnroll];
        size_t off[kUnroll];
        bool live[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int i = i0 + u * kReduceThreads;
          const int r = i / kVecPerRow;
          const int col = nb * BN + (i - r * kVecPerRow) * 4;
          live[u] = (i < RU * kVecPerRow) && (col < p.N);
          off[u] = (static_cast<size_t>(grp) * RU + r) * p.ldc + col;
          acc[u] = live[u] ? __ldcg(reinterpret_cast<const float4*>(p.rs_staging + off[u])) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int w = 1; w < p.world; ++w) {
          float4 v[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u)
            v[u] = live[u] ? __ldcg(reinterpret_cast<const float4*>(p.rs_staging + w * p.rs_slot + off[u])) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) { acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w; }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (!live[u]) continue;
          const int i = i0 + u * kReduceThreads;
          const int r = i / kVecPerRow;
          const int col = nb * BN + (i - r * kVecPerRow) * 4;
          const size_t row = static_cast<size_t>(grp) * RU + r;
          if (out_f32) {
            float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.rs_out) + row * p.rs_ldo + col);
            if (acc_out) {
              const float4 a = *o;
              *o = make_float4(a.x + acc[u].x, a.y + acc[u].y, a.z + acc[u].z, a.w + acc[u].w);
            } else {
              *o = acc[u];
            }
          } else {
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.rs_out) + row * p.rs_ldo + col) =
                make_uint2(pack_bf16x2(acc[u].x, acc[u].y), pack_bf16x2(acc[u].z, acc[u].w));
          }
        }
      }
      reduce_bar_sync();  // nobody is still reading the abort flag when thread 0 starts the next wait
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
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_pair_body<BN, A_MN, B_MN, kPlain>(tmA, tmB, p);
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kScatterThreads, 1)
gemm_pair_scatter_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_pair_body<BN, A_MN, B_MN, kScatter>(tmA, tmB, p);
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kCopyThreads, 1)
gemm_pair_copy_job_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_pair_body<BN, A_MN, B_MN, kCopyJob>(tmA, tmB, p);
}

template <typename Kern>
int max_resident_pairs(Kern kern, int threads, int smem) {
  // as many pairs as can be resident at once (a GPC with an odd number of free SMs cannot host a pair on the last one)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (num_sms() / 2));
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
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
  return n;
}

template <int BN, bool A_MN, bool B_MN>
int make_maps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, const void* B, const Params& p, int lda, int ldb) {
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(tmA, A, p.M, p.K, lda, BMC, BK);  // [M,K] rows=M
  else       rc = make_tmap_2d_bf16(tmA, A, p.K, p.M, lda, BK, 64);   // [K,M] rows=K, box 64 k x 64 m
  if (rc != kErrOk) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(tmB, B, p.N, p.K, ldb, BN / 2, BK);
  else       rc = make_tmap_2d_bf16(tmB, B, p.K, p.N, ldb, BK, 64);
  return rc;
}

template <int BN, bool A_MN, bool B_MN>
int launch_scatter(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream) {
  using L = Smem<BN>;
  constexpr int kSmem = L::kTotal + kEpiExtra;
  static_assert(kSmem <= 232448, "scatter kernel exceeds the shared memory of an SM");
  CUtensorMap tmA, tmB;
  int rc = make_maps<BN, A_MN, B_MN>(&tmA, &tmB, A, B, p, lda, ldb);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BMP - 1) / BMP;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_pair_scatter_kernel<BN, A_MN, B_MN>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return kErrCuda;
    max_pairs = max_resident_pairs(kern, kScatterThreads, kSmem);
  }
  int pairs = p.tiles_m * p.tiles_n;
  if (pairs > max_pairs) pairs = max_pairs;
  kern<<<2 * pairs, kScatterThreads, kSmem, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

template <int BN, bool A_MN, bool B_MN>
int launch_copy_job(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream) {
  using L = Smem<BN>;
  constexpr int kSmem = L::kTotal + kCopyExtra;
  static_assert(kSmem <= 232448, "copy-job kernel exceeds the shared memory of an SM");
  CUtensorMap tmA, tmB;
  int rc = make_maps<BN, A_MN, B_MN>(&tmA, &tmB, A, B, p, lda, ldb);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BMP - 1) / BMP;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_pair_copy_job_kernel<BN, A_MN, B_MN>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return kErrCuda;
    max_pairs = max_resident_pairs(kern, kCopyThreads, kSmem);
  }
  // every resident pair even when there are fewer tiles: every CTA's copy warp moves a share of the units
  kern<<<2 * max_pairs, kCopyThreads, kSmem, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

template <int BN, bool A_MN, bool B_MN>
int launch(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream, int max_ctas) {
  using L = Smem<BN>;
  CUtensorMap tmA, tmB;
  int rc = make_maps<BN, A_MN, B_MN>(&tmA, &tmB, A, B, p, lda, ldb);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BMP - 1) / BMP;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_pair_kernel<BN, A_MN, B_MN>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return kErrCuda;
    max_pairs = max_resident_pairs(kern, kNumThreads, L::kTotal);
  }
  int cap = max_pairs;
  if (max_ctas > 0 && max_ctas / 2 < cap) cap = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  const int tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;
  if (p.splits < 0) {
    // as many (tile, split) pairs as SM pairs, at least 8 k-blocks each
    int sp = cap / tiles;
    if (sp > k_blocks / 8) sp = k_blocks / 8;
    if (sp > 8) sp = 8;
    p.splits = sp < 1 ? 1 : sp;
  }
  if (p.ws == nullptr || (p.N & 3) || (p.flags & kAccumulate)) p.splits = 1;
  if (p.splits > k_blocks) p.splits = k_blocks;
  p.kb_per_split = (k_blocks + p.splits - 1) / p.splits;
  p.splits = (k_blocks + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  int pairs = tiles * p.splits;
  if (pairs > cap) pairs = cap;
  kern<<<2 * pairs, kNumThreads, L::kTotal, stream>>>(tmA, tmB, p);
  if (cudaGetLastError() != cudaSuccess) return kErrCuda;
  if (p.splits > 1)
    return launch_splitk_finalize(p.ws, p.splits, p.M, p.N, p.alpha, p.flags, p.bias, p.residual, p.ldr, p.C, p.ldc, stream);
  return kErrOk;
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

// lvb_gemm_bf16_pair for K-major operands with K split over `splits` CTA pairs per tile (0: chosen by the launcher so that about
// every SM pair gets a piece; at most 8).  `workspace`: lvb_gemm_skinny_workspace_bytes(M, N) bytes of device memory, contents
// irrelevant.  N % 4 == 0 and no accumulate flag, else one split is used.  The partial tiles are summed in a fixed order.
extern "C" int lvb_gemm_bf16_pair_splitk(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int flags,
                                         float alpha, const void* bias, const void* residual, int ldr, int splits, void* workspace,
                                         int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm2;
  if (M <= 0 || N <= 128 || K <= 0 || (lda & 7) || (ldb & 7) || splits < 0 || splits > 8) return kErrBadArg;
  Params p;
  p.C = C; p.bias = bias; p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr;
  p.flags = flags; p.alpha = alpha; p.status = status;
  p.splits = splits == 0 ? -1 : splits;
  p.ws = reinterpret_cast<float*>(workspace);
  return launch<256, false, false>(A, B, p, lda, ldb, reinterpret_cast<cudaStream_t>(stream), 0);
}

// The CTA-pair form of lvb_gemm_reduce_scatter (gemm_bf16.cu) with fp32 staging: same protocol and arguments, except that
// m_order lists 256-row blocks (int32[ceil(M / 256)]) and N must exceed 128.
extern "C" int lvb_gemm_reduce_scatter_pair(const void* A, const void* B, int a_mn, int b_mn, void* const* c_slots, int* const* cnt_peers,
                                            int rank, int world, const void* staging, long long slot_elems, int target,
                                            const int* m_order, void* out, int ldo, int out_f32, int accumulate, int M, int N, int K,
                                            int lda, int ldb, int ldc, float alpha, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm2;
  if (world <= 0 || world > kMaxPeers || rank < 0 || rank >= world || M <= 0 || N <= 128 || K <= 0) return kErrBadArg;
  if (M % world != 0 || (M / world) % 32 != 0 || (N & 7) || (ldc & 7) || (ldo & 7) || (lda & 7) || (ldb & 7)) return kErrBadArg;
  if (m_order == nullptr || (accumulate && !out_f32) || (a_mn != b_mn)) return kErrBadArg;
  Params p;
  p.C = c_slots[rank]; p.bias = nullptr; p.residual = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = 0;
  p.flags = kOutF32; p.alpha = alpha; p.status = status;
  p.rank = rank; p.world = world;
  p.c_rows_per_rank = M / world;
  for (int r = 0; r < kMaxPeers; ++r) {
    p.c_peer[r] = c_slots[r < world ? r : 0];
    p.c_cnt[r] = cnt_peers[r < world ? r : 0];
  }
  p.rs_staging = reinterpret_cast<const float*>(staging); p.rs_slot = slot_elems; p.rs_out = out; p.rs_ldo = ldo; p.rs_out_f32 = out_f32;
  p.c_target = target; p.c_m_order = m_order; p.rs_accumulate = accumulate;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn) return launch_scatter<256, true, true>(A, B, p, lda, ldb, s);
  return launch_scatter<256, false, false>(A, B, p, lda, ldb, s);
}

// The CTA-pair form of lvb_gemm_bf16_copy_job (gemm_bf16.cu): the same arguments; N must exceed 128.
extern "C" int lvb_gemm_bf16_pair_copy_job(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                           int a_mn, int b_mn, int flags, float alpha, const void* bias, const void* residual, int ldr,
                                           const void* table, int u0, int u1, const void* const* srcs, int n_srcs, void* dst,
                                           int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm2;
  if (M <= 0 || N <= 128 || K <= 0 || (lda & 7) || (ldb & 7)) return kErrBadArg;
  if (table == nullptr || dst == nullptr || n_srcs <= 0 || n_srcs > kMaxPeers || u1 < u0) return kErrBadArg;
  Params p;
  p.C = C; p.bias = bias; p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr;
  p.flags = flags; p.alpha = alpha; p.status = status;
  p.rank = 0; p.world = 1; p.c_rows_per_rank = 0;
  p.cj_table = reinterpret_cast<const int4*>(table); p.cj_u0 = u0; p.cj_u1 = u1;
  for (int r = 0; r < kMaxPeers; ++r) p.cj_src[r] = reinterpret_cast<const uint8_t*>(srcs[r < n_srcs ? r : 0]);
  p.cj_dst = reinterpret_cast<uint8_t*>(dst);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch_copy_job<256, false, false>(A, B, p, lda, ldb, s);
  if (!a_mn && b_mn) return launch_copy_job<256, false, true>(A, B, p, lda, ldb, s);
  if (a_mn && b_mn) return launch_copy_job<256, true, true>(A, B, p, lda, ldb, s);
  return launch_copy_job<256, true, false>(A, B, p, lda, ldb, s);
}
