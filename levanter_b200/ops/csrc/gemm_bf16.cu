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
  // ---- fused collectives (see the kernels at the end of this file); unused by the plain GEMM
  int rank, world;
  int m_rot;              // the tile raster starts at this m-block and wraps, so every rank begins with the rows nearest to hand
  int a_rows_per_map;     // gathered A: rows [r * a_rows_per_map, ...) are fetched through tensor map r
  const uint8_t* a_peer[kMaxPeers];  // gathered A: rank r's shard (a pointer into rank r's memory, valid on this GPU)
  uint8_t* a_local;       // gathered A: local [M, K] copy that the remote shards are pulled into
  int* a_cnt;             // gathered A: arrival counter per (rank, 128-row block) of a_local, zeroed before the launch
  int a_units_per_block;  // gathered A: copy units (kCopyUnit bytes) per 128-row block
  int c_rows_per_rank;    // scattered C: rows [r * c_rows_per_rank, ...) are stored to c_peer[r]
  void* c_peer[kMaxPeers];   // scattered C: this rank's slot in rank r's staging buffer
  int* c_cnt[kMaxPeers];     // scattered C: rank r's per-tile arrival counters (in rank r's memory); they only ever grow
  int c_target;              // scattered C: value of a counter once all `world` parts of this call's unit have arrived
  const int* c_m_order;      // scattered C: the raster's i-th row block is block c_m_order[i] (owners dealt round-robin)
  int rs_accumulate;         // scattered C: the reduced rows are added to rs_out (fp32) instead of stored
  const float* rs_staging;   // scattered C: this rank's own staging buffer [world, slot]
  long long rs_slot;         // elements per slot
  void* rs_out;              // this rank's reduced rows [c_rows_per_rank, N] (bf16, or fp32 if rs_out_f32), row stride rs_ldo
  int rs_ldo;
  int rs_out_f32;
  // ---- copy job (kModeCopyJob): units [cj_u0, cj_u1) of a table of {source rank, source offset / 16, destination offset / 16,
  // bytes / 16}; a seventh warp of every CTA moves them (peer or local memory -> shared memory -> cj_dst) beside the GEMM
  const int4* cj_table;
  int cj_u0, cj_u1;
  const uint8_t* cj_src[kMaxPeers];
  uint8_t* cj_dst;
  // ---- grouped GEMM (see lvb_gemm_grouped)
  const int* g_tile_group;  // K-major A: group of every 128-row block of A, or -1 for a block past the last group (skipped)
  int g_b_rows;             // K-major A: rows (K-major B) or reduction rows (MN-major B) of one group's B inside the stacked B
  const int* g_offsets;     // MN-major A (weight gradient): reduction rows [g_offsets[g], g_offsets[g + 1]) belong to group g
  int g_tiles_m;            // MN-major A: 128-row blocks of C per group
};

constexpr int kModePlain = 0;
constexpr int kModeGatherA = 1;   // all-gather fused into the A operand
constexpr int kModeScatterC = 2;  // reduce-scatter fused into the epilogue
constexpr int kModeGrouped = 3;   // one B matrix (or one K range) per group of rows: the expert GEMMs of a mixture-of-experts layer
constexpr int kModeCopyJob = 4;   // plain GEMM whose CTAs also carry out a list of bulk copies (the next layer's weight gather)
constexpr int kCopyUnit = 16384;  // bytes per bulk copy of the gather
constexpr int kCopyExtra = 256 + 2 * kCopyUnit;  // extra dynamic shared memory of the gather kernel
constexpr int kGatherThreads = kNumThreads + 32;  // + one copy warp
constexpr int kReduceThreads = 128;  // scatter mode: four more warps that sum the staging slots
constexpr int kScatterThreads = kNumThreads + kReduceThreads;
constexpr int kEpiStride = 36;   // floats per staged row (144 B: 16-byte aligned, conflict-free for float4 rows)
constexpr int kEpiExtra = 256 + 4 * 32 * kEpiStride * 4;  // extra dynamic shared memory of the scatter kernel

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

__device__ __forceinline__ void reduce_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kReduceThreads) : "memory"); }

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
__device__ __forceinline__ void tile_coords_rot(int t, int tiles_m, int tiles_n, int m_rot, int& mb, int& nb) {
  tile_coords(t, tiles_m, tiles_n, mb, nb);
  mb += m_rot;
  if (mb >= tiles_m) mb -= tiles_m;
}
// Scatter raster: the host passes a permutation of the row blocks that deals them out to their owners in turn (next rank
// first, own rank last of each round), so the peer stores are spread evenly over the kernel's duration and every rank's rows
// complete at a steady rate.
__device__ __forceinline__ void tile_coords_ordered(int t, int tiles_m, int tiles_n, const int* __restrict__ m_order, int& mb, int& nb) {
  tile_coords(t, tiles_m, tiles_n, mb, nb);
  mb = __ldg(m_order + mb);
}

// Grouped mode: what a tile has to do.  K-major A (forward, input gradient): the tile's row block belongs to group g (skip when
// g < 0) and the whole K is reduced.  MN-major A (weight gradient): row block mb of C belongs to group mb / g_tiles_m and only
// that group's rows of the two operands are reduced (k-blocks [kb0, kb1); nothing to do when the group is empty).
template <bool A_MN>
__device__ __forceinline__ bool grouped_tile(const Params& p, int mb, int k_blocks, int& group, int& kb0, int& kb1) {
  if constexpr (!A_MN) {
    group = p.g_tile_group[mb];
    kb0 = 0;
    kb1 = k_blocks;
    return group >= 0;
  } else {
    group = mb / p.g_tiles_m;
    kb0 = p.g_offsets[group] / BK;
    kb1 = p.g_offsets[group + 1] / BK;
    return kb1 > kb0;
  }
}

// kF8: one-byte operands (both K-major); a stage row is still 128 bytes, i.e. 128 elements of K instead of 64.
template <int BN, bool A_MN, bool B_MN, bool kF8 = false, int MODE = kModePlain>
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
  // gather mode only: two copy barriers and two staging buffers behind the GEMM's own shared memory
  uint64_t* copy_bar = reinterpret_cast<uint64_t*>(smem + ((L::kTileBytes + L::kBarBytes + 127) & ~127));
  uint8_t* copy_buf = reinterpret_cast<uint8_t*>(copy_bar) + 128;
  // scatter mode only: a 32 x 32 fp32 transposition buffer per epilogue warp in the same place
  float* epi_buf = reinterpret_cast<float*>(copy_bar);

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
    if constexpr (MODE == kModeGatherA || MODE == kModeCopyJob) {
      mbar_init(&copy_bar[0], 1);
      mbar_init(&copy_bar[1], 1);
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
      int ready_block = -1;  // gather mode: last m-block whose rows are known to have arrived
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb;
        if constexpr (MODE == kModePlain || MODE == kModeGrouped || MODE == kModeCopyJob) tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
        else if constexpr (MODE == kModeScatterC) tile_coords_ordered(t, p.tiles_m, p.tiles_n, p.c_m_order, mb, nb);
        else tile_coords_rot(t, p.tiles_m, p.tiles_n, p.m_rot, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        int a_map = 0, a_row = m0;
        int group = 0, kb_begin = 0, kb_end = k_blocks;
        if constexpr (MODE == kModeGrouped) {
          if (!grouped_tile<A_MN>(p, mb, k_blocks, group, kb_begin, kb_end)) continue;
        }
        if constexpr (MODE == kModeGatherA) {
          a_map = m0 / p.a_rows_per_map;  // the rank these rows belong to
          a_row = m0 - a_map * p.a_rows_per_map;
          if (a_map != p.rank && mb != ready_block) {
            // rows of another rank: wait until the copy warps (of all CTAs) have pulled this 128-row block into a_local
            const int blocks_per_rank = p.a_rows_per_map / BM;
            ok = flag_wait_ge(p.a_cnt + a_map * blocks_per_rank + a_row / BM, p.a_units_per_block, false, abort_flag, p.status, 110, mb);
            if (!ok) break;
            fence_proxy_async_all();  // the block was written by bulk stores of other CTAs; the loads below are TMA
            ready_block = mb;
          }
        }
        // grouped mode: where this tile's operands sit inside the stacked tensors
        int a_col = m0, b_row = n0, b_k = 0;
        if constexpr (MODE == kModeGrouped) {
          if constexpr (A_MN) a_col = (mb - group * p.g_tiles_m) * BM;      // C rows are stacked per group, A's columns are not
          else if constexpr (!B_MN) b_row = group * p.g_b_rows + n0;        // K-major B: [groups * N, K]
          else b_k = group * p.g_b_rows;                                    // MN-major B: [groups * K, N]
        }
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 100, stage);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          const int k0 = kb * BKE;
          if constexpr (!A_MN) {
            tma_load_2d(sa, tmA_maps + a_map, &full_bar[stage], k0, a_row);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (64 * BK * 2), &tmA, &full_bar[stage], a_col + 64 * c, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, b_row);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &tmB, &full_bar[stage], n0 + 64 * c, k0 + b_k);
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
        int n_kb = k_blocks;
        if constexpr (MODE == kModeGrouped) {
          int mb, nb, group, kb0, kb1;
          tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
          if (!grouped_tile<A_MN>(p, mb, k_blocks, group, kb0, kb1)) continue;
          n_kb = kb1 - kb0;
        }
        ok = mbar_wait(&tempty_bar[buf], tphase ^ 1, abort_flag, p.status, 200, buf);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kb = 0; kb < n_kb; ++kb) {
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
  } else if (warp < 6) {
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
      if constexpr (MODE == kModePlain || MODE == kModeGrouped || MODE == kModeCopyJob) tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      else if constexpr (MODE == kModeScatterC) tile_coords_ordered(t, p.tiles_m, p.tiles_n, p.c_m_order, mb, nb);
      else tile_coords_rot(t, p.tiles_m, p.tiles_n, p.m_rot, mb, nb);
      if constexpr (MODE == kModeGrouped) {
        int group, kb0, kb1;
        if (!grouped_tile<A_MN>(p, mb, k_blocks, group, kb0, kb1)) continue;
      }
      ok = mbar_wait(&tfull_bar[buf], tphase, abort_flag, p.status, 300, buf);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = mb * BM + quad * 32 + lane;
      const int n0 = nb * BN;
      void* c_base = p.C;
      size_t c_row = static_cast<size_t>(row);
      int c_dest = 0;
      bool c_live = true;
      if constexpr (MODE == kModeScatterC) {
        // this warp's 32 rows belong to one rank (c_rows_per_rank and M are multiples of 32): they go to that rank's staging slot
        const int row0w = mb * BM + quad * 32;
        c_live = row0w < p.M;
        c_dest = c_live ? row0w / p.c_rows_per_rank : 0;
        c_base = p.c_peer[c_dest];
        c_row = static_cast<size_t>(row - c_dest * p.c_rows_per_rank);
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        const int col0 = n0 + c;
        if constexpr (MODE == kModeScatterC) {
          // Peer stores: turn the row-per-lane fragment into row-contiguous 128-byte segments through shared memory, so a
          // store instruction covers 4 rows x 128 B instead of 32 rows x 16 B (NVLink moves short writes poorly).
          if (col0 < p.N && c_live) {  // warp-uniform; all 32 rows of a live warp are valid
            float* eb = epi_buf + (warp - 2) * (32 * kEpiStride);
            if (out_f32) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(eb + lane * kEpiStride + 4 * q) =
                    make_float4(__uint_as_float(r[4 * q]) * alpha, __uint_as_float(r[4 * q + 1]) * alpha,
                                __uint_as_float(r[4 * q + 2]) * alpha, __uint_as_float(r[4 * q + 3]) * alpha);
              __syncwarp();
              const int col = col0 + 4 * (lane & 7);
              float* dst = reinterpret_cast<float*>(c_base) + (c_row - lane) * p.ldc + col;  // row 0 of this warp's 32 rows
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rl = (lane >> 3) + 4 * i;
                const float4 val = *reinterpret_cast<const float4*>(eb + rl * kEpiStride + 4 * (lane & 7));
                if (col < p.N) *reinterpret_cast<float4*>(dst + static_cast<size_t>(rl) * p.ldc) = val;
              }
              __syncwarp();
            } else {
              // bf16 staging: two 32-column fragments make one 128-byte row segment (the loop below advances c by 64)
              uint32_t r2[32];
              tmem_ld_32x32(taddr + c + 32, r2);
              tmem_ld_wait();
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(r[8 * q + 0]) * alpha, __uint_as_float(r[8 * q + 1]) * alpha);
                o.y = pack_bf16x2(__uint_as_float(r[8 * q + 2]) * alpha, __uint_as_float(r[8 * q + 3]) * alpha);
                o.z = pack_bf16x2(__uint_as_float(r[8 * q + 4]) * alpha, __uint_as_float(r[8 * q + 5]) * alpha);
                o.w = pack_bf16x2(__uint_as_float(r[8 * q + 6]) * alpha, __uint_as_float(r[8 * q + 7]) * alpha);
                *reinterpret_cast<uint4*>(eb + lane * kEpiStride + 4 * q) = o;
                o.x = pack_bf16x2(__uint_as_float(r2[8 * q + 0]) * alpha, __uint_as_float(r2[8 * q + 1]) * alpha);
                o.y = pack_bf16x2(__uint_as_float(r2[8 * q + 2]) * alpha, __uint_as_float(r2[8 * q + 3]) * alpha);
                o.z = pack_bf16x2(__uint_as_float(r2[8 * q + 4]) * alpha, __uint_as_float(r2[8 * q + 5]) * alpha);
                o.w = pack_bf16x2(__uint_as_float(r2[8 * q + 6]) * alpha, __uint_as_float(r2[8 * q + 7]) * alpha);
                *reinterpret_cast<uint4*>(eb + lane * kEpiStride + 16 + 4 * q) = o;
              }
              __syncwarp();
              const int col = col0 + 8 * (lane & 7);
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c_base) + (c_row - lane) * p.ldc + col;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rl = (lane >> 3) + 4 * i;
                const uint4 val = *reinterpret_cast<const uint4*>(eb + rl * kEpiStride + 4 * (lane & 7));
                if (col < p.N) *reinterpret_cast<uint4*>(dst + static_cast<size_t>(rl) * p.ldc) = val;
              }
              __syncwarp();
              c += 32;
            }
          }
          continue;
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
            float* cp = reinterpret_cast<float*>(c_base) + c_row * p.ldc + col0;
            if (full && (p.ldc & 3) == 0) {
              if (accum) {
                // C += tile as vector reductions resolved in L2: the epilogue does not wait for the old values to come back,
                // and every element has exactly one adder per launch, so the sum stays deterministic
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
      if constexpr (MODE == kModeScatterC) __threadfence_system();  // this lane's stores before the arrival below
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty_bar[buf]);
        if constexpr (MODE == kModeScatterC) {
          // one arrival per rank and (32-row group, column tile) of the owner's rows
          if (c_live) {
            const int grp = (mb * BM + quad * 32 - c_dest * p.c_rows_per_rank) >> 5;
            red_release_sys_add(p.c_cnt[c_dest] + grp * p.tiles_n + nb, 1);
          }
        }
      }
      if (++buf == 2) { buf = 0; tphase ^= 1; }
    }
  } else if constexpr (MODE == kModeGatherA) {
    // ------------------------------------------------------------ gather copy warp (warp 6)
    // The remote shards are cut into kCopyUnit-byte units, numbered in the order the tile raster needs them (nearest rank
    // first); CTA b moves units b, b + grid, ...: peer memory -> shared memory -> a_local, both legs as bulk copies, one
    // load in flight while the previous unit is stored.  Each finished unit bumps its 128-row block's arrival counter.
    if (lane == 0 && p.world > 1) {
      const long long blocks_per_rank = p.a_rows_per_map / BM;
      const long long per_rank = blocks_per_rank * p.a_units_per_block;
      const long long total = per_rank * (p.world - 1);
      const long long shard_bytes = static_cast<long long>(p.a_rows_per_map) * p.K * 2;
      auto src_rank = [&](long long g) { int r = p.rank + 1 + static_cast<int>(g / per_rank); return r >= p.world ? r - p.world : r; };
      auto issue = [&](long long g, int b) {
        const int r = src_rank(g);
        const long long off = (g % per_rank) * kCopyUnit;
        mbar_expect_tx(&copy_bar[b], kCopyUnit);
        bulk_load(copy_buf + b * kCopyUnit, p.a_peer[r] + off, kCopyUnit, &copy_bar[b]);
      };
      auto signal = [&](long long g) {
        const int r = src_rank(g);
        const long long blk = (g % per_rank) / p.a_units_per_block;
        fence_proxy_async_all();  // bulk-store writes (async proxy) before the generic-proxy release below
        __threadfence();
        red_release_gpu_add(p.a_cnt + r * blocks_per_rank + blk, 1);
      };
      long long g = blockIdx.x, prev = -1;
      uint32_t ph0 = 0, ph1 = 0;
      int j = 0;
      bool ok = true, pending_load = false;
      if (g < total) issue(g, 0);
      while (g < total) {
        const long long gn = g + gridDim.x;
        const int b = j & 1;
        pending_load = false;
        if (gn < total) {
          bulk_wait_read<0>();  // the store that last read the other buffer has drained it
          issue(gn, b ^ 1);
          pending_load = true;
        }
        ok = mbar_wait(&copy_bar[b], b ? ph1 : ph0, abort_flag, p.status, 400, b);
        if (!ok) break;
        if (b) ph1 ^= 1; else ph0 ^= 1;
        const int r = src_rank(g);
        bulk_store(p.a_local + r * shard_bytes + (g % per_rank) * kCopyUnit, copy_buf + b * kCopyUnit, kCopyUnit);
        bulk_commit();
        if (prev >= 0) {
          bulk_wait<1>();  // the previous unit's store is complete
          signal(prev);
        }
        prev = g;
        g = gn;
        ++j;
      }
      bulk_wait<0>();
      if (ok && prev >= 0) signal(prev);
      if (!ok && pending_load) mbar_wait_quiet(&copy_bar[(j & 1) ^ 1], (j & 1) ? ph0 : ph1);  // let the load in flight land
    }
  } else if constexpr (MODE == kModeCopyJob) {
    // ------------------------------------------------------------ copy-job warp (warp 6)
    // CTA b moves units cj_u0 + b, cj_u0 + b + grid, ... of the table: source (a peer's or this GPU's memory) -> shared
    // memory -> cj_dst, both legs as bulk copies, one load in flight while the previous unit is stored.  Nothing in this
    // kernel reads what is copied: the consumer is a later kernel on the same stream, so completion of the stores before
    // the kernel ends (bulk_wait<0>) is the only ordering needed.
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
  } else if constexpr (MODE == kModeScatterC) {
    // ------------------------------------------------------------ reduce warps (warps 6-9)
    // This rank's rows, concurrently with the main loop, in units of 32 rows x BN columns in the order the raster produces
    // them: wait until all `world` ranks (this one included) have delivered the unit into their staging slots, then sum the
    // slots.  Every rank produces the rows of a given rank at the same steady rate, so these warps trail the tensor cores
    // closely and little is left to reduce when the last tile has been multiplied.
    const int rtid = threadIdx.x - kNumThreads;
    const int own_units = (p.c_rows_per_rank >> 5) * p.tiles_n;
    const bool out_f32 = p.rs_out_f32 != 0;
    const bool acc_out = p.rs_accumulate != 0;
    constexpr int RU = 32;  // rows per unit
    for (int t = blockIdx.x; t < own_units; t += gridDim.x) {
      if (rtid == 0 && !*abort_flag)
        flag_wait_ge(p.c_cnt[p.rank] + t, p.c_target, true, abort_flag, p.status, 500, t);
      reduce_bar_sync();
      if (*abort_flag) break;
      const int grp = t / p.tiles_n, nb = t - grp * p.tiles_n;
      if (!(p.flags & kOutF32)) {
        // bf16 staging slots: 8 elements per 16-byte load, fp32 accumulation
        constexpr int kVec8PerRow = BN / 8;
        constexpr int kU = 4;
        const __nv_bfloat16* stg = reinterpret_cast<const __nv_bfloat16*>(p.rs_staging);
        for (int i0 = rtid; i0 < RU * kVec8PerRow; i0 += kU * kReduceThreads) {
          float acc[kU][8];
          size_t off[kU];
          bool live[kU];
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const int i = i0 + u * kReduceThreads;
            const int r = i / kVec8PerRow;
            const int col = nb * BN + (i - r * kVec8PerRow) * 8;
            live[u] = (i < RU * kVec8PerRow) && (col < p.N);
            off[u] = (static_cast<size_t>(grp) * RU + r) * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
          }
          for (int w = 0; w < p.world; ++w) {
            uint4 v[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u)
              v[u] = live[u] ? __ldcg(reinterpret_cast<const uint4*>(stg + w * p.rs_slot + off[u])) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[u][2 * j] += f.x;
                acc[u][2 * j + 1] += f.y;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            if (!live[u]) continue;
            const int i = i0 + u * kReduceThreads;
            const int r = i / kVec8PerRow;
            const int col = nb * BN + (i - r * kVec8PerRow) * 8;
            const size_t row = static_cast<size_t>(grp) * RU + r;
            if (out_f32) {
              float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.rs_out) + row * p.rs_ldo + col);
              if (acc_out) {
                const float4 a = o[0], b = o[1];
                o[0] = make_float4(a.x + acc[u][0], a.y + acc[u][1], a.z + acc[u][2], a.w + acc[u][3]);
                o[1] = make_float4(b.x + acc[u][4], b.y + acc[u][5], b.z + acc[u][6], b.w + acc[u][7]);
              } else {
                o[0] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
                o[1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
              }
            } else {
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.rs_out) + row * p.rs_ldo + col) =
                  make_uint4(pack_bf16x2(acc[u][0], acc[u][1]), pack_bf16x2(acc[u][2], acc[u][3]),
                             pack_bf16x2(acc[u][4], acc[u][5]), pack_bf16x2(acc[u][6], acc[u][7]));
            }
          }
        }
        reduce_bar_sync();
        continue;
      }
      constexpr int kVecPerRow = BN / 4;
      constexpr int kUnroll = 4;  // independent 16-byte loads in flight per thread and slot
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

// All-gather fused into the A operand: A's row blocks belong to different ranks; the copy warp pulls the remote ones into
// local memory while the tensor cores work on the rows already here (plain bulk loads, no cluster qualifier).
template <int BN>
__global__ void __launch_bounds__(kGatherThreads, 1)
gemm_gather_a_kernel(const __grid_constant__ PeerMaps tmAs, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_body<BN, false, false, false, kModeGatherA>(tmAs.maps, tmB, p);
}

// Reduce-scatter fused into the epilogue: tiles go to the staging slot of the rank that owns their rows, while four more
// warps of every CTA sum this rank's own rows over the slots as the contributions arrive.
template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kScatterThreads, 1)
gemm_scatter_c_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_body<BN, A_MN, B_MN, false, kModeScatterC>(&tmA, tmB, p);
}

// Plain GEMM plus a copy job: a seventh warp per CTA moves a list of 16 KB units (the next layer's weight shards, pulled
// from the peers) while the tensor cores work; bulk copies without any cluster qualifier.
template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGatherThreads, 1)
gemm_copy_job_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_body<BN, A_MN, B_MN, false, kModeCopyJob>(&tmA, tmB, p);
}

// Grouped GEMM: the same pipeline with a per-tile group look-up (see grouped_tile and lvb_gemm_grouped).
template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  gemm_body<BN, A_MN, B_MN, false, kModeGrouped>(&tmA, tmB, p);
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
  p.rank = 0; p.world = 1; p.m_rot = 0;
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
  p.rank = 0; p.world = 1; p.m_rot = 0;
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
int launch_gather_a(const void* B, Params p, int ldb, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  constexpr int kSmem = L::kTotal + kCopyExtra;
  static_assert(kSmem <= 232448, "gather kernel exceeds the shared memory of an SM");
  PeerMaps maps;
  CUtensorMap tmB;
  const size_t shard_bytes = static_cast<size_t>(p.a_rows_per_map) * p.K * 2;
  for (int r = 0; r < p.world; ++r) {
    // own rows are read in place; the other ranks' rows from the local copy that the copy warps fill
    const void* base = (r == p.rank) ? static_cast<const void*>(p.a_peer[r]) : static_cast<const void*>(p.a_local + r * shard_bytes);
    int rc = make_tmap_2d_bf16(&maps.maps[r], base, p.a_rows_per_map, p.K, p.K, BM, BK);
    if (rc != kErrOk) return rc;
  }
  for (int r = p.world; r < kMaxPeers; ++r) maps.maps[r] = maps.maps[0];
  int rc = make_tmap_2d_bf16(&tmB, B, p.N, p.K, ldb, BN, BK);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_gather_a_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  const int blocks = p.world * (p.a_rows_per_map / BM);
  if (cudaMemsetAsync(p.a_cnt, 0, sizeof(int) * blocks, stream) != cudaSuccess) return kErrCuda;
  // one CTA per SM even when there are fewer tiles: every CTA's copy warp moves a share of the remote rows
  kern<<<num_sms(), kGatherThreads, kSmem, stream>>>(maps, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

template <int BN, bool A_MN, bool B_MN>
int launch_scatter_c(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  constexpr int kSmem = L::kTotal + kEpiExtra;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(&tmA, A, p.M, p.K, lda, BM, BK);
  else       rc = make_tmap_2d_bf16(&tmA, A, p.K, p.M, lda, BK, 64);
  if (rc != kErrOk) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tmB, B, p.N, p.K, ldb, BN, BK);
  else       rc = make_tmap_2d_bf16(&tmB, B, p.K, p.N, ldb, BK, 64);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_scatter_c_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  int grid = p.tiles_m * p.tiles_n;
  if (grid > num_sms()) grid = num_sms();
  kern<<<grid, kScatterThreads, kSmem, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

template <int BN, bool A_MN, bool B_MN>
int launch_copy_job(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  constexpr int kSmem = L::kTotal + kCopyExtra;
  static_assert(kSmem <= 232448, "copy-job kernel exceeds the shared memory of an SM");
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(&tmA, A, p.M, p.K, lda, BM, BK);
  else       rc = make_tmap_2d_bf16(&tmA, A, p.K, p.M, lda, BK, 64);
  if (rc != kErrOk) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tmB, B, p.N, p.K, ldb, BN, BK);
  else       rc = make_tmap_2d_bf16(&tmB, B, p.K, p.N, ldb, BK, 64);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_copy_job_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  // one CTA per SM even when there are fewer tiles: every CTA's copy warp moves a share of the units
  kern<<<num_sms(), kGatherThreads, kSmem, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// Stand-alone form of the copy job (no GEMM to ride on: the first layer of a step): two copy warps per CTA.
constexpr int kGatherWarps = 4;
constexpr int kGatherSmem = kGatherWarps * 2 * kCopyUnit + 128;
__global__ void __launch_bounds__(kGatherWarps * 32, 1)
copy_job_kernel(const int4* __restrict__ table, int u0, int u1, Params p) {
  extern __shared__ uint8_t gather_smem_raw[];
  uint8_t* gs = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gather_smem_raw) + 127) & ~uintptr_t(127));
  auto bufs = reinterpret_cast<uint8_t(*)[2][kCopyUnit]>(gs);
  __shared__ __align__(8) uint64_t bars[kGatherWarps][2];
  __shared__ int abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int w = 0; w < kGatherWarps; ++w) {
      mbar_init(&bars[w][0], 1);
      mbar_init(&bars[w][1], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* abort_flag = &abort_word;
  if (lane != 0) return;
  const int stride = static_cast<int>(gridDim.x) * kGatherWarps;
  auto issue = [&](int u, int b) {
    const int4 e = __ldg(table + u);
    const uint32_t bytes = static_cast<uint32_t>(e.w) << 4;
    mbar_expect_tx(&bars[warp][b], bytes);
    bulk_load(bufs[warp][b], p.cj_src[e.x] + (static_cast<size_t>(static_cast<uint32_t>(e.y)) << 4), bytes, &bars[warp][b]);
  };
  int u = u0 + static_cast<int>(blockIdx.x) * kGatherWarps + warp;
  uint32_t ph0 = 0, ph1 = 0;
  int j = 0;
  bool ok = true, pending_load = false;
  if (u < u1) issue(u, 0);
  while (u < u1) {
    const int un = u + stride;
    const int b = j & 1;
    pending_load = false;
    if (un < u1) {
      bulk_wait_read<0>();
      issue(un, b ^ 1);
      pending_load = true;
    }
    ok = mbar_wait(&bars[warp][b], b ? ph1 : ph0, abort_flag, p.status, 420, b);
    if (!ok) break;
    if (b) ph1 ^= 1; else ph0 ^= 1;
    const int4 e = __ldg(table + u);
    bulk_store(p.cj_dst + (static_cast<size_t>(static_cast<uint32_t>(e.z)) << 4), bufs[warp][b], static_cast<uint32_t>(e.w) << 4);
    bulk_commit();
    u = un;
    ++j;
  }
  bulk_wait<0>();
  if (!ok && pending_load) mbar_wait_quiet(&bars[warp][(j & 1) ^ 1], (j & 1) ? ph0 : ph1);
}

}  // namespace gemm
}  // namespace lvb

// Number of int32 arrival counters lvb_gemm_allgather_a needs for an M-row gathered operand.
extern "C" int lvb_gemm_allgather_a_counters(int M) { return (M + lvb::gemm::BM - 1) / lvb::gemm::BM; }

// All-gather fused into a GEMM: C[M, N] = concat_r(A_r)[M, K] B[N, K]^T (+ bias).  A_r [M / world, K] (bf16, contiguous)
// is rank r's shard at a_peers[r], a pointer into rank r's memory that is valid on this GPU (own rank included).  The
// kernel starts with this rank's own rows while its copy warps pull the other shards, nearest rank first, into
// a_local [M, K] (local scratch; the own rows of it are not written), and each later row block is multiplied as soon as
// its arrival counter (a_cnt, lvb_gemm_allgather_a_counters(M) ints of local memory) says it is complete.
// M / world must be a multiple of 128 and K of 64.  The caller orders the ranks: every A_r complete before the launch,
// and no A_r overwritten until every rank's kernel has finished.
extern "C" int lvb_gemm_allgather_a(const void* const* a_peers, int rank, int world, void* a_local, int* a_cnt, const void* B,
                                    void* C, int M, int N, int K, int ldb, int ldc, int flags, float alpha, const void* bias,
                                    int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (world <= 0 || world > kMaxPeers || rank < 0 || rank >= world || M <= 0 || N <= 0 || K <= 0) return kErrBadArg;
  if (M % world != 0 || (M / world) % BM != 0 || K % 64 != 0 || (ldb & 7)) return kErrBadArg;
  if (a_local == nullptr || a_cnt == nullptr) return kErrBadArg;
  Params p;
  p.C = C; p.bias = bias; p.residual = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = 0;
  p.flags = flags & (kOutF32 | kBias | kBiasF32); p.alpha = alpha; p.status = status; p.alpha_dev = nullptr;
  p.a_fmt = p.b_fmt = 0;
  p.rank = rank; p.world = world;
  p.a_rows_per_map = M / world;
  p.m_rot = rank * (p.a_rows_per_map / BM);
  for (int r = 0; r < kMaxPeers; ++r) p.a_peer[r] = reinterpret_cast<const uint8_t*>(a_peers[r < world ? r : 0]);
  p.a_local = reinterpret_cast<uint8_t*>(a_local);
  p.a_cnt = a_cnt;
  p.a_units_per_block = (BM * K * 2) / kCopyUnit;
  p.c_rows_per_rank = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return N > 128 ? launch_gather_a<256>(B, p, ldb, s) : launch_gather_a<128>(B, p, ldb, s);
}

// Reduce-scatter fused into a GEMM: out[M / world, N] (+)= rows [rank * M / world, ...) of sum_s op(A_s) op(B_s)^T, where
// every rank s calls this with its own partial operands (a_mn / b_mn as for lvb_gemm_bf16: the weight-gradient form
// dW = dY^T X is a_mn = b_mn = 1 with the tokens as the reduction index).  Tile by tile the epilogue stores the partial
// product (fp32, or bf16 when staging_f32 is 0: half the NVLink traffic, partial sums rounded as in a bf16 NCCL
// reduce-scatter) into slot `rank` of the staging buffer of the rank that owns the rows (c_slots[r]: a pointer to that slot
// in rank r's memory; staging layout [world, M / world, ldc] elements), 32 rows (one epilogue warp) at a time, and adds 1 to
// that rank's arrival counter of the (32-row group, column tile) unit (cnt_peers[r]: lvb_gemm_rs_counters(M / world, N) ints
// in rank r's memory).  m_order (device, int32[ceil(M / 128)]) is the order in which the row blocks are visited; the
// caller deals them out to their owners in turn.  Four more warps per CTA sum this rank's own units over the slots
// (`staging`: this rank's own buffer) as soon as a unit's counter reaches `target`.  The counters are never reset: the
// caller passes target = world * (number of products, this one included, that have used these counters), and alternates
// between two staging areas with their own counters from call to call, which makes any cross-rank barrier between calls
// unnecessary: a rank can only be one call ahead of its slowest peer, because its own call completes only when every
// peer's parts of that call have arrived.  M / world must be a multiple of 32, N of 8.  With `accumulate` (fp32 out only)
// the reduced rows are added to `out`.
extern "C" int lvb_gemm_reduce_scatter(const void* A, const void* B, int a_mn, int b_mn, void* const* c_slots, int* const* cnt_peers,
                                       int rank, int world, const void* staging, long long slot_elems, int staging_f32, int target,
                                       const int* m_order, void* out, int ldo, int out_f32, int accumulate, int M, int N, int K,
                                       int lda, int ldb, int ldc, float alpha, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (world <= 0 || world > kMaxPeers || rank < 0 || rank >= world || M <= 0 || N <= 0 || K <= 0) return kErrBadArg;
  if (M % world != 0 || (M / world) % 32 != 0 || (N & 7) || (ldc & 7) || (ldo & 7) || (lda & 7) || (ldb & 7)) return kErrBadArg;
  if (m_order == nullptr || (accumulate && !out_f32) || (a_mn != b_mn)) return kErrBadArg;
  Params p;
  p.C = c_slots[rank]; p.bias = nullptr; p.residual = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = 0;
  p.flags = staging_f32 ? kOutF32 : 0; p.alpha = alpha; p.status = status; p.alpha_dev = nullptr;
  p.a_fmt = p.b_fmt = 0;
  p.rank = rank; p.world = world;
  p.a_rows_per_map = 0;
  p.c_rows_per_rank = M / world;
  p.m_rot = 0;
  for (int r = 0; r < kMaxPeers; ++r) {
    p.c_peer[r] = c_slots[r < world ? r : 0];
    p.c_cnt[r] = cnt_peers[r < world ? r : 0];
  }
  p.rs_staging = reinterpret_cast<const float*>(staging); p.rs_slot = slot_elems; p.rs_out = out; p.rs_ldo = ldo; p.rs_out_f32 = out_f32; p.c_target = target;
  p.c_m_order = m_order; p.rs_accumulate = accumulate;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn) return N > 128 ? launch_scatter_c<256, true, true>(A, B, p, lda, ldb, s) : launch_scatter_c<128, true, true>(A, B, p, lda, ldb, s);
  return N > 128 ? launch_scatter_c<256, false, false>(A, B, p, lda, ldb, s) : launch_scatter_c<128, false, false>(A, B, p, lda, ldb, s);
}

// Arrival counters of lvb_gemm_reduce_scatter for an owner's [rows, N] slice.
extern "C" int lvb_gemm_rs_counters(int rows, int N) { return ((rows + 31) / 32) * (N > 128 ? (N + 255) / 256 : 1); }

// lvb_gemm_bf16 whose CTAs also carry out a copy job: units [u0, u1) of `table` (device; int4 {source rank, source byte
// offset / 16, destination byte offset / 16, bytes / 16}, at most 16 KB per unit, offsets and sizes multiples of 16 bytes)
// are moved from srcs[rank] + offset (peer or local memory) to dst + offset by a seventh warp of every CTA while the
// tensor cores multiply.  The GEMM itself does not read what is copied; a later kernel on the same stream may.  N must be
// larger than 128 (the 256-column tile configuration has the shared memory to spare).
extern "C" int lvb_gemm_bf16_copy_job(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                      int a_mn, int b_mn, int flags, float alpha, const void* bias, const void* residual, int ldr,
                                      const void* table, int u0, int u1, const void* const* srcs, int n_srcs, void* dst,
                                      int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (M <= 0 || N <= 128 || K <= 0 || (lda & 7) || (ldb & 7)) return kErrBadArg;
  if (table == nullptr || dst == nullptr || n_srcs <= 0 || n_srcs > kMaxPeers || u1 < u0) return kErrBadArg;
  Params p;
  p.C = C; p.bias = bias; p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr;
  p.flags = flags; p.alpha = alpha; p.status = status; p.alpha_dev = nullptr;
  p.a_fmt = p.b_fmt = 0;
  p.rank = 0; p.world = 1; p.m_rot = 0; p.a_rows_per_map = 0; p.c_rows_per_rank = 0;
  p.cj_table = reinterpret_cast<const int4*>(table); p.cj_u0 = u0; p.cj_u1 = u1;
  for (int r = 0; r < kMaxPeers; ++r) p.cj_src[r] = reinterpret_cast<const uint8_t*>(srcs[r < n_srcs ? r : 0]);
  p.cj_dst = reinterpret_cast<uint8_t*>(dst);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch_copy_job<256, false, false>(A, B, p, lda, ldb, s);
  if (!a_mn && b_mn) return launch_copy_job<256, false, true>(A, B, p, lda, ldb, s);
  if (a_mn && b_mn) return launch_copy_job<256, true, true>(A, B, p, lda, ldb, s);
  return launch_copy_job<256, true, false>(A, B, p, lda, ldb, s);
}

// The copy job on its own (see lvb_gemm_bf16_copy_job): used when no GEMM precedes the consumer, e.g. for the first layer
// of a step.  `ctas` <= 0 means one per SM.
extern "C" int lvb_copy_job(const void* table, int u0, int u1, const void* const* srcs, int n_srcs, void* dst, int ctas, int* status,
                            void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (table == nullptr || dst == nullptr || n_srcs <= 0 || n_srcs > kMaxPeers || u1 < u0) return kErrBadArg;
  if (u1 == u0) return kErrOk;
  Params p;
  p.status = status;
  for (int r = 0; r < kMaxPeers; ++r) p.cj_src[r] = reinterpret_cast<const uint8_t*>(srcs[r < n_srcs ? r : 0]);
  p.cj_dst = reinterpret_cast<uint8_t*>(dst);
  int grid = ctas > 0 ? ctas : num_sms();
  const int need = (u1 - u0 + kGatherWarps - 1) / kGatherWarps;
  if (grid > need) grid = need;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(copy_job_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGatherSmem) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  copy_job_kernel<<<grid, kGatherWarps * 32, kGatherSmem, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const int4*>(table), u0, u1, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// Tiles along N of the kernels above for an N-column output (sizes the per-tile counters).
extern "C" int lvb_gemm_tiles_n(int N) { return N > 128 ? (N + 255) / 256 : 1; }


// ---------------------------------------------------------------------------------------------------------------------
// Grouped GEMMs for mixture-of-experts layers.  Rows (tokens) are sorted by group (expert) and every group's segment is padded
// with zero rows to a multiple of 128, so no 128-row block straddles two groups; the group boundaries live in device memory,
// and nothing about them is read back by the host.
namespace lvb {
namespace gemm {

template <int BN, bool A_MN, bool B_MN>
int launch_grouped(const void* A, const void* B, Params p, int a_rows, int a_cols, int lda, int b_rows, int b_cols, int ldb,
                   cudaStream_t stream) {
  using L = SmemLayout<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(&tmA, A, a_rows, a_cols, lda, BM, BK);
  else       rc = make_tmap_2d_bf16(&tmA, A, a_rows, a_cols, lda, BK, 64);
  if (rc != kErrOk) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tmB, B, b_rows, b_cols, ldb, BN, BK);
  else       rc = make_tmap_2d_bf16(&tmB, B, b_rows, b_cols, ldb, BK, 64);
  if (rc != kErrOk) return rc;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  auto kern = gemm_grouped_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  int grid = p.tiles_m * p.tiles_n;
  if (grid > num_sms()) grid = num_sms();
  kern<<<grid, kNumThreads, L::kTotal, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace gemm
}  // namespace lvb

// kind 0, forward:          C[Tp, N] = A[Tp, K] B[g][N, K]^T      A: padded sorted rows; B: [groups, N, K] (row stride ldb)
// kind 1, input gradient:   C[Tp, N] = A[Tp, K] B[g][K, N]        B: [groups, K, N], i.e. the forward weight [groups, out, in] as it is
// kind 2, weight gradient:  C[g][M, N] (+)= A[rows of g, M]^T B[rows of g, N]     A, B: padded sorted rows; C: [groups, M, N]
// tile_group: int32[ceil(Tp / 128)], the group of every 128-row block of A, -1 beyond the last group (kinds 0 and 1).
// offsets:    int32[groups + 1], padded row offsets (multiples of 128) of the groups (kind 2).
// For kinds 0 and 1, Tp is the static capacity of the padded buffer; blocks marked -1 are neither read nor written.
// flags as lvb_gemm_bf16 (kOutF32, kAccumulate); M, N multiples of 8; for kind 2 M must be a multiple of 128.
extern "C" int lvb_gemm_grouped(int kind, const void* A, const void* B, void* C, int groups, int Tp, int M, int N, int K, int lda,
                                int ldb, int ldc, int flags, float alpha, const int* tile_group, const int* offsets, int* status,
                                void* stream) {
  using namespace lvb;
  using namespace lvb::gemm;
  if (groups <= 0 || Tp <= 0 || (Tp % BM) != 0 || N <= 0 || (lda & 7) || (ldb & 7)) return kErrBadArg;
  Params p;
  p.C = C; p.bias = nullptr; p.residual = nullptr;
  p.ldc = ldc; p.ldr = 0;
  p.flags = flags & (kOutF32 | kAccumulate); p.alpha = alpha; p.status = status; p.alpha_dev = nullptr;
  p.a_fmt = p.b_fmt = 0;
  p.rank = 0; p.world = 1; p.m_rot = 0;
  p.a_rows_per_map = 0; p.c_rows_per_rank = 0;
  p.g_tile_group = tile_group; p.g_offsets = offsets; p.g_b_rows = 0; p.g_tiles_m = 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (kind == 0) {
    if (tile_group == nullptr || K <= 0) return kErrBadArg;
    p.M = Tp; p.N = N; p.K = K; p.g_b_rows = N;
    return N > 128 ? launch_grouped<256, false, false>(A, B, p, Tp, K, lda, groups * N, K, ldb, s)
                   : launch_grouped<128, false, false>(A, B, p, Tp, K, lda, groups * N, K, ldb, s);
  }
  if (kind == 1) {
    if (tile_group == nullptr || K <= 0) return kErrBadArg;
    p.M = Tp; p.N = N; p.K = K; p.g_b_rows = K;
    return N > 128 ? launch_grouped<256, false, true>(A, B, p, Tp, K, lda, groups * K, N, ldb, s)
                   : launch_grouped<128, false, true>(A, B, p, Tp, K, lda, groups * K, N, ldb, s);
  }
  if (kind == 2) {
    if (offsets == nullptr || M <= 0 || (M % BM) != 0) return kErrBadArg;
    p.M = groups * M; p.N = N; p.K = Tp; p.g_tiles_m = M / BM;
    return N > 128 ? launch_grouped<256, true, true>(A, B, p, Tp, M, lda, Tp, N, ldb, s)
                   : launch_grouped<128, true, true>(A, B, p, Tp, M, lda, Tp, N, ldb, s);
  }
  return kErrBadArg;
}
