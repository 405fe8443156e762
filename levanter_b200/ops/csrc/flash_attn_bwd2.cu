// Flash attention backward for sm_100a (head_dim 128, bf16), software-pipelined.
//
// One CTA owns one block of 128 keys of one (batch, KV head): K and V stay in shared memory, dK and dV accumulate in TMEM
// over every block of 64 queries that can see these keys (and over the query heads of the GQA group).  Everything is
// computed TRANSPOSED, keys on the 128 TMEM lanes and queries along the columns:
//
//   MMA      S^T = K Q^T,  dP^T = V dO^T                           [128 keys, 64 queries] each
//   threads  p = exp2(s * scale_log2 - lse2[q]),  ds = p * (dp - delta[q]) * scale       one key row per thread;
//            P^T and dS^T written as bf16 tiles [key, query] with the 128B swizzle
//   MMA      dV += P^T dO,  dK += dS^T Q                            P^T / dS^T are K-major A operands, dO / Q MN-major B
//            dQ^T = K^T dS^T                                        [128 d, 64 queries], written over the S^T columns
//   threads  dQ^T (TMEM) is transposed into a [64 queries, 128 d] fp32 tile in shared memory (the step's own P^T / dS^T tiles,
//            free by then) and added to the fp32 dQ accumulator by ONE bulk tensor reduction (cp.reduce.async.bulk.tensor
//            ... .add): the L2 sees whole 512-byte rows instead of one reduction instruction per element, which is what
//            bounded the per-element version (the dQ traffic is 2 GB of fp32 adds for B2 S4096 H32)
//
// Because a 64-query step needs only 64 + 64 TMEM columns for S^T / dP^T, there is room for two such pairs beside the
// 2 x 128 columns of dV / dK, and the shared memory holds two Q / dO tiles and two P^T / dS^T tiles.  Two softmax warpgroups
// take alternate steps, each with its own TMEM pair and shared tiles, so the single MMA thread issues the S^T / dP^T
// products of step t+1 and the dV / dK / dQ^T products of step t-1 while a warpgroup is busy with the exponentials of step
// t: the tensor cores no longer wait for the softmax and vice versa (the one-buffer kernel in flash_attn_bwd.cu ran the
// five products and the elementwise phase strictly one after the other).
//
// Masks: causal, sliding window, segment ids; logit soft-cap.  delta = rowsum(dO * O) comes from the pre-pass in
// this file.  Semantics of the reference's fused attention (src/levanter/layers/attention.py:533-544,
// src/levanter/models/flash_attention.py:143-385).
#include "common.cuh"

namespace lvb {
namespace fab2 {

constexpr int BKEYS = 128;
constexpr int BQ = 64;
constexpr int D = 128;
constexpr int kKVChunk = 128 * 64 * 2;  // [128 rows, 64 cols] bf16
constexpr int kKVTile = 2 * kKVChunk;
constexpr int kQChunk = 64 * 64 * 2;    // [64 rows, 64 cols]
constexpr int kQTile = 2 * kQChunk;
constexpr int kPTile = 128 * 64 * 2;    // [128 keys, 64 queries], one swizzle chunk
constexpr int kThreads = 320;           // warp0 TMA, warp1 MMA, warps 2-5 warpgroup 0 (even steps), warps 6-9 warpgroup 1 (odd steps)

struct Params {
  float* dQ32;         // [B, S, Hq, D] fp32, zero-initialised by the caller
  __nv_bfloat16* dK;   // [B, S, Hkv, D]
  __nv_bfloat16* dV;   // [B, S, Hkv, D]
  const float* lse2;   // [B, Hq, S]
  const float* delta;  // [B, Hq, S]
  const int* q_seg;
  const int* k_seg;
  int B, S, Hq, Hkv;
  float scale, soft_cap;
  int window;
  int* status;
};

struct Smem {
  static constexpr int kK = 0;
  static constexpr int kV = kK + kKVTile;
  static constexpr int kQ = kV + kKVTile;          // two buffers of {Q tile, dO tile}
  static constexpr int kP = kQ + 2 * 2 * kQTile;   // two buffers of {P^T tile, dS^T tile}
  static constexpr int kStat = kP + 2 * 2 * kPTile;  // per warpgroup: lse2[64], delta[64], q_seg[64]
  static constexpr int kBars = kStat + 2 * 3 * 64 * 4;
  static constexpr int kNumBars = 13;
  static constexpr int kTotal = kBars + kNumBars * 8 + 16 + 1024;
};

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (b, s, h) row of 128 values
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO, float* __restrict__ delta, int B, int S,
                             int H) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long rows = static_cast<long long>(B) * S * H;
  if (row >= rows) return;
  const uint2 a = reinterpret_cast<const uint2*>(O + row * D)[lane];
  const uint2 g = reinterpret_cast<const uint2*>(dO + row * D)[lane];
  const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
  float acc = 0.f;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    float2 x = __bfloat1622float2(ah[t]);
    float2 y = __bfloat1622float2(gh[t]);
    acc += x.x * y.x + x.y * y.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const int h = static_cast<int>(row % H);
    const long long bs = row / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    delta[(static_cast<long long>(b) * H + h) * S + s] = acc;
  }
}

__device__ __forceinline__ uint32_t swz64(int r, int c) {  // element (r, c) of a [rows, 64] bf16 tile with the 128B swizzle
  return static_cast<uint32_t>(r * 128 + ((((c >> 3) ^ (r & 7))) << 4) + ((c & 7) << 1));
}
__device__ __forceinline__ void wg_bar_sync(int wg) { asm volatile("bar.sync %0, 128;" ::"r"(wg + 1) : "memory"); }

template <bool kSeg, bool kCap>
__global__ void __launch_bounds__(kThreads, 1)
flash_bwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                  const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmDQ, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* sdp_full = bars + 5;   // [2] S^T and dP^T ready in TMEM
  uint64_t* pds_full = bars + 7;   // [2] P^T and dS^T ready in shared memory (S^T, dP^T columns consumed)
  uint64_t* dq_done = bars + 9;    // [2] dV, dK, dQ^T products of the step retired
  uint64_t* s_free = bars + 11;    // [2] dQ^T read out of the S^T columns
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nqb = p.S / BQ;
  const int jb = blockIdx.x;
  const int b = blockIdx.y / p.Hkv;
  const int hkv = blockIdx.y % p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int k0 = jb * BKEYS;
  const int ilo = k0 / BQ;  // first block of 64 queries that can see a key of this block
  int ihi = nqb - 1;
  if (p.window > 0) {
    const int last_q = k0 + BKEYS - 1 + p.window - 1;
    ihi = min(ihi, last_q / BQ);
  }
  const int nq = ihi - ilo + 1;
  const int iters = nq * G;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&pds_full[i], 4);
      mbar_init(&dq_done[i], 1);
      mbar_init(&s_free[i], 4);
    }

    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQ);
  }
  if (warp == 1) {
    tmem_alloc<512>(tmem_holder);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // pair w: S^T at columns [128 w, 128 w + 64) (later dQ^T), dP^T at [128 w + 64, 128 w + 128)
  const uint32_t tmem_dV = tmem_base + 256;
  const uint32_t tmem_dK = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int row_k = b * p.S + k0;
      mbar_expect_tx(kv_full, 2 * kKVTile);
      tma_load_2d(smem + Smem::kK, &tmK, kv_full, hkv * D, row_k);
      tma_load_2d(smem + Smem::kK + kKVChunk, &tmK, kv_full, hkv * D + 64, row_k);
      tma_load_2d(smem + Smem::kV, &tmV, kv_full, hkv * D, row_k);
      tma_load_2d(smem + Smem::kV + kKVChunk, &tmV, kv_full, hkv * D + 64, row_k);
      bool ok = true;
      for (int t = 0; t < iters && ok; ++t) {
        const int g = t / nq;
        const int i = ilo + (t % nq);
        const int h = hkv * G + g;
        const int row_q = b * p.S + i * BQ;
        const int bf = t & 1;
        ok = mbar_wait(&qdo_empty[bf], ((t >> 1) & 1) ^ 1, abort_flag, p.status, 900, t);
        if (!ok) break;
        uint8_t* sq = smem + Smem::kQ + bf * (2 * kQTile);
        uint8_t* sdo = sq + kQTile;
        mbar_expect_tx(&qdo_full[bf], 2 * kQTile);
        tma_load_2d(sq, &tmQ, &qdo_full[bf], h * D, row_q);
        tma_load_2d(sq + kQChunk, &tmQ, &qdo_full[bf], h * D + 64, row_q);
        tma_load_2d(sdo, &tmDO, &qdo_full[bf], h * D, row_q);
        tma_load_2d(sdo + kQChunk, &tmDO, &qdo_full[bf], h * D + 64, row_q);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, false, false);   // S^T, dP^T: both operands K-major
      constexpr uint32_t idesc_dv = make_idesc_bf16(128, 128, false, true);   // dV, dK: A K-major, B MN-major
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, true, true);     // dQ^T: both MN-major
      const uint32_t sK = smem_u32(smem + Smem::kK), sV = smem_u32(smem + Smem::kV);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, 1000, 0);
      for (int t = 0; t <= iters && ok; ++t) {
        if (t < iters) {
          const int bf = t & 1;
          const uint32_t n = static_cast<uint32_t>(t >> 1);
          const uint32_t sQ = smem_u32(smem + Smem::kQ + bf * (2 * kQTile)), sDO = sQ + kQTile;
          const uint32_t tmem_ST = tmem_base + bf * 128, tmem_dPT = tmem_ST + 64;
          ok = mbar_wait(&qdo_full[bf], n & 1, abort_flag, p.status, 1001, t);
          if (!ok) break;
          ok = mbar_wait(&s_free[bf], (n & 1) ^ 1, abort_flag, p.status, 1002, t);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t aoff = (kk >> 2) * kKVChunk + (kk & 3) * 32;
            const uint32_t boff = (kk >> 2) * kQChunk + (kk & 3) * 32;
            umma_bf16_ss(tmem_ST, make_smem_desc(sK + aoff, 16, 1024), make_smem_desc(sQ + boff, 16, 1024), idesc_st, kk > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t aoff = (kk >> 2) * kKVChunk + (kk & 3) * 32;
            const uint32_t boff = (kk >> 2) * kQChunk + (kk & 3) * 32;
            umma_bf16_ss(tmem_dPT, make_smem_desc(sV + aoff, 16, 1024), make_smem_desc(sDO + boff, 16, 1024), idesc_st, kk > 0 ? 1u : 0u);
          }
          umma_commit(&sdp_full[bf]);
        }
        if (t >= 1) {
          const int u = t - 1;
          const int bf = u & 1;
          const uint32_t n = static_cast<uint32_t>(u >> 1);
          const uint32_t sQ = smem_u32(smem + Smem::kQ + bf * (2 * kQTile)), sDO = sQ + kQTile;
          const uint32_t sPT = smem_u32(smem + Smem::kP + bf * (2 * kPTile)), sDST = sPT + kPTile;
          const uint32_t tmem_dQT = tmem_base + bf * 128;
          ok = mbar_wait(&pds_full[bf], n & 1, abort_flag, p.status, 1003, u);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < BQ / 16; ++kk) {  // reduction over the 64 queries
            umma_bf16_ss(tmem_dV, make_smem_desc(sPT + kk * 32, 16, 1024), make_smem_desc(sDO + kk * 2048, kQChunk, 1024), idesc_dv,
                         (u > 0 || kk > 0) ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < BQ / 16; ++kk) {
            umma_bf16_ss(tmem_dK, make_smem_desc(sDST + kk * 32, 16, 1024), make_smem_desc(sQ + kk * 2048, kQChunk, 1024), idesc_dv,
                         (u > 0 || kk > 0) ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < BKEYS / 16; ++kk) {  // reduction over the 128 keys
            umma_bf16_ss(tmem_dQT, make_smem_desc(sK + kk * 2048, kKVChunk, 1024), make_smem_desc(sDST + kk * 2048, kPTile, 1024), idesc_dq,
                         kk > 0 ? 1u : 0u);
          }
          umma_commit(&dq_done[bf]);
          umma_commit(&qdo_empty[bf]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups: P^T / dS^T, dQ^T readout, dK / dV epilogue
    const int wg = (warp - 2) >> 2;  // takes the steps t with t % 2 == wg
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // key row of this thread
    const int wtid = threadIdx.x - 64 - wg * 128;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int kj = k0 + r;
    const int my_kseg = kSeg ? p.k_seg[b * p.S + kj] : 0;
    float* s_lse = reinterpret_cast<float*>(smem + Smem::kStat + wg * (3 * 64 * 4));
    float* s_dlt = s_lse + 64;
    int* s_qseg = reinterpret_cast<int*>(s_dlt + 64);
    uint8_t* sPT = smem + Smem::kP + wg * (2 * kPTile);
    uint8_t* sDST = sPT + kPTile;
    const uint32_t tmem_ST = tmem_base + wg * 128, tmem_dPT = tmem_ST + 64;
    bool ok = true;
    // The per-query statistics of a step (64 x {-lse, delta, segment id}) are fetched one step of this warpgroup ahead into a
    // register per thread, so the global-memory latency is not paid between the two barriers that open a step.
    float pre_stat = 0.f;
    int pre_seg = 0;
    auto fetch_stats = [&](int tt) {
      if (tt >= iters) return;
      const int hh = hkv * G + tt / nq;
      const int qq = (ilo + (tt % nq)) * BQ;
      const size_t stat = (static_cast<size_t>(b) * p.Hq + hh) * p.S + qq;
      pre_stat = (wtid < 64) ? p.lse2[stat + wtid] : p.delta[stat + wtid - 64];
      if (kSeg && wtid < 64) pre_seg = p.q_seg[b * p.S + qq + wtid];
    };
    fetch_stats(wg);
    for (int t = wg; t < iters; t += 2) {
      const uint32_t n = static_cast<uint32_t>(t >> 1);
      const int g = t / nq;
      const int i = ilo + (t % nq);
      const int h = hkv * G + g;
      const int q0 = i * BQ;
      // Every warp of the warpgroup passes the three named barriers of a step whatever happened to its waits (a wait that
      // ran out clears `ok` and the work is skipped), or the others would wait for it for ever.
      wg_bar_sync(wg);  // the previous step no longer reads the statistics, and its dQ tile has been handed to the TMA unit
      if (ok) {
        if (wtid < 64) {
          s_lse[wtid] = (pre_stat == -INFINITY) ? -INFINITY : -pre_stat;
        } else {
          s_dlt[wtid - 64] = pre_stat;
        }
        if (kSeg && wtid < 64) s_qseg[wtid] = pre_seg;
        fetch_stats(t + 2);
        // the bulk reduction of the previous step must have read its tile before this step's P^T / dS^T overwrite it
        if (wtid == 0) bulk_wait_read<0>();
      }
      wg_bar_sync(wg);
      if (ok) {
        ok = mbar_wait(&sdp_full[wg], n & 1, abort_flag, p.status, 1100, t);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        const bool need_mask = (q0 < k0 + BKEYS) || kSeg || (p.window > 0 && k0 <= q0 + BQ - 1 - p.window);
#pragma unroll 1
        for (int c = 0; c < BQ; c += 32) {
          uint32_t sv[32], dv[32];
          tmem_ld_32x32(tmem_ST + lane_addr + c, sv);
          tmem_ld_32x32(tmem_dPT + lane_addr + c, dv);
          tmem_ld_wait();
          float pe[32], de[32];
#pragma unroll
          for (int u = 0; u < 32; ++u) {
            float x, dcap = p.scale;
            const float neg_lse = s_lse[c + u];
            if constexpr (kCap) {
              const float th = tanhf(__uint_as_float(sv[u]) * p.scale / p.soft_cap);
              x = p.soft_cap * th * 1.4426950408889634f + neg_lse;
              dcap = p.scale * (1.f - th * th);
            } else {
              x = fmaf(__uint_as_float(sv[u]), scale_log2, neg_lse);
            }
            float pv = exp2f(x);
            if (need_mask) {
              const int qi = q0 + c + u;
              bool valid = kj <= qi;
              if (p.window > 0) valid = valid && (qi - kj < p.window);
              if (kSeg) valid = valid && (s_qseg[c + u] == my_kseg);
              pv = valid ? pv : 0.f;
            }
            pe[u] = pv;
            de[u] = pv * (__uint_as_float(dv[u]) - s_dlt[c + u]) * dcap;
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w, x;
            w.x = pack_bf16x2(pe[q4 * 8 + 0], pe[q4 * 8 + 1]);
            w.y = pack_bf16x2(pe[q4 * 8 + 2], pe[q4 * 8 + 3]);
            w.z = pack_bf16x2(pe[q4 * 8 + 4], pe[q4 * 8 + 5]);
            w.w = pack_bf16x2(pe[q4 * 8 + 6], pe[q4 * 8 + 7]);
            x.x = pack_bf16x2(de[q4 * 8 + 0], de[q4 * 8 + 1]);
            x.y = pack_bf16x2(de[q4 * 8 + 2], de[q4 * 8 + 3]);
            x.z = pack_bf16x2(de[q4 * 8 + 4], de[q4 * 8 + 5]);
            x.w = pack_bf16x2(de[q4 * 8 + 6], de[q4 * 8 + 7]);
            const uint32_t off = swz64(r, c + q4 * 8);
            *reinterpret_cast<uint4*>(sPT + off) = w;
            *reinterpret_cast<uint4*>(sDST + off) = x;
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pds_full[wg]);
        // dQ^T of this step: TMEM [d = lane, query = column] -> fp32 tile [query][d] in the shared memory that held this step's
        // P^T and dS^T (the products that read them have retired once dq_done completes)
        ok = mbar_wait(&dq_done[wg], n & 1, abort_flag, p.status, 1101, t);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        float* stage = reinterpret_cast<float*>(sPT);  // 64 x 128 fp32 = the 32 KB of the two tiles
#pragma unroll 1
        for (int c = 0; c < BQ; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_ST + lane_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 32; ++u) stage[(c + u) * D + r] = __uint_as_float(v[u]);
        }
        tc_fence_before();
        fence_proxy_async_smem();  // these generic-proxy writes are read by the bulk reduction below
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[wg]);
      }
      wg_bar_sync(wg);
      if (ok && wtid == 0) {
        // dQ[b, q0 .. q0 + 63, h, :] += tile, one bulk tensor reduction
        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                         reinterpret_cast<uint64_t>(&tmDQ)),
                     "r"(smem_u32(sPT)), "r"(h * D), "r"(b * p.S + q0)
                     : "memory");
        bulk_commit();  // waited for (read side) at the top of this warpgroup's next step
      }
    }
    if (wtid == 0) bulk_wait<0>();  // every reduction of this warpgroup has been performed before the CTA leaves

    // epilogue: dK, dV -> bf16 (this warpgroup's 64 d columns), once the last step's dV / dK products have retired (the
    // commit on qdo_empty follows them)
    if (ok && iters > 0) {
      const int last = iters - 1;
      ok = mbar_wait(&qdo_empty[last & 1], static_cast<uint32_t>(last >> 1) & 1, abort_flag, p.status, 1102, last);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const int cbase = wg * 64;
      const size_t row = (static_cast<size_t>(b) * p.S + k0 + r) * (static_cast<size_t>(p.Hkv) * D) + static_cast<size_t>(hkv) * D;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? p.dV : p.dK) + row;
        const uint32_t src = (which == 0 ? tmem_dV : tmem_dK) + lane_addr;
#pragma unroll 1
        for (int c = cbase; c < cbase + 64; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(src + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
            reinterpret_cast<uint4*>(dst + c)[q4] = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

}  // namespace fab2
}  // namespace lvb

// Backward of lvb_flash_attn_fwd, pipelined form (same arguments as lvb_flash_attn_bwd).  dq32: fp32 [B,S,Hq,128], must be
// zero on entry.  delta: fp32 [B,Hq,S] scratch.
extern "C" int lvb_flash_attn_bwd2(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2,
                                   float* delta, float* dq32, void* dk, void* dv, const int* q_seg, const int* k_seg, int B, int S,
                                   int Hq, int Hkv, float scale, float soft_cap, int window, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::fab2;
  if (B <= 0 || S <= 0 || (S % BKEYS) != 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv) != 0) return kErrBadArg;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  {
    const long long rows = static_cast<long long>(B) * S * Hq;
    const int block = 256;
    const long long grid = (rows * 32 + block - 1) / block;
    delta_kernel<<<static_cast<unsigned>(grid), block, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(o),
                                                                reinterpret_cast<const __nv_bfloat16*>(d_o), delta, B, S, Hq);
  }
  CUtensorMap tmQ, tmK, tmV, tmDO;
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  int rc = make_tmap_2d_bf16(&tmQ, q, rows, static_cast<uint64_t>(Hq) * D, static_cast<uint64_t>(Hq) * D, BQ, 64);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_bf16(&tmDO, d_o, rows, static_cast<uint64_t>(Hq) * D, static_cast<uint64_t>(Hq) * D, BQ, 64);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_bf16(&tmK, k, rows, static_cast<uint64_t>(Hkv) * D, static_cast<uint64_t>(Hkv) * D, BKEYS, 64);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_bf16(&tmV, v, rows, static_cast<uint64_t>(Hkv) * D, static_cast<uint64_t>(Hkv) * D, BKEYS, 64);
  if (rc != kErrOk) return rc;
  // dQ accumulator as a [B * S, Hq * D] fp32 matrix, box [64 rows, 128 columns], no swizzle (the shared-memory tile is row-major)
  CUtensorMap tmDQ;
  {
    EncodeTiledFn enc = get_encode_tiled();
    if (enc == nullptr) return kErrTensorMap;
    if ((reinterpret_cast<uintptr_t>(dq32) & 15) != 0) return kErrBadArg;
    cuuint64_t gdim[2] = {static_cast<cuuint64_t>(Hq) * D, rows};
    cuuint64_t gstr[1] = {static_cast<cuuint64_t>(Hq) * D * 4};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(D), static_cast<cuuint32_t>(BQ)};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&tmDQ, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dq32, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return kErrTensorMap;
  }
  Params p;
  p.dQ32 = dq32;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.lse2 = lse2;
  p.delta = delta;
  p.q_seg = q_seg;
  p.k_seg = k_seg;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.soft_cap = soft_cap; p.window = window;
  p.status = status;
  dim3 grid(S / BKEYS, B * Hkv);
  const bool seg = q_seg != nullptr;
  const bool cap = soft_cap > 0.f;
#define LVB_LAUNCH_BWD2(SEG, CAP)                                                                                    \
  do {                                                                                                               \
    auto kern = flash_bwd2_kernel<SEG, CAP>;                                                                         \
    static bool attr_set = false;                                                                                    \
    if (!attr_set) {                                                                                                 \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal) != cudaSuccess)      \
        return kErrCuda;                                                                                             \
      attr_set = true;                                                                                               \
    }                                                                                                                \
    kern<<<grid, kThreads, Smem::kTotal, st>>>(tmQ, tmK, tmV, tmDO, tmDQ, p);                                             \
  } while (0)
  if (seg && cap) LVB_LAUNCH_BWD2(true, true);
  else if (seg) LVB_LAUNCH_BWD2(true, false);
  else if (cap) LVB_LAUNCH_BWD2(false, true);
  else LVB_LAUNCH_BWD2(false, false);
#undef LVB_LAUNCH_BWD2
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
