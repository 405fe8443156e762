// Flash attention backward for sm_100a (head_dim 64 or 128, bf16): see the block comment below.
#include "common.cuh"

namespace lvb {
namespace fa {
constexpr int BM = 128;
constexpr int BN = 128;
constexpr int kTileBytes = 128 * 128 * 2;
constexpr int kChunkBytes = 128 * 64 * 2;
__device__ __forceinline__ uint32_t swz_off(int r, int c) {
  const int chunk = c >> 6;
  const int unit = ((c & 63) >> 3) ^ (r & 7);
  return chunk * kChunkBytes + r * 128 + unit * 16 + (c & 7) * 2;
}
}  // namespace fa
}  // namespace lvb

// =====================================================================================================
// Backward.
//
// One CTA owns one block of 128 keys of one (batch, KV head): K and V stay in shared memory, dK and
// dV accumulate in TMEM over every query block that can see these keys (and over the query heads of
// the GQA group).  Per (query head, query block):
//   MMA      S  = Q K^T,  dP = dO V^T                       (TMEM)
//   threads  p  = exp2(s * scale_log2 - lse2),  ds = p * (dp - delta) * scale      one query row per thread,
//            P and dS written as bf16 tiles [query, key] with the 128B swizzle
//   MMA      dV += P^T dO,  dK += dS^T Q,  dQ = dS K        P^T / dS^T are read as MN-major operands of
//                                                           the same tiles, so nothing is transposed
//   threads  dQ tile (TMEM, reusing the S columns) is added to the fp32 dQ accumulator with
//            vector red.global.add
// delta = rowsum(dO * O) comes from a small pre-pass.
namespace lvb {
namespace fa {

constexpr int kBwdThreads = 320;  // warp0 TMA, warp1 MMA, warps 2-5 key columns [0,64), warps 6-9 key columns [64,128)

struct BwdParams {
  float* dQ32;                 // [B, S, Hq, D] fp32, zero-initialised by the caller
  __nv_bfloat16* dK;           // [B, S, Hkv, D]
  __nv_bfloat16* dV;           // [B, S, Hkv, D]
  const float* lse2;           // [B, Hq, S]
  const float* delta;          // [B, Hq, S]
  const int* q_seg;
  const int* k_seg;
  int B, S, Hq, Hkv;           // S: query positions per sequence
  int Sk;                      // key positions per sequence (= S unless the mask has no causal part)
  float scale, soft_cap;
  int window;
  int causal;                  // 0: every key is visible (subject to segment ids); window must be 0 then
  int* status;
};

template <int HD>
struct SmemBT {
  static constexpr int kQKV = 128 * HD * 2;  // a [128 rows, HD] tile: HD / 64 chunks of 64 columns
  static constexpr int kK = 0;
  static constexpr int kV = kK + kQKV;
  static constexpr int kQ = kV + kQKV;
  static constexpr int kDO = kQ + kQKV;
  static constexpr int kP = kDO + kQKV;
  static constexpr int kDS = kP + kTileBytes;
  static constexpr int kBars = kDS + kTileBytes;
  static constexpr int kNumBars = 7;
  static constexpr int kTotal = kBars + kNumBars * 8 + 16 + 1024;
};

template <int HD, bool kSeg, bool kCap>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, BwdParams p) {
  using SmemB = SmemBT<HD>;
  constexpr int D = HD;
  constexpr int kQKV = SmemB::kQKV;
  const bool causal = p.causal != 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SmemB::kBars);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;   // S and dP ready in TMEM
  uint64_t* pds_full = bars + 4;   // P and dS ready in shared memory (S, dP columns consumed)
  uint64_t* mma_done = bars + 5;   // dV, dK, dQ products retired
  uint64_t* s_free = bars + 6;     // dQ read out of the S columns
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + SmemB::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nqb = p.S / BM;
  const int jb = blockIdx.x;
  const int b = blockIdx.y / p.Hkv;
  const int hkv = blockIdx.y % p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int k0 = jb * BN;
  const int ilo = causal ? jb : 0;
  int ihi = nqb - 1;
  if (p.window > 0) {
    const int last_q = k0 + BN - 1 + p.window - 1;
    ihi = min(ihi, last_q / BM);
  }
  const int nq = ihi - ilo + 1;
  const int iters = nq * G;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(mma_done, 1);
    mbar_init(s_free, 8);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    tmem_alloc<512>(tmem_holder);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base;          // also receives dQ
  const uint32_t tmem_dP = tmem_base + 128;
  const uint32_t tmem_dV = tmem_base + 256;
  const uint32_t tmem_dK = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      const int row_k = b * p.Sk + k0;
      mbar_expect_tx(kv_full, 2 * kQKV);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_2d(smem + SmemB::kK + c * kChunkBytes, &tmK, kv_full, hkv * D + 64 * c, row_k);
        tma_load_2d(smem + SmemB::kV + c * kChunkBytes, &tmV, kv_full, hkv * D + 64 * c, row_k);
      }
      bool ok = true;
      for (int t = 0; t < iters && ok; ++t) {
        const int g = t / nq;
        const int i = ilo + (t % nq);
        const int h = hkv * G + g;
        const int row_q = b * p.S + i * BM;
        ok = mbar_wait(qdo_empty, (t & 1) ^ 1, abort_flag, p.status, 900, t);
        if (!ok) break;
        mbar_expect_tx(qdo_full, 2 * kQKV);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_2d(smem + SmemB::kQ + c * kChunkBytes, &tmQ, qdo_full, h * D + 64 * c, row_q);
          tma_load_2d(smem + SmemB::kDO + c * kChunkBytes, &tmDO, qdo_full, h * D + 64 * c, row_q);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, false, false);  // S, dP
      constexpr uint32_t idesc_mm = make_idesc_bf16(128, D, true, true);      // dV, dK: [128 keys, D]
      constexpr uint32_t idesc_km = make_idesc_bf16(128, D, false, true);     // dQ: [128 queries, D]
      const uint32_t sK = smem_u32(smem + SmemB::kK), sV = smem_u32(smem + SmemB::kV);
      const uint32_t sQ = smem_u32(smem + SmemB::kQ), sDO = smem_u32(smem + SmemB::kDO);
      const uint32_t sP = smem_u32(smem + SmemB::kP), sDS = smem_u32(smem + SmemB::kDS);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, 1000, 0);
      for (int t = 0; t < iters && ok; ++t) {
        const uint32_t ph = t & 1;
        ok = mbar_wait(qdo_full, ph, abort_flag, p.status, 1001, t);
        if (!ok) break;
        ok = mbar_wait(s_free, ph ^ 1, abort_flag, p.status, 1002, t);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
          umma_bf16_ss(tmem_S, make_smem_desc(sQ + off, 16, 1024), make_smem_desc(sK + off, 16, 1024), idesc_kk,
                       kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
          umma_bf16_ss(tmem_dP, make_smem_desc(sDO + off, 16, 1024), make_smem_desc(sV + off, 16, 1024), idesc_kk,
                       kk > 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
        ok = mbar_wait(pds_full, ph, abort_flag, p.status, 1003, t);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {  // reduction over the 128 query rows, 16 per step = 2048 B
          const uint32_t off = kk * 2048;
          umma_bf16_ss(tmem_dV, make_smem_desc(sP + off, kChunkBytes, 1024), make_smem_desc(sDO + off, kChunkBytes, 1024),
                       idesc_mm, (t > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {
          const uint32_t off = kk * 2048;
          umma_bf16_ss(tmem_dK, make_smem_desc(sDS + off, kChunkBytes, 1024), make_smem_desc(sQ + off, kChunkBytes, 1024),
                       idesc_mm, (t > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {  // reduction over the 128 keys
          const uint32_t aoff = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
          const uint32_t boff = kk * 2048;
          umma_bf16_ss(tmem_S, make_smem_desc(sDS + aoff, 16, 1024), make_smem_desc(sK + boff, kChunkBytes, 1024),
                       idesc_km, kk > 0 ? 1u : 0u);
        }
        umma_commit(mma_done);
        umma_commit(qdo_empty);
      }
    }
  } else {
    // ------------------------------------------------------------------ P / dS producers, dQ readout, dK/dV epilogue
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;      // which 64 key columns (and which D / 2 columns of dQ / dK / dV)
    const int r = quad * 32 + lane;
    const int cbase = half * 64;
    const int dbase = half * (D / 2);
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int* kseg_g = kSeg ? p.k_seg + b * p.Sk + k0 : nullptr;
    uint8_t* sPp = smem + SmemB::kP;
    uint8_t* sDSp = smem + SmemB::kDS;
    bool ok = true;
    for (int t = 0; t < iters && ok; ++t) {
      const uint32_t ph = t & 1;
      const int g = t / nq;
      const int i = ilo + (t % nq);
      const int h = hkv * G + g;
      const int qi = i * BM + r;
      const size_t stat_idx = (static_cast<size_t>(b) * p.Hq + h) * p.S + qi;
      const float lse = p.lse2[stat_idx];
      const float dlt = p.delta[stat_idx];
      const float neg_lse = (lse == -INFINITY) ? -INFINITY : -lse;
      const int my_seg = kSeg ? p.q_seg[b * p.S + qi] : 0;
      ok = mbar_wait(sdp_full, ph, abort_flag, p.status, 1100, t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = (causal && i == jb) || kSeg || (p.window > 0 && k0 <= i * BM + BM - 1 - p.window);
#pragma unroll 1
      for (int c = cbase; c < cbase + 64; c += 32) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem_S + lane_addr + c, sv);
        tmem_ld_32x32(tmem_dP + lane_addr + c, dv);
        tmem_ld_wait();
        float pe[32], de[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          float x, dcap = p.scale;
          if constexpr (kCap) {
            const float th = tanhf(__uint_as_float(sv[u]) * p.scale / p.soft_cap);
            x = p.soft_cap * th * 1.4426950408889634f + neg_lse;
            dcap = p.scale * (1.f - th * th);
          } else {
            x = fmaf(__uint_as_float(sv[u]), scale_log2, neg_lse);
          }
          float pv = exp2f(x);
          if (need_mask) {
            const int kj = k0 + c + u;
            bool valid = !causal || kj <= qi;
            if (p.window > 0) valid = valid && (qi - kj < p.window);
            if (kSeg) valid = valid && (kseg_g[c + u] == my_seg);
            pv = valid ? pv : 0.f;
          }
          pe[u] = pv;
          de[u] = pv * (__uint_as_float(dv[u]) - dlt) * dcap;
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
          const uint32_t off = swz_off(r, c + q4 * 8);
          *reinterpret_cast<uint4*>(sPp + off) = w;
          *reinterpret_cast<uint4*>(sDSp + off) = x;
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);

      // dQ tile of this (head, query block): TMEM -> fp32 accumulator in global memory (this warp's D / 2 columns)
      ok = mbar_wait(mma_done, ph, abort_flag, p.status, 1101, t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float* dq = p.dQ32 + (static_cast<size_t>(b) * p.S + qi) * (static_cast<size_t>(p.Hq) * D) + static_cast<size_t>(h) * D;
#pragma unroll 1
      for (int c = dbase; c < dbase + D / 2; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_S + lane_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) {
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq + c + q4 * 4),
                       "f"(__uint_as_float(v[q4 * 4 + 0])), "f"(__uint_as_float(v[q4 * 4 + 1])),
                       "f"(__uint_as_float(v[q4 * 4 + 2])), "f"(__uint_as_float(v[q4 * 4 + 3]))
                       : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
    }

    // epilogue: dK, dV -> bf16 (this warp's D / 2 columns)
    if (ok) {
      tc_fence_after();
      const size_t row = (static_cast<size_t>(b) * p.Sk + k0 + r) * (static_cast<size_t>(p.Hkv) * D) + static_cast<size_t>(hkv) * D;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? p.dV : p.dK) + row;
        const uint32_t src = (which == 0 ? tmem_dV : tmem_dK) + lane_addr;
#pragma unroll 1
        for (int c = dbase; c < dbase + D / 2; c += 32) {
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

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (b, s, h) row of D values
template <int D>
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                   float* __restrict__ delta, int B, int S, int H) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long rows = static_cast<long long>(B) * S * H;
  if (row >= rows) return;
  constexpr int kPairs = D / 64;  // bf16 pairs per lane
  float acc = 0.f;
#pragma unroll
  for (int t = 0; t < kPairs; ++t) {
    const float2 x = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(O + row * D)[lane * kPairs + t]);
    const float2 y = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dO + row * D)[lane * kPairs + t]);
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


template <int HD>
int launch_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, BwdParams p, cudaStream_t st) {
  using SmemB = SmemBT<HD>;
  {
    const long long rows = static_cast<long long>(p.B) * p.S * p.Hq;
    const int block = 256;
    const long long grid = (rows * 32 + block - 1) / block;
    flash_delta_kernel<HD><<<static_cast<unsigned>(grid), block, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(o),
                                                                          reinterpret_cast<const __nv_bfloat16*>(d_o),
                                                                          const_cast<float*>(p.delta), p.B, p.S, p.Hq);
  }
  CUtensorMap tmQ, tmK, tmV, tmDO;
  const uint64_t rows = static_cast<uint64_t>(p.B) * p.S;
  int rc = make_tmap_2d_bf16(&tmQ, q, rows, static_cast<uint64_t>(p.Hq) * HD, static_cast<uint64_t>(p.Hq) * HD, BM, 64);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_bf16(&tmDO, d_o, rows, static_cast<uint64_t>(p.Hq) * HD, static_cast<uint64_t>(p.Hq) * HD, BM, 64);
  if (rc != kErrOk) return rc;
  const uint64_t rows_k = static_cast<uint64_t>(p.B) * p.Sk;
  rc = make_tmap_2d_bf16(&tmK, k, rows_k, static_cast<uint64_t>(p.Hkv) * HD, static_cast<uint64_t>(p.Hkv) * HD, BN, 64);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_bf16(&tmV, v, rows_k, static_cast<uint64_t>(p.Hkv) * HD, static_cast<uint64_t>(p.Hkv) * HD, BN, 64);
  if (rc != kErrOk) return rc;
  dim3 grid(p.Sk / BN, p.B * p.Hkv);
  const bool seg = p.q_seg != nullptr;
  const bool cap = p.soft_cap > 0.f;
#define LVB_LAUNCH_BWD(SEG, CAP)                                                                                      \
  do {                                                                                                                \
    auto kern = flash_bwd_kernel<HD, SEG, CAP>;                                                                       \
    static bool attr_set = false;                                                                                     \
    if (!attr_set) {                                                                                                  \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemB::kTotal) != cudaSuccess)      \
        return kErrCuda;                                                                                              \
      attr_set = true;                                                                                                \
    }                                                                                                                 \
    kern<<<grid, kBwdThreads, SmemB::kTotal, st>>>(tmQ, tmK, tmV, tmDO, p);                                           \
  } while (0)
  if (seg && cap) LVB_LAUNCH_BWD(true, true);
  else if (seg) LVB_LAUNCH_BWD(true, false);
  else if (cap) LVB_LAUNCH_BWD(false, true);
  else LVB_LAUNCH_BWD(false, false);
#undef LVB_LAUNCH_BWD
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace fa
}  // namespace lvb

// Backward of lvb_flash_attn_fwd_hd.  dq32: fp32 [B,S,Hq,D], must be zero on entry.  delta: fp32 [B,Hq,S] scratch.  D = head_dim
// is 64 or 128; causal and Sk (keys per sequence: k / v / dk / dv are [B, Sk, Hkv, D]) as in the forward.
extern "C" int lvb_flash_attn_bwd_hd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                     const float* lse2, float* delta, float* dq32, void* dk, void* dv, const int* q_seg,
                                     const int* k_seg, int B, int S, int Sk, int Hq, int Hkv, int head_dim, int causal, float scale,
                                     float soft_cap, int window, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::fa;
  if (B <= 0 || S <= 0 || (S % BM) != 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv) != 0) return kErrBadArg;
  if (!causal && window != 0) return kErrBadArg;
  if (Sk <= 0 || (Sk % BN) != 0 || (causal && Sk != S)) return kErrBadArg;
  BwdParams p;
  p.dQ32 = dq32;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.lse2 = lse2;
  p.delta = delta;
  p.q_seg = q_seg;
  p.k_seg = k_seg;
  p.B = B; p.S = S; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.soft_cap = soft_cap; p.window = window;
  p.causal = causal ? 1 : 0;
  p.status = status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (head_dim == 128) return launch_bwd<128>(q, k, v, o, d_o, p, st);
  if (head_dim == 64) return launch_bwd<64>(q, k, v, o, d_o, p, st);
  return kErrBadArg;
}

// Causal, head_dim 128 (the original entry point).
extern "C" int lvb_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                  const float* lse2, float* delta, float* dq32, void* dk, void* dv, const int* q_seg,
                                  const int* k_seg, int B, int S, int Hq, int Hkv, float scale, float soft_cap,
                                  int window, int* status, void* stream) {
  return lvb_flash_attn_bwd_hd(q, k, v, o, d_o, lse2, delta, dq32, dk, dv, q_seg, k_seg, B, S, S, Hq, Hkv, 128, 1, scale, soft_cap, window,
                               status, stream);
}
