// Flash attention forward, two query tiles per CTA (sequence length a multiple of 256, head_dim 128).
//
// Compared with the one-tile kernel in flash_attn.cu this variant
//   * keeps two 128-row query tiles A and B per CTA, so every K/V tile fetched by TMA is used twice and
//     eight softmax warps (two per scheduler) hide each other's instruction latency;
//   * writes P back into the TMEM columns of S (bf16, two values per 32-bit column) and issues the
//     P V product with the A operand read from tensor memory, so P never touches shared memory;
//   * ping-pongs the tiles on the tensor core: while tile A's rows are in softmax the MMA warp runs
//     P_B V and Q_B K^T, and vice versa.
// TMEM map (512 columns): S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,384)  O_B [384,512).
// Shared memory: Q_A, Q_B, two K stages, two V stages (6 x 32 KB).
// Mask semantics, outputs and the lazy-rescale rule are those of flash_fwd_kernel.
#include "common.cuh"

namespace lvb {
namespace fa2 {

constexpr int BT = 128;            // rows per query tile, keys per block
constexpr int kThreads = 320;      // warp0 TMA, warp1 MMA, warps 2-5 tile A, warps 6-9 tile B
constexpr int kTileBytes = 128 * 128 * 2;
constexpr int kChunkBytes = 128 * 64 * 2;
constexpr int kStages = 2;
constexpr float kRescaleThreshold = 8.0f;
constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  __nv_bfloat16* O;
  float* lse2;
  const int* q_seg;
  const int* k_seg;
  const int* kblock_lo;  // optional [B, S / 128]: first block of 128 keys that a query of this 128-row block can attend to
  const float* sink;     // optional [Hq]: a learned logit per head that takes part in the softmax denominator only
  int B, S, Hq, Hkv;  // S: query positions per sequence
  int Sk;             // key positions per sequence (= S unless the mask has no causal part: cross attention)
  float scale, soft_cap;
  int window;
  int causal;  // 0: every key is visible (subject to segment ids); window must be 0 and kblock_lo null then
  int* status;
};

template <int HD>
struct SmemT {
  static constexpr int kQKV = 128 * HD * 2;                   // a [128 rows, HD] tile: HD / 64 chunks of 64 columns
  static constexpr int kQ = 0;                                // 2 tiles
  static constexpr int kK = kQ + 2 * kQKV;
  static constexpr int kV = kK + kStages * kQKV;
  static constexpr int kBars = kV + kStages * kQKV;
  static constexpr int kNumBars = 1 + 4 * kStages + 2 + 2 + 2;
  static constexpr int kTotal = kBars + kNumBars * 8 + 16 + 1024;
};

template <bool kCap>
__device__ __forceinline__ float to_log2(float s, float scale_log2, float scale, float cap) {
  if constexpr (kCap) return cap * tanhf(s * scale / cap) * kLog2e;
  else return s * scale_log2;
}

template <int HD, bool kSeg, bool kCap>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, Params p) {
  using Smem = SmemT<HD>;
  constexpr int D = HD;
  constexpr int kQKV = Smem::kQKV;
  const bool causal = p.causal != 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + kStages;
  uint64_t* v_full = k_empty + kStages;
  uint64_t* v_empty = v_full + kStages;
  uint64_t* s_full = v_empty + kStages;  // [2 tiles]
  uint64_t* p_full = s_full + 2;         // [2 tiles]
  uint64_t* o_done = p_full + 2;         // [2 tiles]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int ncta = p.S / (2 * BT);
  const int cb = ncta - 1 - static_cast<int>(blockIdx.x);  // heaviest first
  const int b = blockIdx.y / p.Hq;
  const int h = blockIdx.y % p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = cb * 2 * BT;
  // without the causal part there is no diagonal block (the mask test below never matches -1) and both tiles see every block
  const int jdiagA = causal ? 2 * cb : -1, jdiagB = causal ? 2 * cb + 1 : -1;
  int jlo = 0;
  if (p.window > 0) {
    const int first_key = q0 - p.window + 1;
    jlo = first_key > 0 ? first_key / BT : 0;
  }
  if (p.kblock_lo != nullptr) {
    // packed sequences (segment ids ascending): key blocks before the first query's sequence hold nothing these rows can see
    const int lo = p.kblock_lo[b * (p.S / BT) + jdiagA];
    jlo = max(jlo, min(lo, jdiagA));
  }
  const int nB = (causal ? jdiagB : p.Sk / BT - 1) - jlo + 1;  // blocks processed by tile B
  const int nA = causal ? nB - 1 : nB;                        // causal: tile A stops one block earlier (its diagonal)

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);
      mbar_init(&o_done[t], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int row_q = b * p.S + q0;
      mbar_expect_tx(q_full, 2 * kQKV);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_2d(smem + Smem::kQ + t * kQKV + c * kChunkBytes, &tmQ, q_full, h * D + 64 * c, row_q + t * BT);
      bool ok = true;
      for (int it = 0; it < nB && ok; ++it) {
        const int st = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        const int row_k = b * p.Sk + (jlo + it) * BT;
        ok = mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, 1200, it);
        if (!ok) break;
        uint8_t* ks = smem + Smem::kK + st * kQKV;
        mbar_expect_tx(&k_full[st], kQKV);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(ks + c * kChunkBytes, &tmK, &k_full[st], hkv * D + 64 * c, row_k);
        ok = mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, 1201, it);
        if (!ok) break;
        uint8_t* vs = smem + Smem::kV + st * kQKV;
        mbar_expect_tx(&v_full[st], kQKV);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(vs + c * kChunkBytes, &tmV, &v_full[st], hkv * D + 64 * c, row_k);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BT, BT, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BT, D, false, true);  // A = P in TMEM, B = V MN-major
      const uint32_t sq = smem_u32(smem + Smem::kQ);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 1300, 0);

      auto qk = [&](int tile, int it) {
        const int st = it % kStages;
        const uint32_t sk = smem_u32(smem + Smem::kK + st * kQKV);
        const uint32_t sqt = sq + tile * kQKV;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + tile * BT, make_smem_desc(sqt + off, 16, 1024), make_smem_desc(sk + off, 16, 1024),
                       idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[tile]);
      };
      auto pv = [&](int tile, int it) {
        const int st = it % kStages;
        const uint32_t sv = smem_u32(smem + Smem::kV + st * kQKV);
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk) {
          // 16 keys of P = 8 TMEM columns; 16 keys of V = two 8-row groups = 2048 B
          umma_bf16_ts(tmem_base + 2 * BT + tile * D, tmem_base + tile * BT + kk * 8,
                       make_smem_desc(sv + kk * 2048, kChunkBytes, 1024), idesc_pv, (it > 0 || kk > 0) ? 1u : 0u);
        }
      };
      auto wait_k = [&](int it) { return mbar_wait(&k_full[it % kStages], (it / kStages) & 1, abort_flag, p.status, 1301, it); };
      auto wait_v = [&](int it) { return mbar_wait(&v_full[it % kStages], (it / kStages) & 1, abort_flag, p.status, 1302, it); };

      if (ok) ok = wait_k(0);
      if (ok) {
        tc_fence_after();
        qk(0, 0);
        qk(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int it = 0; it < nB && ok; ++it) {
        const int st = it % kStages;
        ok = wait_v(it);
        if (!ok) break;
        if (it < nA) {
          ok = mbar_wait(&p_full[0], it & 1, abort_flag, p.status, 1303, it);
          if (!ok) break;
          tc_fence_after();
          pv(0, it);
          if (it == nA - 1) umma_commit(&o_done[0]);
        }
        const bool more = it + 1 < nB;
        if (more) {
          ok = wait_k(it + 1);
          if (!ok) break;
          tc_fence_after();
          if (it + 1 < nA) qk(0, it + 1);
        }
        ok = mbar_wait(&p_full[1], it & 1, abort_flag, p.status, 1304, it);
        if (!ok) break;
        tc_fence_after();
        pv(1, it);
        umma_commit(&v_empty[st]);
        if (it == nB - 1) umma_commit(&o_done[1]);
        if (more) {
          qk(1, it + 1);
          umma_commit(&k_empty[(it + 1) % kStages]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + correction + epilogue
    const int tile = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int qi = q0 + tile * BT + r;
    const int jdiag = tile == 0 ? jdiagA : jdiagB;
    const int nT = tile == 0 ? nA : nB;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tS = tmem_base + tile * BT + lane_addr;
    const uint32_t tO = tmem_base + 2 * BT + tile * D + lane_addr;
    const float scale_log2 = p.scale * kLog2e;
    const int my_seg = kSeg ? p.q_seg[b * p.S + qi] : 0;
    const int* kseg_row = kSeg ? p.k_seg + b * p.Sk : nullptr;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;

    for (int it = 0; it < nT && ok; ++it) {
      const int j = jlo + it;
      const int k0 = j * BT;
      ok = mbar_wait(&s_full[tile], it & 1, abort_flag, p.status, 1400 + tile, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = (j == jdiag) || kSeg || (p.window > 0 && k0 <= q0 + tile * BT + BT - 1 - p.window);

      // ---- pass 1: row maximum (raw logits; the scale is positive and the soft-cap monotonic)
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BT; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tS + c, v);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const int kj = k0 + c + t;
            bool valid = !causal || kj <= qi;
            if (p.window > 0) valid = valid && (qi - kj < p.window);
            if (kSeg) valid = valid && (kseg_row[kj] == my_seg);
            if (!valid) v[t] = __float_as_uint(-INFINITY);
          }
        }
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(v[t]));
          mx1 = fmaxf(mx1, __uint_as_float(v[t + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(v[t + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(v[t + 3]));
        }
      }
      const float m_raw = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_blk = (m_raw == -INFINITY) ? -INFINITY : to_log2<kCap>(m_raw, scale_log2, p.scale, p.soft_cap);

      // ---- lazy rescale of O (S_T ready implies the previous P_T V has retired).  The decision is per row, but the
      // TMEM load/store are warp-collective, so the whole warp takes the branch as soon as one row needs it and rows
      // that do not need it scale by exactly 1.
      {
        const bool want = (m_blk > m_used + kRescaleThreshold) || (m_used == -INFINITY && m_blk > -INFINITY);
        const float m_new = want ? fmaxf(m_used, m_blk) : m_used;
        const bool scale_row = want && it > 0 && m_used > -INFINITY;
        if (__any_sync(0xffffffffu, scale_row)) {
          const float alpha = scale_row ? exp2f(m_used - m_new) : 1.f;
          l_sum *= alpha;
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tO + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
            tmem_st_32x32(tO + c, v);
          }
        }
        m_used = m_new;
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;

      // ---- pass 2: P = exp2(s - m) -> bf16 pairs written over the first 64 columns of S
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 1
      for (int c = 0; c < BT; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tS + c, v);
        tmem_ld_wait();
        float e[32];
        if (need_mask) {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const int kj = k0 + c + t;
            bool valid = !causal || kj <= qi;
            if (p.window > 0) valid = valid && (qi - kj < p.window);
            if (kSeg) valid = valid && (kseg_row[kj] == my_seg);
            const float x = kCap ? to_log2<kCap>(__uint_as_float(v[t]), scale_log2, p.scale, p.soft_cap) + neg_m
                                 : fmaf(__uint_as_float(v[t]), scale_log2, neg_m);
            e[t] = valid ? exp2f(x) : 0.f;
          }
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const float x = kCap ? to_log2<kCap>(__uint_as_float(v[t]), scale_log2, p.scale, p.soft_cap) + neg_m
                                 : fmaf(__uint_as_float(v[t]), scale_log2, neg_m);
            e[t] = exp2f(x);
          }
        }
        uint32_t pk[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) pk[t] = pack_bf16x2(e[2 * t], e[2 * t + 1]);
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          s0 += e[t];
          s1 += e[t + 1];
          s2 += e[t + 2];
          s3 += e[t + 3];
        }
        tmem_st_32x16(tS + (c >> 1), pk);
      }
      l_sum += (s0 + s1) + (s2 + s3);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[tile]);
    }

    if (ok) {
      ok = mbar_wait(&o_done[tile], 0, abort_flag, p.status, 1410 + tile, nT);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      float o_scale = 1.f;
      if (p.sink != nullptr) {
        // The sink is one more column of the softmax whose value row is zero: it enters the denominator (and the saved
        // log-sum-exp) and nothing else.  If it raises the reference maximum from m to m', the accumulated output and sum
        // (both relative to m) shrink by a = 2^(m - m').
        const float s2 = p.sink[h] * kLog2e;
        const float m_new = fmaxf(m_used, s2);
        o_scale = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
        l_sum = l_sum * o_scale + exp2f(s2 - m_new);
        m_used = m_new;
      }
      const float inv = l_sum > 0.f ? o_scale / l_sum : 0.f;
      __nv_bfloat16* orow = p.O + (static_cast<size_t>(b) * p.S + qi) * (static_cast<size_t>(p.Hq) * D) + static_cast<size_t>(h) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tO + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]) * inv, __uint_as_float(v[q4 * 8 + 1]) * inv);
          w.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]) * inv, __uint_as_float(v[q4 * 8 + 3]) * inv);
          w.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]) * inv, __uint_as_float(v[q4 * 8 + 5]) * inv);
          w.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]) * inv, __uint_as_float(v[q4 * 8 + 7]) * inv);
          reinterpret_cast<uint4*>(orow + c)[q4] = w;
        }
      }
      p.lse2[(static_cast<size_t>(b) * p.Hq + h) * p.S + qi] = (l_sum > 0.f) ? m_used + log2f(l_sum) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

template <int HD, bool kSeg, bool kCap>
int launch(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const Params& p, cudaStream_t st) {
  using Smem = SmemT<HD>;
  auto kern = flash_fwd2_kernel<HD, kSeg, kCap>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  dim3 grid(p.S / (2 * BT), p.B * p.Hq);
  kern<<<grid, kThreads, Smem::kTotal, st>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace fa2
}  // namespace lvb

namespace lvb {
namespace fa2 {
template <int HD>
int launch_hd(const void* q, const void* k, const void* v, const Params& p, cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t rows = static_cast<uint64_t>(p.B) * p.S;
  int rc = make_tmap_2d_bf16(&tmQ, q, rows, static_cast<uint64_t>(p.Hq) * HD, static_cast<uint64_t>(p.Hq) * HD, BT, 64);
  if (rc != kErrOk) return rc;
  const uint64_t rows_k = static_cast<uint64_t>(p.B) * p.Sk;
  rc = make_tmap_2d_bf16(&tmK, k, rows_k, static_cast<uint64_t>(p.Hkv) * HD, static_cast<uint64_t>(p.Hkv) * HD, BT, 64);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_bf16(&tmV, v, rows_k, static_cast<uint64_t>(p.Hkv) * HD, static_cast<uint64_t>(p.Hkv) * HD, BT, 64);
  if (rc != kErrOk) return rc;
  const bool seg = p.q_seg != nullptr;
  const bool cap = p.soft_cap > 0.f;
  if (seg && cap) return launch<HD, true, true>(tmQ, tmK, tmV, p, st);
  if (seg) return launch<HD, true, false>(tmQ, tmK, tmV, p, st);
  if (cap) return launch<HD, false, true>(tmQ, tmK, tmV, p, st);
  return launch<HD, false, false>(tmQ, tmK, tmV, p, st);
}
}  // namespace fa2
}  // namespace lvb

// Same contract as lvb_flash_attn_fwd_hd (head_dim 64 or 128, causal or not, optional sink logits [Hq]), but S must be a
// multiple of 256: two query tiles per CTA.  Sk: keys per sequence, a multiple of 128 (k / v are [B, Sk, Hkv, D], k_seg [B, Sk]);
// Sk must equal S when causal.
extern "C" int lvb_flash_attn_fwd2_hd(const void* q, const void* k, const void* v, void* o, float* lse2, const int* q_seg,
                                      const int* k_seg, const int* kblock_lo, const float* sink, int B, int S, int Sk, int Hq, int Hkv,
                                      int head_dim, int causal, float scale, float soft_cap, int window, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::fa2;
  if (B <= 0 || S <= 0 || (S % (2 * BT)) != 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv) != 0) return kErrBadArg;
  if (!causal && (window != 0 || kblock_lo != nullptr)) return kErrBadArg;
  if (Sk <= 0 || (Sk % BT) != 0 || (causal && Sk != S)) return kErrBadArg;
  Params p;
  p.O = reinterpret_cast<__nv_bfloat16*>(o);
  p.lse2 = lse2;
  p.q_seg = q_seg;
  p.k_seg = k_seg;
  p.kblock_lo = kblock_lo;
  p.sink = sink;
  p.B = B; p.S = S; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.soft_cap = soft_cap; p.window = window;
  p.causal = causal ? 1 : 0;
  p.status = status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (head_dim == 128) return launch_hd<128>(q, k, v, p, st);
  if (head_dim == 64) return launch_hd<64>(q, k, v, p, st);
  return kErrBadArg;
}

// Causal, head_dim 128 (the original entry point).
extern "C" int lvb_flash_attn_fwd2(const void* q, const void* k, const void* v, void* o, float* lse2, const int* q_seg,
                                   const int* k_seg, const int* kblock_lo, int B, int S, int Hq, int Hkv, float scale, float soft_cap,
                                   int window, int* status, void* stream) {
  return lvb_flash_attn_fwd2_hd(q, k, v, o, lse2, q_seg, k_seg, kblock_lo, nullptr, B, S, S, Hq, Hkv, 128, 1, scale, soft_cap, window, status, stream);
}
