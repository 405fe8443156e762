// Causal flash attention forward for sm_100a (head_dim 128, bf16), tcgen05 + TMEM + TMA.
//
// One CTA owns 128 query rows of one (batch, query head) and walks the key blocks of 128 that its
// mask can reach (causal diagonal, sliding-window lower edge).  Per key block:
//   MMA warp     S = Q K^T            tcgen05.mma, fp32 in TMEM (two S buffers so S_{j+1} overlaps softmax_j)
//   softmax x4   one query row per thread (row = TMEM lane, so no shuffles): row max, p = exp2(s - m), row sum,
//                P written as bf16 into shared memory in the 128B-swizzled K-major layout the MMA reads
//   MMA warp     O += P V             V is read as an MN-major operand straight from its [key, d] tile
// The running max is allowed to go stale by up to 2^8 before O (kept in TMEM) is rescaled, so the
// TMEM read-modify-write of O happens only when a row's maximum really moves.
// Outputs: O (bf16) and LSE in the log2 domain, lse2 = m + log2(sum), for the backward pass.
//
// Mask semantics are those of the reference's AttentionMask (src/levanter/layers/attention.py:745-846):
// causal j <= i, sliding window 0 <= i - j < window, segment ids equal; optional tanh soft-cap on the
// scaled logits (:329-378).  GQA: query head h reads KV head h / (Hq / Hkv).
#include "common.cuh"

namespace lvb {
namespace fa {

constexpr int BM = 128;   // query rows per CTA
constexpr int BN = 128;   // keys per block
constexpr int kThreads = 192;  // warp0 TMA, warp1 MMA, warps2-5 softmax
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KB: two 64-column chunks of [128 rows x 128 B]
constexpr int kChunkBytes = 128 * 64 * 2;  // 16 KB
constexpr int kKvStages = 2;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdParams {
  __nv_bfloat16* O;     // [B, S, Hq, D]
  float* lse2;          // [B, Hq, S]
  const int* q_seg;     // [B, S] or null
  const int* k_seg;     // [B, S] or null
  const int* kblock_lo; // optional [B, S / 128]: first block of 128 keys that a query of this 128-row block can attend to
  const float* sink;    // optional [Hq]: a learned logit per head that takes part in the softmax denominator only
  int B, S, Hq, Hkv;    // S: query positions per sequence
  int Sk;               // key positions per sequence (= S unless the mask has no causal part)
  float scale;          // softmax scale (1/sqrt(D) by default)
  float soft_cap;       // 0 = off
  int window;           // 0 = off
  int causal;           // 0: every key is visible (subject to segment ids); window must be 0 then
  int* status;
};

template <int HD>
struct SmemT {
  // tiles first (1024-byte aligned), then barriers.  Q, K and V tiles are [128 rows, HD] as HD / 64 chunks of 64 columns.
  static constexpr int kQKV = 128 * HD * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kQKV;
  static constexpr int kV = kK + kKvStages * kQKV;
  static constexpr int kP = kV + kKvStages * kQKV;
  static constexpr int kKseg = kP + kTileBytes;           // per softmax warp: 2 x 128 ints
  static constexpr int kBars = kKseg + 4 * 2 * BN * 4;
  static constexpr int kNumBars = 1 + 4 * kKvStages + 2 + 2 + 1 + 1;
  static constexpr int kTotal = kBars + kNumBars * 8 + 16 + 1024;
};

// byte offset of element (row r, column c) of a [128 x 128] bf16 tile stored as two 64-column
// chunks with the 128-byte swizzle (16-byte unit index XOR row % 8)
__device__ __forceinline__ uint32_t swz_off(int r, int c) {
  const int chunk = c >> 6;
  const int unit = ((c & 63) >> 3) ^ (r & 7);
  return chunk * kChunkBytes + r * 128 + unit * 16 + (c & 7) * 2;
}

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  using Smem = SmemT<HD>;
  constexpr int D = HD;
  constexpr int kQKV = Smem::kQKV;
  const bool causal = p.causal != 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + kKvStages;
  uint64_t* v_full = k_empty + kKvStages;
  uint64_t* v_empty = v_full + kKvStages;
  uint64_t* s_full = v_empty + kKvStages;   // [2]
  uint64_t* s_empty = s_full + 2;           // [2]
  uint64_t* p_full = s_empty + 2;
  uint64_t* pv_done = p_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* kseg_s = reinterpret_cast<int*>(smem + Smem::kKseg);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nqb = p.S / BM;
  const int qb = nqb - 1 - static_cast<int>(blockIdx.x);  // heaviest (last) query blocks first
  const int bh = blockIdx.y;
  const int b = bh / p.Hq;
  const int h = bh % p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = qb * BM;
  // key blocks [jlo, jhi]
  const int jhi = causal ? qb : p.Sk / BN - 1;
  int jlo = 0;
  if (p.window > 0) {
    const int first_key = q0 - p.window + 1;
    jlo = first_key > 0 ? first_key / BN : 0;
  }
  if (p.kblock_lo != nullptr) {
    // packed sequences (segment ids ascending): key blocks before the first query's sequence hold nothing these rows can see
    const int lo = p.kblock_lo[b * nqb + qb];
    jlo = max(jlo, min(lo, jhi));
  }
  const int nblocks = jhi - jlo + 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
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
  const uint32_t tmem_S0 = tmem_base;        // columns [0,128) and [128,256)
  const uint32_t tmem_O = tmem_base + 256;   // columns [256,384)

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const int row_q = b * p.S + q0;
      mbar_expect_tx(q_full, kQKV);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_2d(smem + Smem::kQ + c * kChunkBytes, &tmQ, q_full, h * D + 64 * c, row_q);
      bool ok = true;
      for (int it = 0; it < nblocks && ok; ++it) {
        const int j = jlo + it;
        const int st = it % kKvStages;
        const uint32_t ph = (it / kKvStages) & 1;
        const int row_k = b * p.Sk + j * BN;
        ok = mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, 600, it);
        if (!ok) break;
        uint8_t* ks = smem + Smem::kK + st * kQKV;
        mbar_expect_tx(&k_full[st], kQKV);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(ks + c * kChunkBytes, &tmK, &k_full[st], hkv * D + 64 * c, row_k);
        ok = mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, 601, it);
        if (!ok) break;
        uint8_t* vs = smem + Smem::kV + st * kQKV;
        mbar_expect_tx(&v_full[st], kQKV);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(vs + c * kChunkBytes, &tmV, &v_full[st], hkv * D + 64 * c, row_k);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BM, BN, false, false);  // A=Q K-major, B=K K-major
      constexpr uint32_t idesc_pv = make_idesc_bf16(BM, D, false, true);    // A=P K-major, B=V MN-major
      const uint32_t sq = smem_u32(smem + Smem::kQ);
      const uint32_t sp = smem_u32(smem + Smem::kP);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 700, 0);

      auto issue_qk = [&](int it) -> bool {
        const int st = it % kKvStages;
        const uint32_t ph = (it / kKvStages) & 1;
        const int sb = it & 1;
        const uint32_t sph = (it >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, 701, it)) return false;
        if (!mbar_wait(&s_empty[sb], sph ^ 1, abort_flag, p.status, 702, it)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + Smem::kK + st * kQKV);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
          umma_bf16_ss(tmem_S0 + sb * BN, make_smem_desc(sq + off, 16, 1024), make_smem_desc(sk + off, 16, 1024),
                       idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        umma_commit(&k_empty[st]);
        return true;
      };

      if (ok) ok = issue_qk(0);
      for (int it = 0; it < nblocks && ok; ++it) {
        if (it + 1 < nblocks) {
          ok = issue_qk(it + 1);
          if (!ok) break;
        }
        const int st = it % kKvStages;
        const uint32_t ph = (it / kKvStages) & 1;
        ok = mbar_wait(&v_full[st], ph, abort_flag, p.status, 703, it);
        if (!ok) break;
        ok = mbar_wait(p_full, it & 1, abort_flag, p.status, 704, it);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + Smem::kV + st * kQKV);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // A = P: K-major over keys: chunk kk/4, 32 B per 16 keys inside the swizzle row
          const uint32_t aoff = (kk >> 2) * kChunkBytes + (kk & 3) * 32;
          // B = V: MN-major (d contiguous): 64-d chunks are kChunkBytes apart (LBO), 8-key groups 1024 B
          // apart (SBO); 16 keys = 2 groups = 2048 B per step
          const uint32_t boff = kk * 2048;
          umma_bf16_ss(tmem_O, make_smem_desc(sp + aoff, 16, 1024), make_smem_desc(sv + boff, kChunkBytes, 1024),
                       idesc_pv, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(pv_done);
        umma_commit(&v_empty[st]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;        // row inside the tile == TMEM lane
    const int qi = q0 + r;                 // absolute query position
    int* kseg_w = kseg_s + quad * (2 * BN);  // this warp's private copy: no cross-warp barrier is needed
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const bool use_seg = p.q_seg != nullptr;
    const int my_seg = use_seg ? p.q_seg[b * p.S + qi] : 0;
    float m_used = -INFINITY;  // log2-domain max the stored exponentials refer to
    float l_sum = 0.f;
    bool ok = true;
    uint8_t* sp = smem + Smem::kP;

    for (int it = 0; it < nblocks && ok; ++it) {
      const int j = jlo + it;
      const int k0 = j * BN;
      const int sb = it & 1;
      const uint32_t sph = (it >> 1) & 1;
      if (use_seg) {
        // stage this block's key segment ids (double-buffered by block parity)
#pragma unroll
        for (int t = 0; t < BN / 32; ++t) kseg_w[sb * BN + t * 32 + lane] = p.k_seg[b * p.Sk + k0 + t * 32 + lane];
        __syncwarp();
      }
      ok = mbar_wait(&s_full[sb], sph, abort_flag, p.status, 800, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = (causal && j == qb) || use_seg || (p.window > 0 && k0 <= q0 + BM - 1 - p.window);
      const uint32_t s_addr = tmem_S0 + lane_addr + sb * BN;

      // pass 1: row maximum of the scaled (and masked) logits, log2 domain
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          float s = __uint_as_float(v[t]);
          if (p.soft_cap > 0.f) s = p.soft_cap * tanhf(s * p.scale / p.soft_cap) * 1.4426950408889634f;
          else s *= scale_log2;
          if (need_mask) {
            const int kj = k0 + c + t;
            bool valid = !causal || kj <= qi;
            if (p.window > 0) valid = valid && (qi - kj < p.window);
            if (use_seg) valid = valid && (kseg_w[sb * BN + c + t] == my_seg);
            if (!valid) s = -INFINITY;
          }
          m_blk = fmaxf(m_blk, s);
        }
      }
      // the P buffer and O are free once the previous P V product has retired
      if (it > 0) {
        ok = mbar_wait(pv_done, (it - 1) & 1, abort_flag, p.status, 801, it);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
      // The rescale decision is per row, but the TMEM load/store are warp-collective: the whole warp takes the branch as
      // soon as one row needs it, and rows that do not need it scale by exactly 1.
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
            tmem_ld_32x32(tmem_O + lane_addr + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
            tmem_st_32x32(tmem_O + lane_addr + c, v);
          }
          tmem_st_wait();
        }
        m_used = m_new;
      }
      const float m_ref = (m_used == -INFINITY) ? 0.f : m_used;

      // pass 2: exponentials -> bf16 P in shared memory, row sum
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c, v);
        tmem_ld_wait();
        float e[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          float s = __uint_as_float(v[t]);
          if (p.soft_cap > 0.f) s = p.soft_cap * tanhf(s * p.scale / p.soft_cap) * 1.4426950408889634f;
          else s *= scale_log2;
          if (need_mask) {
            const int kj = k0 + c + t;
            bool valid = !causal || kj <= qi;
            if (p.window > 0) valid = valid && (qi - kj < p.window);
            if (use_seg) valid = valid && (kseg_w[sb * BN + c + t] == my_seg);
            if (!valid) s = -INFINITY;
          }
          e[t] = exp2f(s - m_ref);
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 w;
          w.x = pack_bf16x2(e[q4 * 8 + 0], e[q4 * 8 + 1]);
          w.y = pack_bf16x2(e[q4 * 8 + 2], e[q4 * 8 + 3]);
          w.z = pack_bf16x2(e[q4 * 8 + 4], e[q4 * 8 + 5]);
          w.w = pack_bf16x2(e[q4 * 8 + 6], e[q4 * 8 + 7]);
          *reinterpret_cast<uint4*>(sp + swz_off(r, c + q4 * 8)) = w;
          // the row sum uses the values the MMA will actually see (bf16-rounded)
          const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            float2 f = __bfloat1622float2(hh[t]);
            l_sum += f.x + f.y;
          }
        }
      }
      // S buffer consumed; P visible to the async proxy
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[sb]);
        mbar_arrive(p_full);
      }
    }

    // epilogue: O / l -> bf16, LSE
    if (ok) {
      ok = mbar_wait(pv_done, (nblocks - 1) & 1, abort_flag, p.status, 802, nblocks);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      float o_scale = 1.f;
      if (p.sink != nullptr) {  // one more softmax column with a zero value row: see flash_attn_fwd2.cu
        const float s2 = p.sink[h] * 1.4426950408889634f;
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
        tmem_ld_32x32(tmem_O + lane_addr + c, v);
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

}  // namespace fa
}  // namespace lvb

namespace lvb {
namespace fa {
template <int HD>
int launch_fwd(const void* q, const void* k, const void* v, FwdParams p, cudaStream_t stream) {
  using Smem = SmemT<HD>;
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t rows = static_cast<uint64_t>(p.B) * p.S;
  int rc = make_tmap_2d_bf16(&tmQ, q, rows, static_cast<uint64_t>(p.Hq) * HD, static_cast<uint64_t>(p.Hq) * HD, BM, 64);
  if (rc != kErrOk) return rc;
  const uint64_t rows_k = static_cast<uint64_t>(p.B) * p.Sk;
  rc = make_tmap_2d_bf16(&tmK, k, rows_k, static_cast<uint64_t>(p.Hkv) * HD, static_cast<uint64_t>(p.Hkv) * HD, BN, 64);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_bf16(&tmV, v, rows_k, static_cast<uint64_t>(p.Hkv) * HD, static_cast<uint64_t>(p.Hkv) * HD, BN, 64);
  if (rc != kErrOk) return rc;
  auto kern = flash_fwd_kernel<HD>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  dim3 grid(p.S / BM, p.B * p.Hq);
  kern<<<grid, kThreads, Smem::kTotal, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
}  // namespace fa
}  // namespace lvb

// q: [B, S, Hq, D], k/v: [B, S, Hkv, D] (bf16, contiguous), o: [B, S, Hq, D] bf16, lse2: [B, Hq, S] fp32; D = head_dim is 64 or 128.
// S must be a multiple of 128.  q_seg/k_seg: int32 [B, S] or null.  window: 0 = none.  soft_cap: 0 = none.  sink: fp32 [Hq] or
// null (a learned logit per head added to the softmax denominator).  Sk: keys per sequence, a multiple of 128 (k / v are
// [B, Sk, Hkv, D], k_seg [B, Sk]); equal to S when causal.  causal: 0 lets
// every query see every key of its segment (encoders); window must be 0 and kblock_lo null then.
extern "C" int lvb_flash_attn_fwd_hd(const void* q, const void* k, const void* v, void* o, float* lse2, const int* q_seg,
                                     const int* k_seg, const int* kblock_lo, const float* sink, int B, int S, int Sk, int Hq, int Hkv,
                                     int head_dim, int causal, float scale, float soft_cap, int window, int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::fa;
  if (B <= 0 || S <= 0 || (S % BM) != 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv) != 0) return kErrBadArg;
  if (!causal && (window != 0 || kblock_lo != nullptr)) return kErrBadArg;
  if (Sk <= 0 || (Sk % BN) != 0 || (causal && Sk != S)) return kErrBadArg;
  FwdParams p;
  p.O = reinterpret_cast<__nv_bfloat16*>(o);
  p.lse2 = lse2;
  p.q_seg = q_seg;
  p.k_seg = k_seg;
  p.kblock_lo = kblock_lo;
  p.sink = sink;
  p.B = B; p.S = S; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale;
  p.soft_cap = soft_cap;
  p.window = window;
  p.causal = causal ? 1 : 0;
  p.status = status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (head_dim == 128) return launch_fwd<128>(q, k, v, p, st);
  if (head_dim == 64) return launch_fwd<64>(q, k, v, p, st);
  return kErrBadArg;
}

// Causal, head_dim 128 (the original entry point).
extern "C" int lvb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse2, const int* q_seg,
                                  const int* k_seg, const int* kblock_lo, int B, int S, int Hq, int Hkv, float scale, float soft_cap,
                                  int window, int* status, void* stream) {
  return lvb_flash_attn_fwd_hd(q, k, v, o, lse2, q_seg, k_seg, kblock_lo, nullptr, B, S, S, Hq, Hkv, 128, 1, scale, soft_cap, window, status, stream);
}
