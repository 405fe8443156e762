// Paged-KV kernels of the inference engine.
//
//  * kv_page_write: scatter the K/V rows of the packed tokens of one forward pass into their (page, slot) destinations.
//  * paged_attention: causal attention of packed query tokens over the pages of their sequences (decode steps and chunked
//    prefill), src/levanter/layers/attention.py:1710-1991 in the reference.
//
// Cache layout: kv_pages[page, slot, 2 * kv_heads, D] bf16 with K at even and V at odd head index, so one token's K and V
// rows of a kv head are adjacent 2*D-element runs.
//
// paged_attention is bandwidth bound (every step re-reads the context once), so the work is cut for parallelism, not for
// tensor cores: one CTA per (query token, kv head, partition of 256 keys).  A CTA scores its keys against the G query heads
// that share the kv head (one key per thread, 16-byte loads), soft-maxes within the partition in shared memory,
// accumulates P.V with eight output dimensions per thread, and writes an un-normalised partial (o, max, sum).  A second small
// kernel merges the partitions of each (token, head).  Nothing here synchronises with the host: sequence boundaries,
// lengths and the number of live sequences are read from device arrays, padding tokens produce zeros.
#include "common.cuh"
#include <cstdlib>
#include <string>

namespace lvb {
namespace paged {

constexpr int kPart = 256;     // keys per partition
constexpr int kThreads = 128;  // 4 warps
constexpr int kMaxG = 16;      // query heads per kv head

__global__ void kv_page_write_kernel(__nv_bfloat16* __restrict__ kv_pages, const __nv_bfloat16* __restrict__ k,
                                     const __nv_bfloat16* __restrict__ v, const int* __restrict__ dests, int kv_heads, int D,
                                     long long total_slots) {
  const int t = blockIdx.x;
  const long long dest = dests[t];
  if (dest < 0 || dest >= total_slots) return;  // padding token
  const int row = kv_heads * D;                 // elements of K (or V) per token
  const int vec = row / 8;                      // uint4 = 8 bf16
  const uint4* ks = reinterpret_cast<const uint4*>(k + static_cast<long long>(t) * row);
  const uint4* vs = reinterpret_cast<const uint4*>(v + static_cast<long long>(t) * row);
  uint4* out = reinterpret_cast<uint4*>(kv_pages + dest * 2 * row);
  const int per_head = D / 8;
  for (int i = threadIdx.x; i < vec; i += blockDim.x) {
    const int h = i / per_head, j = i % per_head;
    out[(2 * h) * per_head + j] = ks[i];
    out[(2 * h + 1) * per_head + j] = vs[i];
  }
}

// kN consecutive bf16 (kN = 2, 4 or 8) with one load of 4, 8 or 16 bytes.
template <int kN>
__device__ __forceinline__ void load_row(const __nv_bfloat16* src, float* dst) {
  if constexpr (kN == 2) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(src);
    dst[0] = __low2float(a); dst[1] = __high2float(a);
  } else if constexpr (kN == 4) {
    const uint2 w = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w.x), b = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
    dst[0] = __low2float(a); dst[1] = __high2float(a); dst[2] = __low2float(b); dst[3] = __high2float(b);
  } else {
    const uint4 w = *reinterpret_cast<const uint4*>(src);
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u[i]);
      dst[2 * i] = __low2float(a); dst[2 * i + 1] = __high2float(a);
    }
  }
}

struct Params {
  const __nv_bfloat16* q;         // [T, H, D]
  const __nv_bfloat16* kv_pages;  // [P, ps, 2 * KV, D]
  const int* kv_lens;             // [S]
  const int* page_indices;        // [S, pages_per_seq]
  const int* cu_q_lens;           // [S + 1]
  const int* num_seqs;            // [1]
  __nv_bfloat16* out;             // [T, H, D]
  float* part_o;                  // [T, H, parts, D]
  float* part_ml;                 // [T, H, parts, 2]
  int T, H, KV, S, pages_per_seq, page_size, num_pages, parts;
  float scale, soft_cap;
};

// Which sequence owns packed token t, and how many keys it may attend to.  Returns false for padding tokens.
__device__ __forceinline__ bool locate(const Params& p, int t, int& seq, int& ctx) {
  int n = p.num_seqs[0];
  n = n < p.S ? n : p.S;
  if (n <= 0 || t >= p.cu_q_lens[n]) return false;
  int lo = 0, hi = n;  // first seq with cu[seq + 1] > t
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (p.cu_q_lens[mid + 1] > t) hi = mid; else lo = mid + 1;
  }
  seq = lo;
  const int q0 = p.cu_q_lens[seq], q1 = p.cu_q_lens[seq + 1];
  const int kl = p.kv_lens[seq];
  if (kl <= 0 || kl > p.pages_per_seq * p.page_size) return false;
  ctx = kl - (q1 - q0) + (t - q0) + 1;  // absolute position of the token + 1
  return ctx > 0;
}

// Dot products of one key row (D bf16, read with 16-byte loads) with the G query rows in shared memory.
template <int D>
__device__ __forceinline__ void score_key(const __nv_bfloat16* __restrict__ krow, const float* __restrict__ s_q, int G, float* acc) {
#pragma unroll
  for (int g = 0; g < kMaxG; ++g) acc[g] = 0.f;
#pragma unroll 4
  for (int c = 0; c < D / 8; ++c) {
    float kf[8];
    load_row<8>(krow + c * 8, kf);
#pragma unroll
    for (int g = 0; g < kMaxG; ++g) {
      if (g < G) {
        const float4 qa = *reinterpret_cast<const float4*>(s_q + g * D + c * 8);
        const float4 qb = *reinterpret_cast<const float4*>(s_q + g * D + c * 8 + 4);
        acc[g] = fmaf(kf[0], qa.x, acc[g]); acc[g] = fmaf(kf[1], qa.y, acc[g]);
        acc[g] = fmaf(kf[2], qa.z, acc[g]); acc[g] = fmaf(kf[3], qa.w, acc[g]);
        acc[g] = fmaf(kf[4], qb.x, acc[g]); acc[g] = fmaf(kf[5], qb.y, acc[g]);
        acc[g] = fmaf(kf[6], qb.z, acc[g]); acc[g] = fmaf(kf[7], qb.w, acc[g]);
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads) paged_attention_kernel(Params p) {
  constexpr int kDimGroups = D / 8;                   // 16-byte column groups of a row
  constexpr int kKeyGroups = kThreads / kDimGroups;   // rows read side by side in the P.V phase
  constexpr int kGChunk = 4;                          // heads accumulated per pass over V
  const int t = blockIdx.x, kvh = blockIdx.y, part = blockIdx.z;
  const int G = p.H / p.KV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ __align__(16) float s_q[kMaxG * D];
  __shared__ __align__(16) float s_red[(kKeyGroups / 2) * kGChunk * D];  // 2048 floats for every D
  __shared__ float s_p[kMaxG * kPart];
  __shared__ float s_m[kMaxG], s_l[kMaxG];
  __shared__ int s_rows[kPart];  // flat slot (page * page_size + offset) of each key of the partition

  int seq = 0, ctx = 0;
  const bool live = locate(p, t, seq, ctx);
  const int k0 = part * kPart;
  if (!live || k0 >= ctx) {
    if (part == 0 && !live) {  // padding token: defined output
      for (int i = threadIdx.x; i < G * D; i += kThreads)
        p.out[(static_cast<long long>(t) * p.H + kvh * G) * D + i] = __float2bfloat16(0.f);
    }
    return;
  }
  const int nk = min(kPart, ctx - k0);
  for (int i = threadIdx.x; i < G * D; i += kThreads)
    s_q[i] = __bfloat162float(p.q[(static_cast<long long>(t) * p.H + kvh * G) * D + i]) * p.scale;
  for (int i = threadIdx.x; i < nk; i += kThreads) {
    const int key = k0 + i;
    const int page = p.page_indices[seq * p.pages_per_seq + key / p.page_size];
    s_rows[i] = (page >= 0 && page < p.num_pages) ? page * p.page_size + key % p.page_size : -1;
  }
  __syncthreads();

  const long long tok_stride = 2LL * p.KV * D;  // elements per cache slot
  // ---- scores: one key per thread, the whole row in 16-byte loads (rows of neighbouring threads are tok_stride apart, so
  // every 32-byte sector is fetched once and its second half comes from L1)
  for (int i = threadIdx.x; i < nk; i += kThreads) {
    const int r = s_rows[i];
    float acc[kMaxG];
    if (r >= 0) {
      score_key<D>(p.kv_pages + r * tok_stride + (2LL * kvh) * D, s_q, G, acc);
    }
#pragma unroll
    for (int g = 0; g < kMaxG; ++g) {
      if (g < G) {
        float v = (r >= 0) ? acc[g] : -INFINITY;
        if (p.soft_cap > 0.f && r >= 0) v = p.soft_cap * tanhf(v / p.soft_cap);
        s_p[g * kPart + i] = v;
      }
    }
  }
  __syncthreads();
  // ---- softmax within the partition: warp w handles heads w, w + 4, ...
  for (int g = warp; g < G; g += kThreads / 32) {
    float m = -INFINITY;
    for (int i = lane; i < nk; i += 32) m = fmaxf(m, s_p[g * kPart + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.f;
    for (int i = lane; i < nk; i += 32) {
      const float e = (m == -INFINITY) ? 0.f : __expf(s_p[g * kPart + i] - m);
      s_p[g * kPart + i] = e;
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) { s_m[g] = m; s_l[g] = l; }
  }
  __syncthreads();
  // ---- P.V: thread (key group kg, dim group dg) walks keys kg, kg + kKeyGroups, ... and owns 8 output dimensions, so a
  // warp reads whole 256-byte rows; heads are taken kGChunk at a time to bound registers (V re-reads hit L1/L2).
  const int dg = threadIdx.x % kDimGroups, kg = threadIdx.x / kDimGroups;
  for (int g0 = 0; g0 < G; g0 += kGChunk) {
    float o[kGChunk][8];
#pragma unroll
    for (int g = 0; g < kGChunk; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) o[g][e] = 0.f;
    for (int i = kg; i < nk; i += kKeyGroups) {
      const int r = s_rows[i];
      if (r < 0) continue;
      float vf[8];
      load_row<8>(p.kv_pages + r * tok_stride + (2LL * kvh + 1) * D + dg * 8, vf);
#pragma unroll
      for (int g = 0; g < kGChunk; ++g) {
        if (g0 + g < G) {
          const float w = s_p[(g0 + g) * kPart + i];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[g][e] = fmaf(w, vf[e], o[g][e]);
        }
      }
    }
    // tree-reduce the key groups through shared memory
    for (int half = kKeyGroups / 2; half >= 1; half >>= 1) {
      if (kg >= half && kg < 2 * half) {
#pragma unroll
        for (int g = 0; g < kGChunk; ++g)
#pragma unroll
          for (int e = 0; e < 8; ++e) s_red[((kg - half) * kGChunk + g) * D + dg * 8 + e] = o[g][e];
      }
      __syncthreads();
      if (kg < half) {
#pragma unroll
        for (int g = 0; g < kGChunk; ++g)
#pragma unroll
          for (int e = 0; e < 8; ++e) o[g][e] += s_red[(kg * kGChunk + g) * D + dg * 8 + e];
      }
      __syncthreads();
    }
    if (kg == 0) {
#pragma unroll
      for (int g = 0; g < kGChunk; ++g) {
        if (g0 + g >= G) continue;
        const long long hrow = static_cast<long long>(t) * p.H + kvh * G + g0 + g;
        if (p.parts == 1) {
          const float l = s_l[g0 + g];
          const float inv = l > 0.f ? 1.f / l : 0.f;
          uint4 w;
          w.x = pack_bf16x2(o[g][0] * inv, o[g][1] * inv); w.y = pack_bf16x2(o[g][2] * inv, o[g][3] * inv);
          w.z = pack_bf16x2(o[g][4] * inv, o[g][5] * inv); w.w = pack_bf16x2(o[g][6] * inv, o[g][7] * inv);
          *reinterpret_cast<uint4*>(p.out + hrow * D + dg * 8) = w;
        } else {
          float4* dst = reinterpret_cast<float4*>(p.part_o + (hrow * p.parts + part) * D + dg * 8);
          dst[0] = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
          dst[1] = make_float4(o[g][4], o[g][5], o[g][6], o[g][7]);
        }
      }
    }
  }
  if (p.parts > 1 && threadIdx.x < G) {
    const long long hrow = static_cast<long long>(t) * p.H + kvh * G + threadIdx.x;
    p.part_ml[(hrow * p.parts + part) * 2 + 0] = s_m[threadIdx.x];
    p.part_ml[(hrow * p.parts + part) * 2 + 1] = s_l[threadIdx.x];
  }
}

// Staged variant for D = 128 and at most 8 query heads per KV head.  K and V of a key are adjacent in the cache (512 bytes
// per (slot, kv head)), so a stage of 32 keys is 16 KB that the CTA copies into shared memory with fully coalesced 16-byte
// cp.async requests (one pass over the cache instead of separate K and V passes with strided rows), double-buffered
// against the arithmetic.  Scores, an online softmax (running maximum and sum per head) and P.V all run from shared
// memory; rows are padded to 576 bytes, which makes the 16-byte reads of a quarter-warp conflict-free in both phases.
constexpr int kStageKeys = 32;
constexpr int kStageRow = 2 * 128 + 32;  // bf16 elements per staged row: K (128), V (128), padding (32)
constexpr int kStagedMaxG = 8;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

__global__ void __launch_bounds__(kThreads) paged_attention_staged_kernel(Params p) {
  constexpr int D = 128;
  const int t = blockIdx.x, kvh = blockIdx.y, part = blockIdx.z;
  const int G = p.H / p.KV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ __align__(16) __nv_bfloat16 s_kv[2][kStageKeys * kStageRow];  // 36 KB
  __shared__ __align__(16) float s_q[kStagedMaxG * D];                      // 4 KB; reused for the final reduction
  __shared__ float s_p[kStagedMaxG * kStageKeys];
  __shared__ float s_m[kStagedMaxG], s_l[kStagedMaxG], s_alpha[kStagedMaxG];
  __shared__ int s_rows[kPart];

  int seq = 0, ctx = 0;
  const bool live = locate(p, t, seq, ctx);
  const int k0 = part * kPart;
  if (!live || k0 >= ctx) {
    if (part == 0 && !live) {
      for (int i = threadIdx.x; i < G * D; i += kThreads)
        p.out[(static_cast<long long>(t) * p.H + kvh * G) * D + i] = __float2bfloat16(0.f);
    }
    return;
  }
  const int nk = min(kPart, ctx - k0);
  for (int i = threadIdx.x; i < G * D; i += kThreads)
    s_q[i] = __bfloat162float(p.q[(static_cast<long long>(t) * p.H + kvh * G) * D + i]) * p.scale;
  for (int i = threadIdx.x; i < nk; i += kThreads) {
    const int key = k0 + i;
    const int page = p.page_indices[seq * p.pages_per_seq + key / p.page_size];
    s_rows[i] = (page >= 0 && page < p.num_pages) ? page * p.page_size + key % p.page_size : -1;
  }
  if (threadIdx.x < kStagedMaxG) { s_m[threadIdx.x] = -INFINITY; s_l[threadIdx.x] = 0.f; }
  __syncthreads();

  const long long tok_stride = 2LL * p.KV * D;
  const int stages = (nk + kStageKeys - 1) / kStageKeys;
  // copy of one stage: 32 rows x 32 chunks of 16 bytes, 8 per thread; rows without a key (or a bad page) are zero-filled
  auto issue = [&](int st) {
    __nv_bfloat16* dst = s_kv[st & 1];
    for (int c = threadIdx.x; c < kStageKeys * 32; c += kThreads) {
      const int r = c >> 5, ch = c & 31;
      const int i = st * kStageKeys + r;
      const int slot = i < nk ? s_rows[i] : -1;
      __nv_bfloat16* d = dst + r * kStageRow + ch * 8;
      if (slot >= 0) cp_async_16(d, p.kv_pages + slot * tok_stride + (2LL * kvh) * D + ch * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(0);

  const int key_l = threadIdx.x >> 2, quarter = threadIdx.x & 3;   // scoring: 4 threads per key
  const int dg = threadIdx.x & 15, kg = threadIdx.x >> 4;          // P.V: 16 dimension groups x 8 key groups
  float o[kStagedMaxG][8];
#pragma unroll
  for (int g = 0; g < kStagedMaxG; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) o[g][e] = 0.f;

  for (int st = 0; st < stages; ++st) {
    if (st + 1 < stages) issue(st + 1);
    else asm volatile("cp.async.commit_group;" ::: "memory");  // keep "all but the newest group" meaning the current stage
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const __nv_bfloat16* buf = s_kv[st & 1];
    {  // scores of key key_l: this thread takes chunks quarter, quarter + 4, ... of the K row
      float acc[kStagedMaxG];
#pragma unroll
      for (int g = 0; g < kStagedMaxG; ++g) acc[g] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int ch = j * 4 + quarter;
        float kf[8];
        load_row<8>(buf + key_l * kStageRow + ch * 8, kf);
#pragma unroll
        for (int g = 0; g < kStagedMaxG; ++g) {
          if (g < G) {
            const float4 qa = *reinterpret_cast<const float4*>(s_q + g * D + ch * 8);
            const float4 qb = *reinterpret_cast<const float4*>(s_q + g * D + ch * 8 + 4);
            acc[g] = fmaf(kf[0], qa.x, acc[g]); acc[g] = fmaf(kf[1], qa.y, acc[g]);
            acc[g] = fmaf(kf[2], qa.z, acc[g]); acc[g] = fmaf(kf[3], qa.w, acc[g]);
            acc[g] = fmaf(kf[4], qb.x, acc[g]); acc[g] = fmaf(kf[5], qb.y, acc[g]);
            acc[g] = fmaf(kf[6], qb.z, acc[g]); acc[g] = fmaf(kf[7], qb.w, acc[g]);
          }
        }
      }
      const int i = st * kStageKeys + key_l;
      const bool valid = i < nk && s_rows[i] >= 0;
#pragma unroll
      for (int g = 0; g < kStagedMaxG; ++g) {
        if (g < G) {
          float v = acc[g];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          if (p.soft_cap > 0.f) v = p.soft_cap * tanhf(v / p.soft_cap);
          if (quarter == 0) s_p[g * kStageKeys + key_l] = valid ? v : -INFINITY;
        }
      }
    }
    __syncthreads();
    // online softmax: warp w updates heads w, w + 4; one key per lane
    for (int g = warp; g < G; g += kThreads / 32) {
      const float sc = s_p[g * kStageKeys + lane];
      float m_st = sc;
#pragma unroll
      for (int of = 16; of > 0; of >>= 1) m_st = fmaxf(m_st, __shfl_xor_sync(0xffffffffu, m_st, of));
      const float m_old = s_m[g];
      const float m_new = fmaxf(m_old, m_st);
      const float e = (sc == -INFINITY || m_new == -INFINITY) ? 0.f : __expf(sc - m_new);
      const float alpha = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
      const float sum = warp_sum(e);
      s_p[g * kStageKeys + lane] = e;
      if (lane == 0) { s_m[g] = m_new; s_l[g] = s_l[g] * alpha + sum; s_alpha[g] = alpha; }
    }
    __syncthreads();
    {  // P.V: keys kg, kg + 8, kg + 16, kg + 24 of the stage; 8 output dimensions per thread
#pragma unroll
      for (int g = 0; g < kStagedMaxG; ++g) {
        if (g < G) {
          const float a = s_alpha[g];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[g][e] *= a;
        }
      }
#pragma unroll
      for (int j = 0; j < kStageKeys / 8; ++j) {
        const int r = kg + 8 * j;
        float vf[8];
        load_row<8>(buf + r * kStageRow + D + dg * 8, vf);
#pragma unroll
        for (int g = 0; g < kStagedMaxG; ++g) {
          if (g < G) {
            const float w = s_p[g * kStageKeys + r];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[g][e] = fmaf(w, vf[e], o[g][e]);
          }
        }
      }
    }
    __syncthreads();  // the next iteration's copy overwrites the other buffer, its scores overwrite s_p
  }
  // sum the 8 key groups (through the first stage buffer, which nothing reads any more) and write the result
  float* s_red = reinterpret_cast<float*>(&s_kv[0][0]);  // 8 groups x G x 128 floats <= 32 KB
#pragma unroll
  for (int g = 0; g < kStagedMaxG; ++g) {
    if (g < G) {
#pragma unroll
      for (int e = 0; e < 8; ++e) s_red[(kg * kStagedMaxG + g) * D + dg * 8 + e] = o[g][e];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += kThreads) {
    const int g = idx / D, d = idx - g * D;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += s_red[(k * kStagedMaxG + g) * D + d];
    const long long hrow = static_cast<long long>(t) * p.H + kvh * G + g;
    if (p.parts == 1) {
      const float l = s_l[g];
      p.out[hrow * D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
    } else {
      p.part_o[(hrow * p.parts + part) * D + d] = acc;
    }
  }
  if (p.parts > 1 && threadIdx.x < G) {
    const long long hrow = static_cast<long long>(t) * p.H + kvh * G + threadIdx.x;
    p.part_ml[(hrow * p.parts + part) * 2 + 0] = s_m[threadIdx.x];
    p.part_ml[(hrow * p.parts + part) * 2 + 1] = s_l[threadIdx.x];
  }
}

// Tensor-core variant for D = 128 and at most 16 query heads per KV head.  The query heads that share a KV head are the M rows
// of warp-level MMAs (m16n8k16, bf16, fp32 accumulation; rows beyond G are zero), so one pass over a key's K and V rows
// serves all of them at a sixteenth of the instruction count of the scalar kernels, which were bound by instruction issue
// and shared-memory reads, not by the cache traffic.  Each of the four warps owns 64 keys of the partition and is its own
// pipeline: it copies stages of 16 keys (K and V rows are adjacent in the cache: 512 bytes per key, padded to 528 in
// shared memory so that ldmatrix reads are conflict-free) with cp.async, double-buffered, and needs no CTA-wide barrier
// inside the loop.  Scores S = Q K^T come from ldmatrix'd K rows, the online softmax runs on the accumulator fragments,
// P is re-packed in registers as the A operand of O += P V (V rows through ldmatrix.trans), and the four warps' (max, sum,
// O) are merged through shared memory at the end.
constexpr int kMmaStageKeys = 16;
constexpr int kMmaRowBytes = 528;  // K (256 B) + V (256 B) + 16 B padding
constexpr int kMmaWarpKeys = kPart / (kThreads / 32);  // 64
constexpr int kMmaStageBytes = kMmaStageKeys * kMmaRowBytes;

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kThreads) paged_attention_mma_kernel(Params p) {
  constexpr int D = 128;
  const int t = blockIdx.x, kvh = blockIdx.y, part = blockIdx.z;
  const int G = p.H / p.KV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  extern __shared__ __align__(16) uint8_t s_dyn[];
  uint8_t* s_stage = s_dyn;                                   // [4 warps][2 stages][16 keys][528 B] = 67584 B; reused for the merge
  int* s_rows = reinterpret_cast<int*>(s_dyn + 4 * 2 * kMmaStageBytes);  // [kPart]
  float* s_ml = reinterpret_cast<float*>(s_rows + kPart);     // [4 warps][16 rows][2]

  int seq = 0, ctx = 0;
  const bool live = locate(p, t, seq, ctx);
  const int k0 = part * kPart;
  if (!live || k0 >= ctx) {
    if (part == 0 && !live) {
      for (int i = threadIdx.x; i < G * D; i += kThreads)
        p.out[(static_cast<long long>(t) * p.H + kvh * G) * D + i] = __float2bfloat16(0.f);
    }
    return;
  }
  const int nk = min(kPart, ctx - k0);
  for (int i = threadIdx.x; i < kPart; i += kThreads) {
    int slot = -1;
    if (i < nk) {
      const int key = k0 + i;
      const int page = p.page_indices[seq * p.pages_per_seq + key / p.page_size];
      slot = (page >= 0 && page < p.num_pages) ? page * p.page_size + key % p.page_size : -1;
    }
    s_rows[i] = slot;
  }
  __syncthreads();

  // ---- Q as A fragments (rows = query heads of this KV head, zero beyond G): 8 k-steps of 16 dimensions
  const int row_lo = lane >> 2, row_hi = row_lo + 8, kq = (lane & 3) * 2;
  uint32_t qa[8][4];
  {
    const __nv_bfloat16* qbase = p.q + (static_cast<long long>(t) * p.H + kvh * G) * D;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int d0 = ks * 16 + kq;
      qa[ks][0] = row_lo < G ? *reinterpret_cast<const uint32_t*>(qbase + row_lo * D + d0) : 0u;
      qa[ks][1] = row_hi < G ? *reinterpret_cast<const uint32_t*>(qbase + row_hi * D + d0) : 0u;
      qa[ks][2] = row_lo < G ? *reinterpret_cast<const uint32_t*>(qbase + row_lo * D + d0 + 8) : 0u;
      qa[ks][3] = row_hi < G ? *reinterpret_cast<const uint32_t*>(qbase + row_hi * D + d0 + 8) : 0u;
    }
  }

  const long long tok_stride = 2LL * p.KV * D;
  const int wk0 = warp * kMmaWarpKeys;                       // this warp's first key inside the partition
  const int wnk = max(0, min(kMmaWarpKeys, nk - wk0));       // and how many of its 64 are real
  const int stages = (wnk + kMmaStageKeys - 1) / kMmaStageKeys;
  uint8_t* my_stage = s_stage + warp * (2 * kMmaStageBytes);
  // one stage: 16 rows x 32 chunks of 16 bytes, 16 per lane; rows without a key are zero-filled (0 * NaN would poison O)
  auto issue = [&](int st) {
    uint8_t* dst = my_stage + (st & 1) * kMmaStageBytes;
#pragma unroll 4
    for (int c = lane; c < kMmaStageKeys * 32; c += 32) {
      const int r = c >> 5, ch = c & 31;
      const int i = wk0 + st * kMmaStageKeys + r;
      const int slot = (st * kMmaStageKeys + r < wnk) ? s_rows[i] : -1;
      uint8_t* d = dst + r * kMmaRowBytes + ch * 16;
      if (slot >= 0) cp_async_16(d, p.kv_pages + slot * tok_stride + (2LL * kvh) * D + ch * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;  // running max / sum of rows row_lo and row_hi
  const float sc_log2 = p.scale * 1.4426950408889634f;

  if (stages > 0) issue(0);
  for (int st = 0; st < stages; ++st) {
    if (st + 1 < stages) issue(st + 1);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncwarp();
    const uint32_t buf = smem_u32(my_stage + (st & 1) * kMmaStageBytes);
    // ---- S[16 heads, 16 keys] = Q K^T: two n-tiles of 8 keys
    float sacc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {  // 32 dimensions per ldmatrix.x4: matrices (d 0-7), (8-15), (16-23), (24-31) of the 8 keys
        uint32_t b0, b1, b2, b3;
        const uint32_t addr = buf + (8 * j + (lane & 7)) * kMmaRowBytes + (kp * 32 + (lane >> 3) * 8) * 2;
        ldmatrix_x4(addr, b0, b1, b2, b3);
        mma_16816(sacc[j], qa[2 * kp], b0, b1);
        mma_16816(sacc[j], qa[2 * kp + 1], b2, b3);
      }
    }
    // ---- online softmax on the fragments: this lane holds keys (lane % 4) * 2 + {0, 1} of each n-tile, rows row_lo / row_hi
    float rmax_lo = -INFINITY, rmax_hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kcol = st * kMmaStageKeys + 8 * j + kq + (e & 1);
        const bool valid = kcol < wnk && s_rows[wk0 + kcol] >= 0;
        float v = sacc[j][e];
        if (p.soft_cap > 0.f) v = p.soft_cap * tanhf(v * p.scale / p.soft_cap) * 1.4426950408889634f;
        else v *= sc_log2;
        v = valid ? v : -INFINITY;
        sacc[j][e] = v;
        if (e < 2) rmax_lo = fmaxf(rmax_lo, v); else rmax_hi = fmaxf(rmax_hi, v);
      }
    }
    rmax_lo = fmaxf(rmax_lo, __shfl_xor_sync(0xffffffffu, rmax_lo, 1));
    rmax_lo = fmaxf(rmax_lo, __shfl_xor_sync(0xffffffffu, rmax_lo, 2));
    rmax_hi = fmaxf(rmax_hi, __shfl_xor_sync(0xffffffffu, rmax_hi, 1));
    rmax_hi = fmaxf(rmax_hi, __shfl_xor_sync(0xffffffffu, rmax_hi, 2));
    const float mn_lo = fmaxf(m_lo, rmax_lo), mn_hi = fmaxf(m_hi, rmax_hi);
    const float a_lo = (m_lo == -INFINITY) ? 0.f : exp2f(m_lo - mn_lo);
    const float a_hi = (m_hi == -INFINITY) ? 0.f : exp2f(m_hi - mn_hi);
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pa[4];
    {
      float pv[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        pv[j][0] = (mn_lo == -INFINITY) ? 0.f : exp2f(sacc[j][0] - mn_lo);
        pv[j][1] = (mn_lo == -INFINITY) ? 0.f : exp2f(sacc[j][1] - mn_lo);
        pv[j][2] = (mn_hi == -INFINITY) ? 0.f : exp2f(sacc[j][2] - mn_hi);
        pv[j][3] = (mn_hi == -INFINITY) ? 0.f : exp2f(sacc[j][3] - mn_hi);
        sum_lo += pv[j][0] + pv[j][1];
        sum_hi += pv[j][2] + pv[j][3];
      }
      pa[0] = pack_bf16x2(pv[0][0], pv[0][1]);  // (row_lo, keys 0-7 tile)
      pa[1] = pack_bf16x2(pv[0][2], pv[0][3]);  // (row_hi, keys 0-7 tile)
      pa[2] = pack_bf16x2(pv[1][0], pv[1][1]);  // (row_lo, keys 8-15 tile)
      pa[3] = pack_bf16x2(pv[1][2], pv[1][3]);  // (row_hi, keys 8-15 tile)
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * a_lo + sum_lo;
    l_hi = l_hi * a_hi + sum_hi;
    m_lo = mn_lo;
    m_hi = mn_hi;
    // ---- O[16 heads, 128 d] = O * alpha + P V: pairs of 8-wide d tiles per ldmatrix.x4.trans
#pragma unroll
    for (int np = 0; np < 8; ++np) {
      uint32_t b0, b1, b2, b3;
      // matrices: (keys 0-7, d 16 np .. +7), (keys 8-15, same d), (keys 0-7, d 16 np + 8 ..), (keys 8-15, same)
      const int mi = lane >> 3;
      const uint32_t addr = buf + ((mi & 1) * 8 + (lane & 7)) * kMmaRowBytes + 256 + (np * 16 + (mi >> 1) * 8) * 2;
      ldmatrix_x4_trans(addr, b0, b1, b2, b3);
      float* oa = o[2 * np];
      float* ob = o[2 * np + 1];
      oa[0] *= a_lo; oa[1] *= a_lo; oa[2] *= a_hi; oa[3] *= a_hi;
      ob[0] *= a_lo; ob[1] *= a_lo; ob[2] *= a_hi; ob[3] *= a_hi;
      mma_16816(o[2 * np], pa, b0, b1);
      mma_16816(o[2 * np + 1], pa, b2, b3);
    }
    __syncwarp();  // every lane is done with this buffer before the copy of stage st + 2 overwrites it
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();  // all warps are out of their pipelines: the stage memory becomes the merge buffer

  // ---- merge the four warps: per row the global max, then the rescaled sums and outputs
  if ((lane & 3) == 0) {
    s_ml[(warp * 16 + row_lo) * 2 + 0] = m_lo;
    s_ml[(warp * 16 + row_lo) * 2 + 1] = l_lo;
    s_ml[(warp * 16 + row_hi) * 2 + 0] = m_hi;
    s_ml[(warp * 16 + row_hi) * 2 + 1] = l_hi;
  }
  float* s_o = reinterpret_cast<float*>(s_stage);  // [4 warps][16 rows][128] fp32 = 32 KB
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    const int d0 = n * 8 + kq;
    *reinterpret_cast<float2*>(s_o + (warp * 16 + row_lo) * D + d0) = make_float2(o[n][0], o[n][1]);
    *reinterpret_cast<float2*>(s_o + (warp * 16 + row_hi) * D + d0) = make_float2(o[n][2], o[n][3]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += kThreads) {
    const int g = idx / D, d = idx - g * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, s_ml[(w * 16 + g) * 2]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = s_ml[(w * 16 + g) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      acc = fmaf(s_o[(w * 16 + g) * D + d], f, acc);
      l = fmaf(s_ml[(w * 16 + g) * 2 + 1], f, l);
    }
    const long long hrow = static_cast<long long>(t) * p.H + kvh * G + g;
    if (p.parts == 1) {
      p.out[hrow * D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
    } else {
      p.part_o[(hrow * p.parts + part) * D + d] = acc;
      if (d == 0) {
        // the merge kernel works with natural-log maxima: this kernel's are in base 2
        p.part_ml[(hrow * p.parts + part) * 2 + 0] = (m == -INFINITY) ? -INFINITY : m * 0.6931471805599453f;
        p.part_ml[(hrow * p.parts + part) * 2 + 1] = l;
      }
    }
  }
}
constexpr int kMmaSmem = 4 * 2 * kMmaStageBytes + kPart * 4 + 4 * 16 * 2 * 4;

// One CTA per (token, head): merge the partials of the partitions that were live for this token.
template <int D>
__global__ void __launch_bounds__(D <= 128 ? 128 : 256) paged_merge_kernel(Params p) {
  const int t = blockIdx.x, h = blockIdx.y;
  int seq = 0, ctx = 0;
  if (!locate(p, t, seq, ctx)) return;  // zeros were written by the attention kernel
  const int np = (ctx + kPart - 1) / kPart;
  const long long hrow = static_cast<long long>(t) * p.H + h;
  float m = -INFINITY;
  for (int i = 0; i < np; ++i) m = fmaxf(m, p.part_ml[(hrow * p.parts + i) * 2]);
  float l = 0.f;
  for (int i = 0; i < np; ++i) {
    const float mi = p.part_ml[(hrow * p.parts + i) * 2];
    l += (mi == -INFINITY) ? 0.f : p.part_ml[(hrow * p.parts + i) * 2 + 1] * __expf(mi - m);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int i = 0; i < np; ++i) {
      const float mi = p.part_ml[(hrow * p.parts + i) * 2];
      if (mi == -INFINITY) continue;
      o = fmaf(p.part_o[(hrow * p.parts + i) * D + d], __expf(mi - m), o);
    }
    p.out[hrow * D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
  }
}

// LVB_PAGED_ATTENTION=direct selects the kernel that reads the cache rows straight from global memory for every shape,
// LVB_PAGED_ATTENTION=staged the scalar kernel on staged rows; the default for D = 128 is the tensor-core kernel.
inline int paged_variant() {
  static const int v = [] {
    const char* e = std::getenv("LVB_PAGED_ATTENTION");
    if (e != nullptr && std::string(e) == "direct") return 0;
    if (e != nullptr && std::string(e) == "staged") return 1;
    return 2;
  }();
  return v;
}

template <int D>
int launch(const Params& p, cudaStream_t s) {
  dim3 grid(p.T, p.KV, p.parts);
  const int variant = paged_variant();
  if (D == 128 && p.H / p.KV <= 16 && variant == 2) {
    static bool attr_set = false;
    if (!attr_set) {
      if (cudaFuncSetAttribute(paged_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem) != cudaSuccess) return kErrCuda;
      attr_set = true;
    }
    paged_attention_mma_kernel<<<grid, kThreads, kMmaSmem, s>>>(p);
  } else if (D == 128 && p.H / p.KV <= kStagedMaxG && variant >= 1) {
    paged_attention_staged_kernel<<<grid, kThreads, 0, s>>>(p);
  } else {
    paged_attention_kernel<D><<<grid, kThreads, 0, s>>>(p);
  }
  if (p.parts > 1) paged_merge_kernel<D><<<dim3(p.T, p.H), D <= 128 ? 128 : 256, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace paged
}  // namespace lvb

// kv_pages[num_pages, page_size, 2 * kv_heads, D]; k, v [T, kv_heads, D] bf16; dests int32 [T] (page * page_size + slot;
// out-of-range values are skipped).  D must be a multiple of 8.
extern "C" int lvb_kv_page_write(void* kv_pages, const void* k, const void* v, const int* dests, int T, int kv_heads, int D,
                                 long long total_slots, void* stream) {
  using namespace lvb;
  if (T <= 0) return kErrOk;
  if (kv_heads <= 0 || D <= 0 || (D & 7)) return kErrBadArg;
  paged::kv_page_write_kernel<<<T, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(kv_pages), reinterpret_cast<const __nv_bfloat16*>(k),
      reinterpret_cast<const __nv_bfloat16*>(v), dests, kv_heads, D, total_slots);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// Number of key partitions for a cache whose sequences hold at most max_context tokens: sizes the scratch buffers
// part_o fp32 [T, H, parts, D] and part_ml fp32 [T, H, parts, 2] (unused when parts == 1).
extern "C" int lvb_paged_attention_parts(int max_context) { return (max_context + lvb::paged::kPart - 1) / lvb::paged::kPart; }

extern "C" int lvb_paged_attention(const void* q, const void* kv_pages, const int* kv_lens, const int* page_indices,
                                   const int* cu_q_lens, const int* num_seqs, void* out, float* part_o, float* part_ml, int T,
                                   int H, int KV, int D, int S, int pages_per_seq, int page_size, int num_pages, float scale,
                                   float soft_cap, void* stream) {
  using namespace lvb;
  using namespace lvb::paged;
  if (T <= 0) return kErrOk;
  if (H <= 0 || KV <= 0 || H % KV != 0 || H / KV > kMaxG || S <= 0) return kErrBadArg;
  Params p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.kv_pages = reinterpret_cast<const __nv_bfloat16*>(kv_pages);
  p.kv_lens = kv_lens; p.page_indices = page_indices; p.cu_q_lens = cu_q_lens; p.num_seqs = num_seqs;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.part_o = part_o; p.part_ml = part_ml;
  p.T = T; p.H = H; p.KV = KV; p.S = S; p.pages_per_seq = pages_per_seq; p.page_size = page_size; p.num_pages = num_pages;
  p.parts = lvb_paged_attention_parts(pages_per_seq * page_size);
  p.scale = scale; p.soft_cap = soft_cap;
  if (p.parts > 1 && (part_o == nullptr || part_ml == nullptr)) return kErrBadArg;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (D) {
    case 64: return launch<64>(p, s);
    case 128: return launch<128>(p, s);
    case 256: return launch<256>(p, s);
    default: return kErrBadArg;
  }
}
