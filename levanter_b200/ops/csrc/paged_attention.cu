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

// LVB_PAGED_ATTENTION=direct selects the kernel that reads the cache rows straight from global memory for every shape.
inline bool staged_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LVB_PAGED_ATTENTION");
    return !(v != nullptr && std::string(v) == "direct");
  }();
  return on;
}

template <int D>
int launch(const Params& p, cudaStream_t s) {
  dim3 grid(p.T, p.KV, p.parts);
  if (D == 128 && p.H / p.KV <= kStagedMaxG && staged_enabled())
    paged_attention_staged_kernel<<<grid, kThreads, 0, s>>>(p);
  else
    paged_attention_kernel<D><<<grid, kThreads, 0, s>>>(p);
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
