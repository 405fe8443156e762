// Gated delta rule: the sequential part of the chunked scan as one kernel per direction.
//
// The chunk-parallel quantities (the WY factors u, w, the decayed queries/keys and the masked intra-chunk scores) are
// batched matrix products that the caller computes for all chunks at once.  What is left is a loop over the chunks that
// carries the [d_k, d_v] state of every (batch, head):
//
//     v_new = u_n - w_n S                 [C, d_v]
//     o_n   = qg_n S + P_n v_new          [C, d_v]
//     S     = a_n S + kd_n^T v_new        [d_k, d_v]
//
// Written with framework ops this is about nine launches per chunk on small matrices; here one CTA owns one (batch, head)
// and one slice of the d_v columns (the columns of S never mix), keeps its slice of S in shared memory for the whole
// sequence and streams the chunk tiles through shared memory with cp.async while the previous step computes.  The backward
// kernel walks the chunks in reverse with the gradient of the state in shared memory, recomputes v_new from the saved
// entering states and writes the gradients of every tile; sums over d_v (dw, dqg, dkd, dP, da) are written per slice and
// added by the caller in a fixed order, so results are bitwise reproducible.
//
// The products are warp-level m16n8k8 TF32 tensor-core operations with fp32 accumulation on fp32 operands in shared
// memory (the state stays fp32 across the sequence); `exact != 0` selects plain fp32 FMAs with the same tiling, which is
// the oracle for the fragment layout.  The reference framework has no such model family or kernel.
#include "common.cuh"

namespace lvb {
namespace delta {

constexpr int kC = 64;         // chunk length
constexpr int kThreads = 256;  // 8 warps

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// acc[j][i] (+)= sum_k A(row, k) * B(k, col) for k in [k_begin, k_end) (multiples of 8), where this lane's elements are
//   row = m0 + (lane >> 2) + 8 * (i >> 1),   col = n0 + 8 * j + 2 * (lane & 3) + (i & 1).
// A and B are callables returning fp32 from shared memory, so any operand may be read transposed or negated.
template <int NT, class FA, class FB>
__device__ __forceinline__ void warp_gemm(float (&acc)[NT][4], int m0, int n0, int k_begin, int k_end, bool exact, FA A, FB B) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if (!exact) {
    for (int k0 = k_begin; k0 < k_end; k0 += 8) {
      const uint32_t a0 = to_tf32(A(m0 + g, k0 + t));
      const uint32_t a1 = to_tf32(A(m0 + g + 8, k0 + t));
      const uint32_t a2 = to_tf32(A(m0 + g, k0 + t + 4));
      const uint32_t a3 = to_tf32(A(m0 + g + 8, k0 + t + 4));
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint32_t b0 = to_tf32(B(k0 + t, n0 + 8 * j + g));
        const uint32_t b1 = to_tf32(B(k0 + t + 4, n0 + 8 * j + g));
        mma_tf32(acc[j], a0, a1, a2, a3, b0, b1);
      }
    }
  } else {
    for (int k = k_begin; k < k_end; ++k) {
      const float x0 = A(m0 + g, k), x1 = A(m0 + g + 8, k);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const float y0 = B(k, n0 + 8 * j + 2 * t), y1 = B(k, n0 + 8 * j + 2 * t + 1);
        acc[j][0] = fmaf(x0, y0, acc[j][0]);
        acc[j][1] = fmaf(x0, y1, acc[j][1]);
        acc[j][2] = fmaf(x1, y0, acc[j][2]);
        acc[j][3] = fmaf(x1, y1, acc[j][3]);
      }
    }
  }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_newest() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// rows x COLS fp32 from global (row stride src_ld floats, 16-byte aligned rows) into shared memory (row stride ld floats)
template <int COLS>
__device__ __forceinline__ void tile_load_async(float* dst, int ld, const float* src, size_t src_ld, int rows) {
  constexpr int V = COLS / 4;
  for (int i = threadIdx.x; i < rows * V; i += kThreads) {
    const int r = i / V, c4 = i - r * V;
    cp_async16(dst + r * ld + c4 * 4, src + static_cast<size_t>(r) * src_ld + c4 * 4);
  }
}

struct FwdParams {
  const float *w, *qg, *kd, *P, *u, *a, *S0;
  float *out, *S_hist, *S_final;
  int BH, N, DV, exact;
};

template <int DK, int DVT>
struct FwdSmem {
  static constexpr int ldW = DK + 4;    // read as A(m, k) = [m][k]
  static constexpr int ldQ = DK + 4;
  static constexpr int ldK = DK + 8;    // read transposed, A(m, k) = [k][m]
  static constexpr int ldP = kC + 4;
  static constexpr int ldV = DVT + 8;   // read as B(k, n) = [k][n]
  static constexpr int ldS = DVT + 8;
  static constexpr int oW = 0;
  static constexpr int oQ = oW + kC * ldW;
  static constexpr int oK = oQ + kC * ldQ;
  static constexpr int oP = oK + kC * ldK;
  static constexpr int oV = oP + kC * ldP;
  static constexpr int oS = oV + 2 * kC * ldV;  // u / v_new is double-buffered
  static constexpr int floats = oS + DK * ldS;
};

template <int DK, int DVT>
__global__ void __launch_bounds__(kThreads) delta_fwd_kernel(const FwdParams p) {
  using L = FwdSmem<DK, DVT>;
  extern __shared__ __align__(16) float smem[];
  float* sW = smem + L::oW;
  float* sQ = smem + L::oQ;
  float* sK = smem + L::oK;
  float* sP = smem + L::oP;
  float* sVbuf = smem + L::oV;
  float* sS = smem + L::oS;

  const int bh = blockIdx.y;
  const int dv0 = blockIdx.x * DVT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const bool exact = p.exact != 0;
  const size_t DV = p.DV;

  const size_t tile_k = static_cast<size_t>(kC) * DK;
  const float* gw = p.w + static_cast<size_t>(bh) * p.N * tile_k;
  const float* gq = p.qg + static_cast<size_t>(bh) * p.N * tile_k;
  const float* gk = p.kd + static_cast<size_t>(bh) * p.N * tile_k;
  const float* gP = p.P + static_cast<size_t>(bh) * p.N * kC * kC;
  const float* gu = p.u + static_cast<size_t>(bh) * p.N * kC * DV + dv0;
  float* gout = p.out + static_cast<size_t>(bh) * p.N * kC * DV + dv0;

  // chunk 0 tiles.  Copy groups complete in order and every wait below is "all but the newest group": the keys of a chunk
  // are only needed by its last step, so their copy (always the newest group at the top of an iteration) stays in flight
  // through the first two steps.
  tile_load_async<DK>(sW, L::ldW, gw, DK, kC);
  tile_load_async<DK>(sQ, L::ldQ, gq, DK, kC);
  tile_load_async<kC>(sP, L::ldP, gP, kC, kC);
  tile_load_async<DVT>(sVbuf, L::ldV, gu, DV, kC);
  cp_async_commit();
  tile_load_async<DK>(sK, L::ldK, gk, DK, kC);
  cp_async_commit();
  for (int i = threadIdx.x; i < DK * DVT; i += kThreads) {
    const int r = i / DVT, c = i - r * DVT;
    sS[r * L::ldS + c] = p.S0 ? p.S0[(static_cast<size_t>(bh) * DK + r) * DV + dv0 + c] : 0.f;
  }

  // warp tiles: [C, DVT] products use 4 row tiles x 2 column halves; the state update uses DK/16 row tiles
  constexpr int NT_O = DVT / 16;
  const int mo = (warp & 3) * 16, no = (warp >> 2) * (DVT / 2);
  constexpr int MW = DK / 16;            // warps along the rows of S (8 or 4)
  constexpr int NW = 8 / MW;             // warps along its columns (1 or 2)
  constexpr int NT_S = DVT / 8 / NW;
  const int ms = (warp % MW) * 16, ns = (warp / MW) * (DVT / NW);

  for (int n = 0; n < p.N; ++n) {
    cp_async_wait_but_newest();  // everything but this chunk's keys
    __syncthreads();
    const bool more = n + 1 < p.N;
    float* sV = sVbuf + (n & 1) * kC * L::ldV;
    {  // v_new = u - w S (in place over u)
      float acc[NT_O][4];
      zero_acc(acc);
      warp_gemm<NT_O>(acc, mo, no, 0, DK, exact, [&](int m, int k) { return sW[m * L::ldW + k]; },
                      [&](int k, int c) { return sS[k * L::ldS + c]; });
#pragma unroll
      for (int j = 0; j < NT_O; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = mo + g + 8 * (i >> 1), c = no + 8 * j + 2 * t + (i & 1);
          sV[r * L::ldV + c] -= acc[j][i];
        }
    }
    __syncthreads();
    if (more) {  // the other u buffer was last read by the previous chunk's state update
      tile_load_async<DK>(sW, L::ldW, gw + (n + 1) * tile_k, DK, kC);
      tile_load_async<DVT>(sVbuf + ((n + 1) & 1) * kC * L::ldV, L::ldV, gu + static_cast<size_t>(n + 1) * kC * DV, DV, kC);
    }
    cp_async_commit();  // committed even when empty, so that "all but the newest" always means the same groups
    {  // o = qg S + P v_new; P is lower triangular, so rows mo..mo+15 need k < mo + 16 only
      float acc[NT_O][4];
      zero_acc(acc);
      warp_gemm<NT_O>(acc, mo, no, 0, DK, exact, [&](int m, int k) { return sQ[m * L::ldQ + k]; },
                      [&](int k, int c) { return sS[k * L::ldS + c]; });
      warp_gemm<NT_O>(acc, mo, no, 0, mo + 16, exact, [&](int m, int k) { return sP[m * L::ldP + k]; },
                      [&](int k, int c) { return sV[k * L::ldV + c]; });
      float* o = gout + static_cast<size_t>(n) * kC * DV;
#pragma unroll
      for (int j = 0; j < NT_O; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = mo + g + 8 * h, c = no + 8 * j + 2 * t;
          *reinterpret_cast<float2*>(o + static_cast<size_t>(r) * DV + c) = make_float2(acc[j][2 * h], acc[j][2 * h + 1]);
        }
    }
    cp_async_wait_but_newest();  // this chunk's keys have landed (the newest group is the next w / u)
    __syncthreads();
    if (more) {
      tile_load_async<DK>(sQ, L::ldQ, gq + (n + 1) * tile_k, DK, kC);
      tile_load_async<kC>(sP, L::ldP, gP + static_cast<size_t>(n + 1) * kC * kC, kC, kC);
    }
    cp_async_commit();
    {  // S = a S + kd^T v_new; the entering state is saved for the backward pass
      const float a = p.a[static_cast<size_t>(bh) * p.N + n];
      float acc[NT_S][4];
      float* hist = p.S_hist ? p.S_hist + ((static_cast<size_t>(bh) * p.N + n) * DK) * DV + dv0 : nullptr;
#pragma unroll
      for (int j = 0; j < NT_S; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = ms + g + 8 * h, c = ns + 8 * j + 2 * t;
          const float2 s = *reinterpret_cast<const float2*>(&sS[r * L::ldS + c]);
          if (hist) *reinterpret_cast<float2*>(hist + static_cast<size_t>(r) * DV + c) = s;
          acc[j][2 * h] = a * s.x;
          acc[j][2 * h + 1] = a * s.y;
        }
      warp_gemm<NT_S>(acc, ms, ns, 0, kC, exact, [&](int m, int k) { return sK[k * L::ldK + m]; },
                      [&](int k, int c) { return sV[k * L::ldV + c]; });
#pragma unroll
      for (int j = 0; j < NT_S; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = ms + g + 8 * h, c = ns + 8 * j + 2 * t;
          *reinterpret_cast<float2*>(&sS[r * L::ldS + c]) = make_float2(acc[j][2 * h], acc[j][2 * h + 1]);
        }
    }
    __syncthreads();
    if (more) tile_load_async<DK>(sK, L::ldK, gk + (n + 1) * tile_k, DK, kC);
    cp_async_commit();
  }
  if (p.S_final)
    for (int i = threadIdx.x; i < DK * DVT; i += kThreads) {
      const int r = i / DVT, c = i - r * DVT;
      p.S_final[(static_cast<size_t>(bh) * DK + r) * DV + dv0 + c] = sS[r * L::ldS + c];
    }
}

struct BwdParams {
  const float *w, *qg, *kd, *P, *u, *a, *S_hist, *dout, *dS_final;
  // per-slice partial sums over d_v: [slices][BH][N][...]; du and dS0 are complete
  float *dw, *dqg, *dkd, *dP, *da, *du, *dS0;
  int BH, N, DV, exact;
};

template <int DK, int DVT>
struct BwdSmem {
  static constexpr int ldW = DK + 4;   // A(m, k) = [m][k] for v_new; read transposed for dS
  static constexpr int ldQ = DK + 8;   // only read transposed
  static constexpr int ldK = DK + 4;   // A(m, k) = [m][k]
  static constexpr int ldP = kC + 8;   // only read transposed
  static constexpr int ldV = DVT + 8;  // v_new, dout, dv_new
  static constexpr int ldS = DVT + 8;  // S and dS
  static constexpr int oW = 0;
  static constexpr int oQ = oW + kC * ldW;
  static constexpr int oK = oQ + kC * ldQ;
  static constexpr int oP = oK + kC * ldK;
  static constexpr int oV = oP + kC * ldP;
  static constexpr int oDO = oV + kC * ldV;
  static constexpr int oDV = oDO + kC * ldV;
  static constexpr int oS = oDV + kC * ldV;
  static constexpr int oDS = oS + DK * ldS;
  static constexpr int oRed = oDS + DK * ldS;
  static constexpr int floats = oRed + 8;
};

template <int DK, int DVT>
__global__ void __launch_bounds__(kThreads) delta_bwd_kernel(const BwdParams p) {
  using L = BwdSmem<DK, DVT>;
  extern __shared__ __align__(16) float smem[];
  float* sW = smem + L::oW;
  float* sQ = smem + L::oQ;
  float* sK = smem + L::oK;
  float* sP = smem + L::oP;
  float* sV = smem + L::oV;
  float* sDO = smem + L::oDO;
  float* sDV = smem + L::oDV;
  float* sS = smem + L::oS;
  float* sDS = smem + L::oDS;
  float* sRed = smem + L::oRed;

  const int bh = blockIdx.y, slice = blockIdx.x;
  const int dv0 = slice * DVT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const bool exact = p.exact != 0;
  const size_t DV = p.DV;
  const size_t tile_k = static_cast<size_t>(kC) * DK;
  const size_t chunk0 = static_cast<size_t>(bh) * p.N;               // index of this (batch, head)'s first chunk
  const size_t part0 = (static_cast<size_t>(slice) * p.BH + bh) * p.N;  // same, inside this slice's partial outputs

  for (int i = threadIdx.x; i < DK * DVT; i += kThreads) {
    const int r = i / DVT, c = i - r * DVT;
    sDS[r * L::ldS + c] = p.dS_final ? p.dS_final[(static_cast<size_t>(bh) * DK + r) * DV + dv0 + c] : 0.f;
  }

  constexpr int NT_O = DVT / 16;  // [C, DVT] products: 4 row tiles x 2 column halves
  const int mo = (warp & 3) * 16, no = (warp >> 2) * (DVT / 2);
  constexpr int NT_K = DK / 16;   // [C, DK] products: 4 row tiles x 2 column halves
  const int nk = (warp >> 2) * (DK / 2);
  constexpr int NT_P = kC / 16;   // [C, C] product
  const int np = (warp >> 2) * (kC / 2);
  constexpr int MW = DK / 16, NW = 8 / MW, NT_S = DVT / 8 / NW;  // [DK, DVT] state gradient
  const int ms = (warp % MW) * 16, ns = (warp / MW) * (DVT / NW);

  for (int n = p.N - 1; n >= 0; --n) {
    __syncthreads();  // the previous iteration is done with every tile
    tile_load_async<DK>(sW, L::ldW, p.w + (chunk0 + n) * tile_k, DK, kC);
    tile_load_async<DK>(sQ, L::ldQ, p.qg + (chunk0 + n) * tile_k, DK, kC);
    tile_load_async<DK>(sK, L::ldK, p.kd + (chunk0 + n) * tile_k, DK, kC);
    tile_load_async<kC>(sP, L::ldP, p.P + (chunk0 + n) * kC * kC, kC, kC);
    tile_load_async<DVT>(sV, L::ldV, p.u + (chunk0 + n) * kC * DV + dv0, DV, kC);
    tile_load_async<DVT>(sDO, L::ldV, p.dout + (chunk0 + n) * kC * DV + dv0, DV, kC);
    tile_load_async<DVT>(sS, L::ldS, p.S_hist + (chunk0 + n) * DK * DV + dv0, DV, DK);
    cp_async_commit();
    cp_async_wait_all();
    __syncthreads();
    const float a = p.a[chunk0 + n];
    {  // v_new = u - w S
      float acc[NT_O][4];
      zero_acc(acc);
      warp_gemm<NT_O>(acc, mo, no, 0, DK, exact, [&](int m, int k) { return sW[m * L::ldW + k]; },
                      [&](int k, int c) { return sS[k * L::ldS + c]; });
#pragma unroll
      for (int j = 0; j < NT_O; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) sV[(mo + g + 8 * (i >> 1)) * L::ldV + no + 8 * j + 2 * t + (i & 1)] -= acc[j][i];
    }
    {  // dv_new = P^T dout + kd dS  (P^T is upper triangular: rows mo.. need k >= mo only); also du
      float acc[NT_O][4];
      zero_acc(acc);
      warp_gemm<NT_O>(acc, mo, no, mo, kC, exact, [&](int m, int k) { return sP[k * L::ldP + m]; },
                      [&](int k, int c) { return sDO[k * L::ldV + c]; });
      warp_gemm<NT_O>(acc, mo, no, 0, DK, exact, [&](int m, int k) { return sK[m * L::ldK + k]; },
                      [&](int k, int c) { return sDS[k * L::ldS + c]; });
      float* du = p.du + (chunk0 + n) * kC * DV + dv0;
#pragma unroll
      for (int j = 0; j < NT_O; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = mo + g + 8 * h, c = no + 8 * j + 2 * t;
          const float2 v = make_float2(acc[j][2 * h], acc[j][2 * h + 1]);
          *reinterpret_cast<float2*>(&sDV[r * L::ldV + c]) = v;
          *reinterpret_cast<float2*>(du + static_cast<size_t>(r) * DV + c) = v;
        }
    }
    __syncthreads();
    {  // dP = dout v_new^T
      float acc[NT_P][4];
      zero_acc(acc);
      warp_gemm<NT_P>(acc, mo, np, 0, DVT, exact, [&](int m, int k) { return sDO[m * L::ldV + k]; },
                      [&](int k, int c) { return sV[c * L::ldV + k]; });
      float* o = p.dP + (part0 + n) * kC * kC;
#pragma unroll
      for (int j = 0; j < NT_P; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<float2*>(o + (mo + g + 8 * h) * kC + np + 8 * j + 2 * t) = make_float2(acc[j][2 * h], acc[j][2 * h + 1]);
    }
    // dkd = v_new dS^T, dqg = dout S^T, dw = -dv_new S^T
    for (int which = 0; which < 3; ++which) {
      const float* sA = which == 0 ? sV : (which == 1 ? sDO : sDV);
      const float* sB = which == 0 ? sDS : sS;
      float* o = (which == 0 ? p.dkd : (which == 1 ? p.dqg : p.dw)) + (part0 + n) * tile_k;
      const float sign = which == 2 ? -1.f : 1.f;
      float acc[NT_K][4];
      zero_acc(acc);
      warp_gemm<NT_K>(acc, mo, nk, 0, DVT, exact, [&](int m, int k) { return sA[m * L::ldV + k]; },
                      [&](int k, int c) { return sB[c * L::ldS + k]; });
#pragma unroll
      for (int j = 0; j < NT_K; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<float2*>(o + (mo + g + 8 * h) * DK + nk + 8 * j + 2 * t) =
              make_float2(sign * acc[j][2 * h], sign * acc[j][2 * h + 1]);
    }
    {  // da = <S, dS> over this slice, summed in a fixed order
      float s = 0.f;
      for (int i = threadIdx.x; i < DK * DVT; i += kThreads) {
        const int r = i / DVT, c = i - r * DVT;
        s = fmaf(sS[r * L::ldS + c], sDS[r * L::ldS + c], s);
      }
      s = warp_sum(s);
      if (lane == 0) sRed[warp] = s;
    }
    __syncthreads();  // every read of dS above is done; sRed is complete
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int i = 0; i < kThreads / 32; ++i) s += sRed[i];
      p.da[part0 + n] = s;
    }
    {  // dS = a dS + qg^T dout - w^T dv_new
      float acc[NT_S][4];
#pragma unroll
      for (int j = 0; j < NT_S; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = a * sDS[(ms + g + 8 * (i >> 1)) * L::ldS + ns + 8 * j + 2 * t + (i & 1)];
      warp_gemm<NT_S>(acc, ms, ns, 0, kC, exact, [&](int m, int k) { return sQ[k * L::ldQ + m]; },
                      [&](int k, int c) { return sDO[k * L::ldV + c]; });
      warp_gemm<NT_S>(acc, ms, ns, 0, kC, exact, [&](int m, int k) { return -sW[k * L::ldW + m]; },
                      [&](int k, int c) { return sDV[k * L::ldV + c]; });
#pragma unroll
      for (int j = 0; j < NT_S; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) sDS[(ms + g + 8 * (i >> 1)) * L::ldS + ns + 8 * j + 2 * t + (i & 1)] = acc[j][i];
    }
  }
  __syncthreads();
  if (p.dS0)
    for (int i = threadIdx.x; i < DK * DVT; i += kThreads) {
      const int r = i / DVT, c = i - r * DVT;
      p.dS0[(static_cast<size_t>(bh) * DK + r) * DV + dv0 + c] = sDS[r * L::ldS + c];
    }
}

constexpr int kFwdSlice = 64;  // d_v columns per CTA, forward
constexpr int kBwdSlice = 32;  // backward keeps twice as many tiles resident, so its slices are narrower

template <int DK>
int launch_fwd(const FwdParams& p, cudaStream_t stream) {
  auto kern = delta_fwd_kernel<DK, kFwdSlice>;
  const int bytes = FwdSmem<DK, kFwdSlice>::floats * static_cast<int>(sizeof(float));
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return kErrCuda;
  kern<<<dim3(p.DV / kFwdSlice, p.BH), kThreads, bytes, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

template <int DK>
int launch_bwd(const BwdParams& p, cudaStream_t stream) {
  auto kern = delta_bwd_kernel<DK, kBwdSlice>;
  const int bytes = BwdSmem<DK, kBwdSlice>::floats * static_cast<int>(sizeof(float));
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return kErrCuda;
  kern<<<dim3(p.DV / kBwdSlice, p.BH), kThreads, bytes, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

}  // namespace delta
}  // namespace lvb

using namespace lvb;

// All tensors fp32 and contiguous: w, qg, kd [BH, N, 64, DK]; P [BH, N, 64, 64] (zero above the diagonal); u, out
// [BH, N, 64, DV]; a [BH, N]; S0 (may be null), S_final [BH, DK, DV]; S_hist (may be null) [BH, N, DK, DV].
// DK is 64 or 128, DV a multiple of 64.
extern "C" int lvb_delta_rule_fwd(const float* w, const float* qg, const float* kd, const float* P, const float* u,
                                  const float* a, const float* S0, float* out, float* S_hist, float* S_final, int BH, int N,
                                  int DK, int DV, int exact, void* stream) {
  if (BH <= 0 || N <= 0 || DV <= 0 || DV % delta::kFwdSlice != 0 || BH > 65535) return kErrBadArg;
  delta::FwdParams p{w, qg, kd, P, u, a, S0, out, S_hist, S_final, BH, N, DV, exact};
  if (DK == 128) return delta::launch_fwd<128>(p, static_cast<cudaStream_t>(stream));
  if (DK == 64) return delta::launch_fwd<64>(p, static_cast<cudaStream_t>(stream));
  return kErrBadArg;
}

extern "C" int lvb_delta_rule_bwd_slices(int DV) { return DV / delta::kBwdSlice; }

// dw, dqg, dkd [slices, BH, N, 64, DK], dP [slices, BH, N, 64, 64] and da [slices, BH, N] are per-slice partial sums
// (slices = lvb_delta_rule_bwd_slices(DV)) that the caller adds over the first axis; du [BH, N, 64, DV] and dS0
// [BH, DK, DV] (may be null) are complete.  dS_final may be null (no gradient flows into the final state).
extern "C" int lvb_delta_rule_bwd(const float* w, const float* qg, const float* kd, const float* P, const float* u,
                                  const float* a, const float* S_hist, const float* dout, const float* dS_final, float* dw,
                                  float* dqg, float* dkd, float* dP, float* da, float* du, float* dS0, int BH, int N, int DK,
                                  int DV, int exact, void* stream) {
  if (BH <= 0 || N <= 0 || DV <= 0 || DV % delta::kFwdSlice != 0 || BH > 65535 || S_hist == nullptr) return kErrBadArg;
  delta::BwdParams p{w, qg, kd, P, u, a, S_hist, dout, dS_final, dw, dqg, dkd, dP, da, du, dS0, BH, N, DV, exact};
  if (DK == 128) return delta::launch_bwd<128>(p, static_cast<cudaStream_t>(stream));
  if (DK == 64) return delta::launch_bwd<64>(p, static_cast<cudaStream_t>(stream));
  return kErrBadArg;
}
