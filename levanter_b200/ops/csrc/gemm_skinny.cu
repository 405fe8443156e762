// bf16 GEMM for a few row blocks (M <= 512: decode steps, small batches) on sm_100a.
//
//   C[M,N] = alpha * A[M,K] B[N,K]^T (+ bias[N]) (+ residual[M,N]),   A and B K-major (the forward layout of a Linear).
//
// With so few rows the kernel is a stream over the weight matrix B, and the tensor cores idle; what decides its speed is how
// many bytes of B are in flight.  Compared with the general kernel (gemm_bf16.cu) this one therefore
//   * loads only the rows of A that exist (TMA box of round_up(M, 8) rows instead of 128; the MMA still spans 128 rows and
//     reads whatever the rest of the stage holds, which only feeds accumulator rows that are never stored),
//   * spends the shared memory this frees on a deeper ring of B tiles (up to 24 stages, sized at launch),
//   * splits K over several CTAs per column tile when there are few tiles: measured on B200, a CTA of this kernel advances
//     one 64-wide k-block every ~0.28 us whatever the tile width (32, 64 or 128 columns: 4 to 16 KB of B), the ring depth,
//     the number of rows of A, and whether B comes from DRAM or L2; so time = ~7 us + 0.28 us x (k-blocks per CTA), and the
//     way to go faster is 128-column tiles (most bytes per k-block) with fewer k-blocks per CTA.  Each split stores its
//     fp32 partial tile to a workspace slab [split, M, N]; a second small kernel sums the slabs in a fixed order (so the
//     result does not depend on timing) and applies alpha, bias, residual and the output type,
//   * spreads the K loop over several accumulators (k-block kb adds into accumulator kb % kAcc; the epilogue sums them):
//     MMAs into one accumulator run one after the other, and with a 32-column tile each of them is almost all latency, so
//     one chain of K/16 dependent MMAs, not the memory system, set the pace (measured: time proportional to K and the same
//     for 32- and 64-column tiles).  Independent chains overlap.
//   * takes up to four row blocks of 128 (M <= 512): a piece of work is (column tile, K split, row block) with the row block
//     fastest, so the CTAs that need the same tile of B run side by side and all but the first read it from L2.  Against the
//     general kernel's 256 x 256 pair tiles this fills the SMs when N / 256 is far below their number (the attention-output
//     and MLP-down projections of a 256-request decode round).
// Roles as in the general kernel: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue; two TMEM accumulators.
// Every wait is bounded (common.cuh).
#include "common.cuh"

namespace lvb {
namespace skinny {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kMaxStages = 24;
constexpr int kSmemBudget = 200 * 1024;  // ring bytes; the rest of the 227 KB holds barriers, slack and alignment

enum Flags : int { kOutF32 = 1, kBias = 4, kResidual = 8, kBiasF32 = 16 };

struct Params {
  void* C;
  const void* bias;
  const __nv_bfloat16* residual;
  int M, N, K;
  int ldc, ldr;
  int flags;
  float alpha;
  int tiles_n;
  int tiles_m;       // row blocks of 128
  int stages;        // ring depth
  int a_bytes;       // bytes of A loaded per stage (a_box_rows * 128)
  int splits;        // CTAs per column tile along K (1: the epilogue writes C itself)
  int kb_per_split;  // k-blocks per split
  float* ws;         // splits > 1: fp32 partials [splits, M, N]
  int* status;
};

template <int BN, int kAcc>
__global__ void __launch_bounds__(kThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  constexpr int kBBytes = BN * BK * 2;
  constexpr int kTmemCols = 2 * kAcc * BN;  // two buffers of kAcc accumulators
  static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // barriers first (1 KB), then the ring; the ring is followed by 16 KB of slack because the MMA addresses 128 rows of A
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* tfull_bar = empty_bar + kMaxStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  uint8_t* ring = smem + 1024;
  const int stride = p.a_bytes + kBBytes;
  const int stages = p.stages;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int num_work = p.tiles_n * p.splits * p.tiles_m;  // (column tile, K split, row block), row block fastest

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<kTmemCols>(tmem_holder);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_work && ok; t += gridDim.x) {
        const int m0 = (t % p.tiles_m) * BM;
        const int u = t / p.tiles_m;
        const int n0 = (u / p.splits) * BN;
        const int kb0 = (u % p.splits) * p.kb_per_split;
        const int kb1 = min(k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 100, stage);
          if (!ok) break;
          uint8_t* sa = ring + stage * stride;
          mbar_expect_tx(&full_bar[stage], stride);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, m0);
          tma_load_2d(sa + p.a_bytes, &tmB, &full_bar[stage], kb * BK, n0);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t tphase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_work && ok; t += gridDim.x) {
        ok = mbar_wait(&tempty_bar[buf], tphase ^ 1, abort_flag, p.status, 200, buf);
        if (!ok) break;
        tc_fence_after();
        const int kb0 = ((t / p.tiles_m) % p.splits) * p.kb_per_split;
        const int n_kb = min(k_blocks, kb0 + p.kb_per_split) - kb0;
        for (int kb = 0; kb < n_kb; ++kb) {
          const uint32_t tmem_acc = tmem_base + (buf * kAcc + (kb % kAcc)) * BN;
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 201, stage);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(ring + stage * stride);
          const uint64_t adesc = make_smem_desc(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc(sa + p.a_bytes, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_ss(tmem_acc, adesc + k * 2, bdesc + k * 2, idesc, (kb >= kAcc || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[buf]);
        if (++buf == 2) { buf = 0; tphase ^= 1; }
      }
    }
  } else {
    const int quad = warp & 3;
    int buf = 0;
    uint32_t tphase = 0;
    bool ok = true;
    const bool out_f32 = (p.flags & kOutF32) != 0;
    for (int t = blockIdx.x; t < num_work && ok; t += gridDim.x) {
      ok = mbar_wait(&tfull_bar[buf], tphase, abort_flag, p.status, 300, buf);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int m0 = (t % p.tiles_m) * BM;
      const int u = t / p.tiles_m;
      const int n0 = (u / p.splits) * BN;
      const int split = u % p.splits;
      const int row = m0 + quad * 32 + lane;
      const int kb0 = split * p.kb_per_split;
      const int n_kb = min(k_blocks, kb0 + p.kb_per_split) - kb0;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * kAcc * BN;
      const int n_acc = n_kb < kAcc ? n_kb : kAcc;  // accumulators that were written for this piece of work
      // warps whose 32 rows are all beyond M still take part in the barrier protocol but skip the loads
      const bool warp_has_rows = m0 + quad * 32 < p.M;
#pragma unroll 1
      for (int c = 0; c < BN && warp_has_rows; c += 32) {
        float v[32];
        {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        }
        for (int a = 1; a < n_acc; ++a) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + a * BN + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(r[j]);
        }
        const int col0 = n0 + c;
        if (p.splits > 1) {
          // partial sum of this K split: raw fp32 to the workspace slab (N is a multiple of 4 on this path)
          if (row < p.M && col0 < p.N) {
            float* wp = p.ws + (static_cast<size_t>(split) * p.M + row) * p.N + col0;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (col0 + 4 * q < p.N) reinterpret_cast<float4*>(wp)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
          continue;
        }
        if (row < p.M && col0 < p.N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
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
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += __bfloat162float(rr[j]);
          }
          if (out_f32) {
            float* cp = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            if (full && (p.ldc & 3) == 0) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                reinterpret_cast<float4*>(cp)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) cp[j] = v[j];
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            if (full && (p.ldc & 7) == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
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
                if (col0 + j < p.N) cp[j] = __float2bfloat16(v[j]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      if (++buf == 2) { buf = 0; tphase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

// out[m, n] = type(alpha * sum_s ws[s, m, n] + bias[n] + residual[m, n]); four columns per thread, slabs summed in order.
__global__ void splitk_finalize_kernel(const float* __restrict__ ws, int splits, int M, int N, float alpha, int flags, const void* bias,
                                       const __nv_bfloat16* residual, int ldr, void* C, int ldc) {
  const int n4 = N >> 2;
  const long long total = static_cast<long long>(M) * n4;
  const size_t slab = static_cast<size_t>(M) * N;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / n4);
    const int n = static_cast<int>(i - static_cast<long long>(m) * n4) * 4;
    const float* wp = ws + static_cast<size_t>(m) * N + n;
    float4 acc = *reinterpret_cast<const float4*>(wp);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(wp + s * slab);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float o[4] = {acc.x * alpha, acc.y * alpha, acc.z * alpha, acc.w * alpha};
    if (flags & kBias) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] += (flags & kBiasF32) ? reinterpret_cast<const float*>(bias)[n + j] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n + j]);
    }
    if (flags & kResidual) {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] += __bfloat162float(residual[static_cast<size_t>(m) * ldr + n + j]);
    }
    if (flags & kOutF32) {
      float* cp = reinterpret_cast<float*>(C) + static_cast<size_t>(m) * ldc + n;
#pragma unroll
      for (int j = 0; j < 4; ++j) cp[j] = o[j];
    } else {
      __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(C) + static_cast<size_t>(m) * ldc + n;
#pragma unroll
      for (int j = 0; j < 4; ++j) cp[j] = __float2bfloat16(o[j]);
    }
  }
}

template <int BN, int kAcc>
int launch(const void* A, const void* B, Params p, int lda, int ldb, cudaStream_t stream) {
  constexpr int kBBytes = BN * BK * 2;
  p.tiles_m = (p.M + BM - 1) / BM;
  const int a_rows = p.tiles_m > 1 ? BM : ((p.M + 7) / 8) * 8;  // rows past M in the last block are zero-filled by TMA
  p.a_bytes = a_rows * BK * 2;
  const int stride = p.a_bytes + kBBytes;
  int stages = kSmemBudget / stride;
  if (stages > kMaxStages) stages = kMaxStages;
  const int k_blocks = (p.K + BK - 1) / BK;
  if (p.splits > k_blocks) p.splits = k_blocks;
  p.kb_per_split = (k_blocks + p.splits - 1) / p.splits;
  p.splits = (k_blocks + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  if (stages > k_blocks + 1) stages = k_blocks + 1;
  if (stages < 2) stages = 2;
  p.stages = stages;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int smem_bytes = 1024 /*alignment*/ + 1024 /*barriers*/ + stages * stride + BM * BK * 2 /*slack read by the MMA*/;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d_bf16(&tmA, A, p.M, p.K, lda, a_rows, BK);
  if (rc != kErrOk) return rc;
  rc = make_tmap_2d_bf16(&tmB, B, p.N, p.K, ldb, BN, BK);
  if (rc != kErrOk) return rc;
  auto kern = gemm_skinny_kernel<BN, kAcc>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448) != cudaSuccess) return kErrCuda;
    attr_set = true;
  }
  const int work = p.tiles_n * p.splits * p.tiles_m;
  const int grid = work < num_sms() ? work : num_sms();
  kern<<<grid, kThreads, smem_bytes, stream>>>(tmA, tmB, p);
  if (cudaGetLastError() != cudaSuccess) return kErrCuda;
  if (p.splits > 1) {
    const long long total = static_cast<long long>(p.M) * (p.N / 4);
    const int blocks = static_cast<int>((total + 255) / 256 < 4LL * num_sms() ? (total + 255) / 256 : 4LL * num_sms());
    splitk_finalize_kernel<<<blocks, 256, 0, stream>>>(p.ws, p.splits, p.M, p.N, p.alpha, p.flags, p.bias, p.residual, p.ldr, p.C, p.ldc);
    if (cudaGetLastError() != cudaSuccess) return kErrCuda;
  }
  return kErrOk;
}

}  // namespace skinny

int launch_splitk_finalize(const float* ws, int splits, int M, int N, float alpha, int flags, const void* bias, const void* residual,
                           int ldr, void* C, int ldc, cudaStream_t stream) {
  const long long total = static_cast<long long>(M) * (N / 4);
  const int blocks = static_cast<int>((total + 255) / 256 < 4LL * num_sms() ? (total + 255) / 256 : 4LL * num_sms());
  skinny::splitk_finalize_kernel<<<blocks, 256, 0, stream>>>(ws, splits, M, N, alpha, flags, bias,
                                                             reinterpret_cast<const __nv_bfloat16*>(residual), ldr, C, ldc);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
}  // namespace lvb

// Bytes of fp32 workspace lvb_gemm_skinny may use for an [M, N] product (the most splits it ever picks is 8).
extern "C" long long lvb_gemm_skinny_workspace_bytes(int M, int N) { return 8LL * M * N * 4; }

// C[M,N] = alpha * A[M,K] B[N,K]^T (+ bias) (+ residual) for M <= 512.  flags: 1 = fp32 output, 4 = bias, 16 = bias is fp32,
// 8 = residual (bf16 [M, N], row stride ldr).  bn: tile width (32, 64 or 128), or 0 to let the launcher choose.
// splits: CTAs per column tile along K, or 0 to let the launcher choose; more than one needs `workspace`
// (lvb_gemm_skinny_workspace_bytes(M, N) bytes of device memory, contents irrelevant) and N % 4 == 0, else 1 is used.
extern "C" int lvb_gemm_skinny(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int flags,
                               float alpha, const void* bias, const void* residual, int ldr, int bn, int splits, void* workspace,
                               int* status, void* stream) {
  using namespace lvb;
  using namespace lvb::skinny;
  if (M <= 0 || M > 4 * BM || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7) || splits < 0 || splits > 8) return kErrBadArg;
  Params p;
  p.C = C; p.bias = bias; p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr;
  p.flags = flags; p.alpha = alpha; p.status = status;
  p.ws = reinterpret_cast<float*>(workspace);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 0) bn = (N >= 96) ? 128 : (N > 32) ? 64 : 32;
  if (splits == 0) {
    // enough (tile, split) pairs for about one per SM, but keep at least ~12 k-blocks per CTA (the fixed cost of a CTA is
    // worth about 25 k-blocks)
    const int tiles = ((N + bn - 1) / bn) * ((M + BM - 1) / BM);
    const int k_blocks = (K + BK - 1) / BK;
    splits = num_sms() / tiles;
    if (splits > k_blocks / 12) splits = k_blocks / 12;
    if (splits > 8) splits = 8;
    if (splits < 1) splits = 1;
  }
  if (workspace == nullptr || (N & 3)) splits = 1;
  p.splits = splits;
  if (bn == 128) return skinny::launch<128, 2>(A, B, p, lda, ldb, s);
  if (bn == 64) return skinny::launch<64, 4>(A, B, p, lda, ldb, s);
  if (bn == 32) return skinny::launch<32, 8>(A, B, p, lda, ldb, s);
  return kErrBadArg;
}
