// Expert-parallel token exchange over peer memory: the router's permutation and the all-to-all in one kernel per direction.
//
// Every rank holds E / W experts.  The (token, choice) pairs of a rank, sorted by global expert, have to reach the ranks
// that own those experts and arrive there grouped by expert, each expert's segment padded to a multiple of 128 rows (the
// layout the grouped tcgen05 GEMM consumes).  With a collective library this is a count exchange, a host read-back of the
// split sizes, an all-to-all of rows and a regrouping copy per direction.  Here:
//
//   1. `counts_push` writes this rank's per-expert counts into row `rank` of every peer's [W, E] table (an all-gather of
//      W * E integers by plain peer stores).
//   2. After a barrier every rank derives, on the device, where each of its rows goes: the padded start of the expert on the
//      owning rank plus the rows that lower ranks send to the same expert plus the row's position among this rank's rows
//      for that expert.  `rows_kernel<PUSH>` gathers the rows through the sort permutation and stores them straight into the
//      owner's buffer (16-byte peer stores, one warp per row); the owner's block 0 also writes the expert offsets and the
//      expert of every 128-row block for the grouped GEMM and clears the padding rows.  Nothing is read back by the host.
//   3. `rows_kernel<PULL>` is the way back: every rank loads its rows from the owners' buffers at the same positions and
//      scatters them into (token, choice) order.  The backward pass uses the same two kernels with the roles swapped.
//
// Capacity is bounded: a row whose position is past `cap` is dropped (pulled back as zeros) and the bounds code is left in
// the status word.  Loads and stores of peer memory are plain global accesses (no multicast qualifier anywhere).
// The reference framework has no expert parallelism (its MoE permutes within a data shard,
// src/levanter/models/mixtral.py:374-415); this is the distributed form of that permutation.
#include "common.cuh"

namespace lvb {
namespace ep {

constexpr int kMaxWorld = 16;
constexpr int kMaxExperts = 64;
constexpr int kBlock = 256;
constexpr int kPad = 128;

struct Peers {
  void* p[kMaxWorld];
};

__global__ void counts_push_kernel(const int* __restrict__ counts, Peers tables, int W, int rank, int E) {
  for (int i = threadIdx.x; i < W * E; i += blockDim.x) {
    const int r = i / E, e = i - r * E;
    static_cast<int*>(tables.p[r])[rank * E + e] = counts[e];
  }
}

__device__ __forceinline__ int round_up_pad(int n) { return (n + kPad - 1) / kPad * kPad; }

struct Plan {
  int send_base[kMaxExperts];     // row on the owning rank where this rank's first row for the expert goes
  int my_start[kMaxExperts + 1];  // first sorted row of this rank for the expert
  int loc_off[kMaxExperts + 1];   // padded start of every local expert in this rank's buffer
  int loc_tot[kMaxExperts];       // rows every local expert receives
};

__device__ __forceinline__ void build_plan(Plan& s, const int* __restrict__ table, int W, int rank, int E) {
  const int n_local = E / W;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / n_local;
    int base = 0;
    for (int e2 = d * n_local; e2 < e; ++e2) {
      int tot = 0;
      for (int r = 0; r < W; ++r) tot += table[r * E + e2];
      base += round_up_pad(tot);
    }
    for (int r = 0; r < rank; ++r) base += table[r * E + e];
    s.send_base[e] = base;
    int start = 0;
    for (int e2 = 0; e2 < e; ++e2) start += table[rank * E + e2];
    s.my_start[e] = start;
    if (e == E - 1) s.my_start[E] = start + table[rank * E + e];
  }
  for (int le = threadIdx.x; le < n_local; le += blockDim.x) {
    int off = 0, tot = 0;
    for (int l2 = 0; l2 <= le; ++l2) {
      tot = 0;
      for (int r = 0; r < W; ++r) tot += table[r * E + rank * n_local + l2];
      if (l2 < le) off += round_up_pad(tot);
    }
    s.loc_off[le] = off;
    s.loc_tot[le] = tot;
    if (le == n_local - 1) s.loc_off[n_local] = off + round_up_pad(tot);
  }
  __syncthreads();
}

// PUSH: row i of this rank's expert-sorted order, taken from local[index[i] / div] (or local[i]), is stored at its
// position in the owner's buffer.  PULL: the row at that position in the owner's buffer is loaded into
// local[index[i] / div] (or local[i]).  R = rows of this rank; H8 = row length in 16-byte units.
template <bool PUSH>
__global__ void __launch_bounds__(kBlock)
rows_kernel(const int* __restrict__ table, int W, int rank, int E, uint4* __restrict__ local, const long long* __restrict__ index,
            int div, Peers peers, int H8, int R, int cap, int* __restrict__ offsets_out, int* __restrict__ tile_group_out,
            int clear_padding, int* __restrict__ status) {
  __shared__ Plan s;
  build_plan(s, table, W, rank, E);
  const int n_local = E / W;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarps = kBlock / 32;

  if (PUSH && blockIdx.x == 0 && offsets_out != nullptr) {
    for (int le = threadIdx.x; le <= n_local; le += kBlock) offsets_out[le] = min(s.loc_off[le], cap);  // never past the buffer
    for (int b = threadIdx.x; b < cap / kPad; b += kBlock) {
      int grp = -1;
      for (int le = 0; le < n_local; ++le)
        if (b * kPad >= s.loc_off[le] && b * kPad < s.loc_off[le + 1]) grp = le;
      tile_group_out[b] = grp;
    }
    if (threadIdx.x == 0 && s.loc_off[n_local] > cap) record_status(status, 4, 30, s.loc_off[n_local]);
  }
  if (PUSH && clear_padding) {
    // rows between an expert's last received row and the end of its padded segment belong to this rank alone
    uint4* mine = static_cast<uint4*>(peers.p[rank]);
    for (int v = blockIdx.x * kWarps + warp; v < n_local * kPad; v += gridDim.x * kWarps) {
      const int le = v / kPad;
      const int row = s.loc_off[le] + s.loc_tot[le] + (v - le * kPad);
      if (row < s.loc_off[le + 1] && row < cap)
        for (int c = lane; c < H8; c += 32) mine[static_cast<size_t>(row) * H8 + c] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  for (int i = blockIdx.x * kWarps + warp; i < R; i += gridDim.x * kWarps) {
    int e = 0;
    while (e < E - 1 && s.my_start[e + 1] <= i) ++e;
    const int row = s.send_base[e] + (i - s.my_start[e]);
    const long long li = index != nullptr ? index[i] / div : i;
    uint4* loc = local + static_cast<size_t>(li) * H8;
    if (row >= cap) {
      if (lane == 0) record_status(status, 4, PUSH ? 31 : 32, row);
      if (!PUSH)
        for (int c = lane; c < H8; c += 32) loc[c] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    uint4* rem = static_cast<uint4*>(peers.p[e / n_local]) + static_cast<size_t>(row) * H8;
    if (PUSH) {
      for (int c = lane; c < H8; c += 32) rem[c] = __ldg(reinterpret_cast<const uint4*>(loc) + c);
    } else {
      for (int c = lane; c < H8; c += 32) loc[c] = __ldcg(reinterpret_cast<const uint4*>(rem) + c);
    }
  }
}

inline int fill_peers(Peers& out, void* const* host_ptrs, int W) {
  if (W < 1 || W > kMaxWorld) return kErrBadArg;
  for (int r = 0; r < kMaxWorld; ++r) out.p[r] = r < W ? host_ptrs[r] : nullptr;
  return kErrOk;
}

}  // namespace ep
}  // namespace lvb

using namespace lvb;

// counts: int32 [E] on this device; tables: W device addresses (a host array) of every rank's int32 [W, E] table.
extern "C" int lvb_ep_counts_push(const int* counts, void* const* tables, int W, int rank, int E, void* stream) {
  ep::Peers t;
  if (ep::fill_peers(t, tables, W) != kErrOk || E < W || E % W != 0 || E > ep::kMaxExperts || rank < 0 || rank >= W) return kErrBadArg;
  ep::counts_push_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, t, W, rank, E);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}

// push != 0: local rows -> owners' buffers (offsets_out [E / W + 1] and tile_group_out [cap / 128] may be null);
// push == 0: owners' buffers -> local rows.  `table` is this rank's complete [W, E] table, `bufs` the W addresses of the
// ranks' exchange buffers ([cap, H] 16-bit elements), H a multiple of 8, cap a multiple of 128.
extern "C" int lvb_ep_rows(int push, const int* table, int W, int rank, int E, void* local, const long long* index, int div,
                           void* const* bufs, int H, int R, int cap, int* offsets_out, int* tile_group_out, int clear_padding,
                           int* status, void* stream) {
  ep::Peers b;
  if (ep::fill_peers(b, bufs, W) != kErrOk || E < W || E % W != 0 || E > ep::kMaxExperts || rank < 0 || rank >= W || H <= 0 ||
      H % 8 != 0 || cap <= 0 || cap % ep::kPad != 0 || R < 0 || div < 1)
    return kErrBadArg;
  const int warps = ep::kBlock / 32;
  int grid = (R + warps - 1) / warps;
  grid = grid < 1 ? 1 : (grid > 148 * 4 ? 148 * 4 : grid);
  auto s = static_cast<cudaStream_t>(stream);
  if (push)
    ep::rows_kernel<true><<<grid, ep::kBlock, 0, s>>>(table, W, rank, E, static_cast<uint4*>(local), index, div, b, H / 8, R, cap,
                                                      offsets_out, tile_group_out, clear_padding, status);
  else
    ep::rows_kernel<false><<<grid, ep::kBlock, 0, s>>>(table, W, rank, E, static_cast<uint4*>(local), index, div, b, H / 8, R, cap,
                                                       nullptr, nullptr, 0, status);
  return cudaGetLastError() == cudaSuccess ? kErrOk : kErrCuda;
}
