"""Expert parallelism: experts are sliced over a process group and tokens travel to their experts and back by all-to-all.

The reference's MoE is shard-local (no token exchange, src/levanter/models/mixtral.py:343-347); this is the distributed form
of the same routing.  After the router has sorted the ``T * k`` (token, choice) rows by expert, rows bound for rank ``r``'s
experts are contiguous, so dispatch is one ``all_to_all_single`` with split sizes taken from the per-expert counts (themselves
exchanged first: ``[ranks, local experts]`` int64), the experts run the grouped MLP on what they received regrouped by local
expert, and combine is the mirrored all-to-all followed by the inverse permutation.  Both exchanges are autograd functions
whose backward is the opposite exchange."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class ExpertParallel:
    """The process group experts are sliced over (``size`` ranks; this one is ``rank``)."""

    def __init__(self, group=None):
        self.group = group
        ok = dist.is_available() and dist.is_initialized()
        self.size = dist.get_world_size(group) if ok else 1
        self.rank = dist.get_rank(group) if ok else 0

    def peer_exchange(self, num_experts: int, hidden: int, rows_per_rank: int, dtype, capacity_factor: float = 2.0):
        """The exchange on this library's peer-memory kernels, shared by every layer that asks with the same shapes (a
        collective call the first time: all ranks allocate and exchange their buffers).  ``None`` where it cannot be used:
        no CUDA, one rank, 32-bit activations, or ``LEVANTER_B200_EP_COMM=nccl``."""
        import os

        from .symm import p2p_available

        if os.environ.get("LEVANTER_B200_EP_COMM", "peer") == "nccl" or dtype not in (torch.bfloat16, torch.float16):
            return None
        if hidden % 8 != 0 or num_experts > 64 or not p2p_available(self.group):
            return None
        cache = self.__dict__.setdefault("_exchanges", {})
        key = (num_experts, hidden, rows_per_rank, dtype, capacity_factor)
        if key not in cache:
            cache[key] = PeerExchange(self, num_experts, hidden, rows_per_rank, dtype, capacity_factor)
        return cache[key]

    @staticmethod
    def from_mesh(mesh) -> Optional["ExpertParallel"]:
        """Experts are sliced over the data axis (each data-parallel rank holds ``E / data_size`` experts)."""
        if mesh is None or mesh.data_size <= 1:
            return None
        return ExpertParallel(mesh.data_group)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, in_splits: List[int], out_splits: List[int], group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits, group=ctx.group)
        return out, None, None, None


def all_to_all(x: torch.Tensor, in_splits: List[int], out_splits: List[int], group) -> torch.Tensor:
    return _AllToAll.apply(x, in_splits, out_splits, group)


def dispatch_combine(ep: ExpertParallel, x_flat: torch.Tensor, sort_idx: torch.Tensor, group_sizes: torch.Tensor, k: int, experts) -> torch.Tensor:
    """Route ``x_flat[T, H]`` through the sharded ``experts`` and return ``[T * k, H]`` in (token, choice) order.

    ``sort_idx`` is the stable argsort of the flattened expert choices, ``group_sizes[E]`` the rows per global expert."""
    W = ep.size
    E = group_sizes.numel()
    n_local = E // W
    x_sorted = x_flat.index_select(0, sort_idx // k)  # rows grouped by global expert, hence by destination rank
    # counts[r, e]: rows this rank sends to local expert e of rank r; recv[r, e]: rows rank r sends to my local expert e
    counts = group_sizes.reshape(W, n_local).to(torch.int64).contiguous()
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts, group=ep.group)
    counts_h, recv_h = counts.cpu(), recv.cpu()  # split sizes are host integers: one small sync per layer
    in_splits = counts_h.sum(1).tolist()
    out_splits = recv_h.sum(1).tolist()
    got = all_to_all(x_sorted, in_splits, out_splits, ep.group)  # grouped by source rank, then by local expert
    # regroup by local expert: rows of expert e from all sources become contiguous
    n_got = got.shape[0]
    seg_expert = torch.arange(n_local).repeat(W)  # expert of each (source, expert) segment, in arrival order
    seg_len = recv_h.reshape(-1)
    order = torch.argsort(torch.repeat_interleave(seg_expert, seg_len), stable=True).to(got.device)
    by_expert = got.index_select(0, order)
    local_sizes = recv_h.sum(0).to(group_sizes.device)
    out_by_expert = experts(by_expert, local_sizes)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(n_got, device=order.device)
    back = all_to_all(out_by_expert.index_select(0, inv), out_splits, in_splits, ep.group)  # rows return in sorted order
    unsort = torch.empty_like(sort_idx)
    unsort[sort_idx] = torch.arange(sort_idx.numel(), device=sort_idx.device)
    return back.index_select(0, unsort)


# ------------------------------------------------------------------------------------------------ exchange over peer memory
class PeerExchange:
    """Dispatch/combine on this library's own kernels over symmetric memory (``ops/csrc/ep_dispatch.cu``) instead of a
    collective library: the count all-gather, the permutation into the owners' padded expert-sorted buffers and the way back
    are peer loads and stores issued by the kernels, and nothing is read back by the host.

    One exchange buffer of ``capacity`` rows and one ``[ranks, E]`` count table per rank are shared by every MoE layer (the
    layers run one after the other).  Every exchange starts with a barrier (all ranks are done with the buffer's previous
    contents) and has one more between writing and reading it.  Rows beyond ``capacity`` are dropped and reported through
    the kernel status word; ``capacity_factor`` is relative to a balanced load (``T * k`` rows per rank)."""

    def __init__(self, ep: ExpertParallel, num_experts: int, hidden: int, rows_per_rank: int, dtype=torch.bfloat16,
                 capacity_factor: float = 2.0, device=None):
        from ..ops.ep_dispatch import capacity_rows
        from .symm import SymmetricBuffer

        assert num_experts % ep.size == 0
        self.ep, self.E, self.H = ep, num_experts, hidden
        self.n_local = num_experts // ep.size
        self.rows_per_rank = rows_per_rank
        self.cap = capacity_rows(rows_per_rank, self.n_local, capacity_factor)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.buf = SymmetricBuffer(self.cap * hidden, dtype, device, ep.group)
        self.table = SymmetricBuffer(ep.size * num_experts, torch.int32, device, ep.group)
        self.rows = self.buf.tensor.view(self.cap, hidden)

    def barrier(self):
        self.buf.barrier()


class _Plan:
    """What one layer call needs again in its combine and backward exchanges (the shared table is overwritten by then)."""

    def __init__(self, table, offsets, tile_group, sort_idx, k, num_rows):
        self.table, self.offsets, self.tile_group, self.sort_idx, self.k, self.num_rows = table, offsets, tile_group, sort_idx, k, num_rows


class _PeerDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_flat, counts, sort_idx, k, ex: PeerExchange, holder: list):
        from ..ops import ep_dispatch as K

        W, rank = ex.ep.size, ex.ep.rank
        R = sort_idx.numel()
        ex.barrier()  # every rank is done with the previous contents of the table and the buffer
        K.counts_push(counts, ex.table.c_ptrs, W, rank)
        ex.barrier()
        table = ex.table.tensor.clone()
        offsets = torch.empty(ex.n_local + 1, dtype=torch.int32, device=x_flat.device)
        tile_group = torch.empty(ex.cap // K.PAD, dtype=torch.int32, device=x_flat.device)
        K.rows(True, table, W, rank, x_flat.contiguous(), sort_idx, k, ex.buf.c_ptrs, R, ex.cap, offsets, tile_group, True)
        ex.barrier()
        plan = _Plan(table, offsets, tile_group, sort_idx, k, R)
        holder.append(plan)
        ctx.plan, ctx.ex, ctx.T = plan, ex, x_flat.shape[0]
        return ex.rows.clone()

    @staticmethod
    def backward(ctx, g_pad):
        from ..ops import ep_dispatch as K

        ex, plan = ctx.ex, ctx.plan
        ex.barrier()
        ex.rows.copy_(g_pad)
        ex.barrier()
        g_sorted = torch.empty(plan.num_rows, ex.H, dtype=g_pad.dtype, device=g_pad.device)
        K.rows(False, plan.table, ex.ep.size, ex.ep.rank, g_sorted, None, 1, ex.buf.c_ptrs, plan.num_rows, ex.cap)
        gx = torch.zeros(ctx.T, ex.H, dtype=torch.float32, device=g_pad.device)
        gx.index_add_(0, plan.sort_idx // plan.k, g_sorted.float())  # the k choices of a token add up
        return gx.to(g_pad.dtype), None, None, None, None, None


class _PeerCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_pad, ex: PeerExchange, plan: _Plan):
        from ..ops import ep_dispatch as K

        ex.barrier()
        ex.rows.copy_(y_pad)
        ex.barrier()
        out = torch.empty(plan.num_rows, ex.H, dtype=y_pad.dtype, device=y_pad.device)
        K.rows(False, plan.table, ex.ep.size, ex.ep.rank, out, plan.sort_idx, 1, ex.buf.c_ptrs, plan.num_rows, ex.cap)
        ctx.ex, ctx.plan = ex, plan
        return out  # (token, choice) order

    @staticmethod
    def backward(ctx, g_out):
        from ..ops import ep_dispatch as K

        ex, plan = ctx.ex, ctx.plan
        ex.barrier()
        K.rows(True, plan.table, ex.ep.size, ex.ep.rank, g_out.contiguous(), plan.sort_idx, 1, ex.buf.c_ptrs, plan.num_rows, ex.cap,
               None, None, True)
        ex.barrier()
        return ex.rows.clone(), None, None


def dispatch_combine_peer(ex: PeerExchange, x_flat: torch.Tensor, sort_idx: torch.Tensor, group_sizes: torch.Tensor, k: int,
                          experts) -> torch.Tensor:
    """Same contract as :func:`dispatch_combine`, on the peer-memory kernels.  ``experts`` holds the local ``w1, w3, w2`` and
    ``act``; the grouped GEMMs run directly on the padded layout that the dispatch kernel produced."""
    from ..ops.moe import grouped_mlp_on_padded

    assert sort_idx.numel() == ex.rows_per_rank, "the exchange buffer was sized for a different number of rows per rank"
    holder: list = []
    x_pad = _PeerDispatch.apply(x_flat, group_sizes.to(torch.int32).contiguous(), sort_idx.contiguous(), k, ex, holder)
    plan = holder[0]
    y_pad = grouped_mlp_on_padded(x_pad, plan.tile_group, plan.offsets, experts.w1, experts.w3, experts.w2, experts.act)
    return _PeerCombine.apply(y_pad, ex, plan)
