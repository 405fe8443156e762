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
