"""Tensor-parallel regions (Megatron style) over the mesh's ``model`` axis.

The reference gets TP from axis names (``tensor_parallel_axes: [mlp, heads]`` mapped to the ``model`` mesh axis,
src/levanter/trainer.py:677,851-855) and lets XLA insert the collectives.  Here the column-parallel side (q/k/v,
gate/up) needs no forward communication and an all-reduce of the input gradient; the row-parallel side (o_proj,
down_proj) all-reduces its forward output.  This NCCL path is the baseline and oracle; ``parallel.fused`` supplies the
kernels that overlap these collectives with the GEMMs."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class _CopyToRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class TensorParallel:
    def __init__(self, group: Optional[dist.ProcessGroup], size: int, rank: int):
        self.group = group
        self.size = size
        self.rank = rank

    @staticmethod
    def from_mesh(mesh) -> Optional["TensorParallel"]:
        ax = mesh.axes["model"]
        if ax.size <= 1:
            return None
        return TensorParallel(ax.group, ax.size, ax.rank)

    def copy_to_region(self, x: torch.Tensor) -> torch.Tensor:
        return _CopyToRegion.apply(x, self.group)

    def reduce_from_region(self, x: torch.Tensor) -> torch.Tensor:
        return _ReduceFromRegion.apply(x, self.group)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather_last_dim(self, x: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


def shard_full_state_(model: torch.nn.Module, full_state: dict, tp: Optional["TensorParallel"]) -> None:
    """Fill a tensor-parallel ``model`` from the tensors of the unsharded model: every parameter marked ``tp_dim`` takes
    this rank's slice along that dimension (heads and MLP columns are contiguous per rank), the others are copied whole.
    Used to serve (or continue training) a checkpoint on a model axis of any size."""
    rank = tp.rank if tp is not None else 0
    with torch.no_grad():
        for name, p in model.named_parameters():
            src = full_state[name]
            dim = getattr(p, "tp_dim", None)
            if dim is not None and src.shape != p.shape:
                n = p.shape[dim]
                src = src.narrow(dim, rank * n, n)
            if src.shape != p.shape:
                raise ValueError(f"{name}: cannot place {tuple(full_state[name].shape)} into {tuple(p.shape)} (tp_dim={dim})")
            p.copy_(src.to(p.dtype))
