"""Gradient accumulation over micro-batches (src/levanter/grad_accum.py:36-155).

``microbatched(fn, microbatch_size)`` turns a ``(loss, grads)`` function of a batch into one that splits the batch
into ``AccumStep x Microbatch`` slices, runs them in sequence and reduces losses and gradients by MEAN (default) or
SUM.  The trainer's hot path does the same accumulation without materialising per-micro-batch gradient trees: the GEMM
epilogues add ``dW`` straight into the engine's fp32 buffer."""
from __future__ import annotations

import enum
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


class ReductionType(enum.Enum):
    SUM = enum.auto()
    MEAN = enum.auto()


def microbatch_slices(batch_size: int, microbatch_size: Optional[int]) -> List[Tuple[int, int]]:
    if microbatch_size is None or microbatch_size <= 0 or microbatch_size >= batch_size:
        return [(0, batch_size)]
    if batch_size % microbatch_size != 0:
        raise ValueError(f"Bad value for microbatch_size: {batch_size} % {microbatch_size} != 0")
    return [(i, i + microbatch_size) for i in range(0, batch_size, microbatch_size)]


def _slice_tree(x, a: int, b: int):
    if hasattr(x, "slice") and not isinstance(x, torch.Tensor):
        return x.slice(a, b)
    if isinstance(x, torch.Tensor):
        return x[a:b]
    if isinstance(x, tuple):
        return tuple(_slice_tree(v, a, b) for v in x)
    if isinstance(x, list):
        return [_slice_tree(v, a, b) for v in x]
    if isinstance(x, dict):
        return {k: _slice_tree(v, a, b) for k, v in x.items()}
    return x


def _batch_size_of(x) -> int:
    if hasattr(x, "tokens"):
        return x.tokens.shape[0]
    if isinstance(x, torch.Tensor):
        return x.shape[0]
    if isinstance(x, (tuple, list)):
        return _batch_size_of(x[0])
    if isinstance(x, dict):
        return _batch_size_of(next(iter(x.values())))
    raise TypeError(type(x))


def microbatched(fn: Callable[..., Tuple[torch.Tensor, Dict[str, torch.Tensor]]], microbatch_size: Optional[int],
                 reduce: ReductionType = ReductionType.MEAN, accum_dtype: Optional[torch.dtype] = torch.float32):
    """Wrap ``fn(batch, *args) -> (loss, grads_tree)`` to run over micro-batches and reduce.

    Every micro-batch contributes with equal weight under MEAN regardless of how many unmasked tokens it has
    (src/levanter/grad_accum.py:133-134)."""

    def wrapped(batch, *args, **kwargs):
        n = _batch_size_of(batch)
        slices = microbatch_slices(n, microbatch_size)
        tot_loss = None
        tot_grads: Dict[str, torch.Tensor] = {}
        for a, b in slices:
            loss, grads = fn(_slice_tree(batch, a, b), *args, **kwargs)
            tot_loss = loss.detach().clone() if tot_loss is None else tot_loss + loss.detach()
            for k, g in grads.items():
                if g is None:
                    continue
                g = g.to(accum_dtype) if accum_dtype is not None else g
                if k in tot_grads:
                    tot_grads[k] += g
                else:
                    tot_grads[k] = g.clone()
        if reduce == ReductionType.MEAN and len(slices) > 1:
            tot_loss = tot_loss / len(slices)
            for k in tot_grads:
                tot_grads[k] /= len(slices)
        return tot_loss, tot_grads

    return wrapped
