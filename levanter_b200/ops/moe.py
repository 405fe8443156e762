"""Grouped (per-expert) SwiGLU MLP over rows sorted by expert: the reference's three ``hnn.MoELinear`` ragged dots
(src/levanter/models/mixtral.py:245-277).

Rows ``[sum(group_sizes), hidden]`` are contiguous per expert.  Each expert's slice runs through the tcgen05 GEMM
(gate and up projections, the gated-activation kernel, then the down projection); expert boundaries are read back once
per call."""
from __future__ import annotations

import torch

from ..utils.activation import ActivationFunctionEnum
from .gemm import linear
from .glu import gated_activation


def grouped_mlp(x_sorted: torch.Tensor, group_sizes: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor,
                act: ActivationFunctionEnum, first_expert: int = 0) -> torch.Tensor:
    """``out[rows of expert e] = (act(x w1[e]^T) * (x w3[e]^T)) w2[e]^T``; ``w1/w3: [E, mlp, hidden]``, ``w2: [E, hidden, mlp]``.
    ``group_sizes`` covers the experts held in ``w*`` starting at global expert ``first_expert``."""
    sizes = group_sizes.tolist()
    n_local = w1.shape[0]
    sizes = sizes[first_expert:first_expert + n_local] if len(sizes) != n_local else sizes
    outs = []
    start = 0
    dt = x_sorted.dtype
    for e, n in enumerate(sizes):
        if n == 0:
            continue
        xe = x_sorted[start:start + n]
        a, b, c = w1[e], w3[e], w2[e]
        if a.dtype != dt:
            a, b, c = a.to(dt), b.to(dt), c.to(dt)
        h = gated_activation(linear(xe, a), linear(xe, b), act)
        outs.append(linear(h, c))
        start += n
    if not outs:
        return x_sorted.new_zeros((0, w2.shape[1]))
    return torch.cat(outs, dim=0)
