"""Basic modules: Linear, Embedding, RmsNorm, LayerNorm, Dropout.

These replace the Haliax ``hnn`` modules the reference is built from.  Weights are kept as plain 2-D
``[out, in]`` matrices (what the tcgen05 GEMM consumes).  Each parameter carries the metadata needed to write
it in the reference's checkpoint layout:

``lev_shape``        the articulated shape, e.g. ``(kv_head, q_per_group, head_size, embed)``
``lev_transposed``   True when the reference stores ``[in..., out...]`` (``out_first=False``, GPT-2 style)
``tp_dim``           which local dim is tensor-parallel sharded (None when replicated)

Class names matter: the default weight-decay mask excludes parameters whose class-qualified path contains
``LayerNorm``, ``RmsNorm`` or ``Embedding`` (src/levanter/optim/config.py:149-161).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def _prod(xs: Sequence[int]) -> int:
    out = 1
    for x in xs:
        out *= int(x)
    return out


def trunc_normal_(t: torch.Tensor, std: float) -> torch.Tensor:
    with torch.no_grad():
        return nn.init.trunc_normal_(t, mean=0.0, std=std, a=-3 * std, b=3 * std)


class Linear(nn.Module):
    """``y = x W^T + b`` with ``W`` stored ``[out, in]``; bf16 CUDA inputs run on the tcgen05 GEMM."""

    def __init__(self, in_features: int, out_features: int, *, bias: bool = False, init_std: Optional[float] = None,
                 lev_out: Optional[Tuple[int, ...]] = None, lev_in: Optional[Tuple[int, ...]] = None,
                 out_first: bool = True, parallel=None, device=None, dtype=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        std = init_std if init_std is not None else 1.0 / math.sqrt(in_features)
        if self.weight.device.type != "meta":
            trunc_normal_(self.weight, std)
        lev_out = tuple(lev_out) if lev_out is not None else (out_features,)
        lev_in = tuple(lev_in) if lev_in is not None else (in_features,)
        assert _prod(lev_out) == out_features and _prod(lev_in) == in_features
        self.weight.lev_shape = (lev_out + lev_in) if out_first else (lev_in + lev_out)
        self.weight.lev_transposed = not out_first
        kind = parallel[0] if parallel is not None and parallel[1] is not None and parallel[1].size > 1 else None
        self.weight.tp_dim = {None: None, "column": 0, "row": 1}[kind]
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype))
            self.bias.lev_shape = lev_out
            self.bias.lev_transposed = False
            self.bias.tp_dim = 0 if kind == "column" else None
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor, *, skip_bias: bool = False) -> torch.Tensor:
        from .ops.gemm import linear

        b = None if skip_bias else self.bias
        w = self.weight
        if w.dtype != x.dtype:
            w = w.to(x.dtype)
            b = b.to(x.dtype) if b is not None else None
        return linear(x, w, b)

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


class Embedding(nn.Module):
    """Token embedding ``weight[vocab, embed]`` with ``unembed`` for tied LM heads."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, init_std: float = 0.02, device=None, dtype=None):
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim, device=device, dtype=dtype))
        if self.weight.device.type != "meta":
            trunc_normal_(self.weight, init_std)
        self.weight.lev_shape = (num_embeddings, embedding_dim)
        self.weight.lev_transposed = False
        self.weight.tp_dim = None

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        from .ops.embedding import embedding

        return embedding(ids, self.weight)

    embed = forward

    def unembed(self, x: torch.Tensor) -> torch.Tensor:
        from .ops.gemm import linear

        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)
        return linear(x, w, None)

    def resize_embeddings(self, new_size: int, init_std: float = 0.02) -> "Embedding":
        """Return a copy with ``new_size`` rows; new rows are freshly initialised."""
        new = Embedding(new_size, self.embedding_dim, init_std=init_std, device=self.weight.device, dtype=self.weight.dtype)
        n = min(new_size, self.num_embeddings)
        with torch.no_grad():
            new.weight[:n].copy_(self.weight[:n])
        return new


class RmsNorm(nn.Module):
    """``x * rsqrt(mean(x^2) + eps) * weight (+ bias)`` computed in fp32."""

    def __init__(self, dim: int, eps: float = 1e-6, use_weight: bool = True, use_bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.dim = dim
        self.eps = eps
        if use_weight:
            self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
            self.weight.lev_shape = (dim,)
        else:
            self.register_parameter("weight", None)
        if use_bias:
            self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))
            self.bias.lev_shape = (dim,)
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .ops.norm import rms_norm

        return rms_norm(x, self.weight, self.bias, self.eps)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, use_weight: bool = True, use_bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.dim = dim
        self.eps = eps
        if use_weight:
            self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
            self.weight.lev_shape = (dim,)
        else:
            self.register_parameter("weight", None)
        if use_bias:
            self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))
            self.bias.lev_shape = (dim,)
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .ops.norm import layer_norm

        return layer_norm(x, self.weight, self.bias, self.eps)


class Dropout(nn.Module):
    """Dropout that is inert at ``p == 0`` or in eval mode (all shipped configs use ``p = 0``)."""

    def __init__(self, p: float = 0.0):
        super().__init__()
        self.p = p

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.p == 0.0 or not self.training:
            return x
        from .ops.dropout import dropout

        return dropout(x, self.p, training=True)
