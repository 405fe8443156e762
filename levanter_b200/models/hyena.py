"""The Hyena operator: gated long convolutions with implicitly parametrised filters
(src/levanter/models/hyena.py:39-556; Poli et al. 2023).

The long convolution is a direct causal sum on this library's kernel for sequences up to 4096 (``ops/long_conv.py``) and an
FFT convolution in fp32 otherwise; the filter is generated once per call from
a small sine-activated MLP over positional features and is shared by every sequence of the batch.  Sequences may be split
into ``num_blocks`` independent blocks; filters are generated for one block only."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn import Dropout, Linear
from ..utils.activation import ActivationFunctionEnum


@dataclass(frozen=True)
class HyenaConfig:
    seq_len: int = 1024
    hidden_dim: int = 768
    num_heads: int = 1
    order: int = 2  # depth of the recurrence
    filter_order: int = 16  # width of the filter MLP
    short_filter_order: int = 3  # length of the explicit depthwise input filter
    outer_mixing: bool = False
    activation: ActivationFunctionEnum = ActivationFunctionEnum.gelu_new
    num_blocks: int = 1
    num_hidden_layers_filter_mlp: int = 2
    filter_emb_dim: int = 3  # 1 + 2 * bands positional features
    filter_dropout: float = 0.0
    fast_decay_pct: float = 0.3
    slow_decay_pct: float = 1.5
    target: float = 1e-2
    modulate: bool = True
    shift: float = 0.0
    resid_pdrop: float = 0.0
    use_bias: bool = True

    def __post_init__(self):
        if self.hidden_dim % self.num_heads:
            raise ValueError(f"hidden_dim {self.hidden_dim} must be divisible by num_heads {self.num_heads}")
        if self.seq_len % self.num_blocks:
            raise ValueError(f"seq_len {self.seq_len} must be divisible by num_blocks {self.num_blocks}")

    @property
    def head_size(self) -> int:
        return self.hidden_dim // self.num_heads

    @property
    def pos_per_block(self) -> int:
        return self.seq_len // self.num_blocks


class PositionalEmbedding(nn.Module):
    """Features ``[t, Re exp(-i f w), Im exp(-i f w)]`` of the positions of one block (fixed, not trained)."""

    def __init__(self, pos_per_block: int, emb_dim: int):
        super().__init__()
        if emb_dim <= 1:
            raise ValueError("emb_dim must be greater than 1")
        L = pos_per_block
        t = torch.linspace(0, 1, L)
        bands = (emb_dim - 1) // 2
        w = 2 * math.pi * torch.linspace(0, L - 1, L) / L
        f = torch.linspace(1e-4, bands - 1, bands)
        z = torch.exp(-1j * f[None, :] * w[:, None])
        self.register_buffer("z", torch.cat([t[:, None].expand(L, bands), z.real, z.imag], dim=1).contiguous(), persistent=False)
        self.register_buffer("t", t, persistent=False)
        self.pos_per_block = L

    def forward(self, L: int):
        if L > self.pos_per_block:
            raise ValueError(f"Requested length {L} > max size {self.pos_per_block}")
        return self.z[:L], self.t[:L]


class ExponentialModulation(nn.Module):
    """Per-channel exponential decay window ``exp(-t * |delta_c|) + shift`` applied to the generated filters."""

    def __init__(self, channels: int, fast_decay_pct: float, slow_decay_pct: float, target: float, modulate: bool, shift: float):
        super().__init__()
        max_decay = math.log(target) / fast_decay_pct
        min_decay = math.log(target) / slow_decay_pct
        self.register_buffer("deltas_abs", torch.linspace(min_decay, max_decay, channels).abs(), persistent=False)
        self.modulate, self.shift = modulate, shift

    def forward(self, t, x):
        if self.modulate:
            x = x * (torch.exp(-t[:, None] * self.deltas_abs[None, :]) + self.shift)
        return x


class Sin(nn.Module):
    """``sin(freq * x)`` with a trainable per-unit frequency, shared by all layers of the filter MLP."""

    def __init__(self, width: int, w: float = 10.0):
        super().__init__()
        self.freq = nn.Parameter(w * torch.ones(width))

    def forward(self, x):
        return torch.sin(self.freq * x)


class MLPTrainableActivation(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, width: int, depth: int, activation: nn.Module, use_bias: bool = True,
                 use_final_bias: bool = True):
        super().__init__()
        dims = [in_dim] + [width] * depth + [out_dim]
        self.layers = nn.ModuleList([Linear(a, b, bias=(use_bias if i < depth else use_final_bias), init_std=1.0 / math.sqrt(a))
                                     for i, (a, b) in enumerate(zip(dims[:-1], dims[1:]))])
        self.activation = activation

    def forward(self, x):
        for layer in self.layers[:-1]:
            x = self.activation(layer(x))
        return self.layers[-1](x)


def fft_conv(u: torch.Tensor, k: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal convolution along the second-to-last axis: ``u[..., L, C]`` with ``k[L, C]`` (+ per-channel bias).  On a B200 and
    for ``L <= 4096`` this is a direct sum in shared memory (``ops/long_conv.py``); otherwise a zero-padded FFT of size 2L."""
    from ..ops.long_conv import long_conv

    return long_conv(u, k, bias)


class HyenaFilter(nn.Module):
    def __init__(self, config: HyenaConfig):
        super().__init__()
        c = config
        channels = c.head_size * (c.order - 1)
        self.pos_emb = PositionalEmbedding(c.pos_per_block, c.filter_emb_dim)
        self.implicit_filter = MLPTrainableActivation(c.filter_emb_dim, channels, c.filter_order, c.num_hidden_layers_filter_mlp,
                                                      Sin(c.filter_order, w=1), use_bias=c.use_bias)
        self.modulation = ExponentialModulation(channels, c.fast_decay_pct, c.slow_decay_pct, c.target, c.modulate, c.shift)
        self.bias = nn.Parameter(torch.randn(c.head_size))
        self.use_bias = c.use_bias
        self.normalized = False
        self.dropout = Dropout(c.filter_dropout)

    def generate_filters(self, input_length: int) -> torch.Tensor:
        """``[L, head_size * (order - 1)]``."""
        z, t = self.pos_emb(input_length)
        h = self.implicit_filter(z.to(self.bias.dtype))
        h = self.modulation(t, h.float()).to(h.dtype)
        if self.normalized:
            h = h / h.abs().sum(dim=1, keepdim=True)
        return h

    def forward(self, x: torch.Tensor, k: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x[..., L, head_size]``, ``k[L, head_size]``."""
        bias = self.bias if bias is None else bias
        y = fft_conv(x, k, bias if self.use_bias else None)
        return self.dropout(y)


class HyenaOperator(nn.Module):
    def __init__(self, config: HyenaConfig):
        super().__init__()
        c = config
        self.config = c
        width = c.hidden_dim * (c.order + 1)
        self.in_proj = Linear(c.hidden_dim, width, bias=c.use_bias)
        self.out_proj = Linear(c.hidden_dim, c.hidden_dim, bias=c.use_bias)
        # depthwise causal convolution: left padding k - 1, keep the first L outputs
        self.short_filter = nn.Conv1d(width, width, c.short_filter_order, groups=width, padding=c.short_filter_order - 1)
        self.filter_fn = HyenaFilter(c)
        self.dropout = Dropout(c.resid_pdrop)
        self.activation = c.activation.to_fn()

    def forward(self, u: torch.Tensor) -> torch.Tensor:
        c = self.config
        B, L, _ = u.shape
        l_filter = min(L, c.seq_len)
        u = self.in_proj(u)
        from ..ops.dwconv import causal_dwconv

        uc = causal_dwconv(u, self.short_filter.weight, self.short_filter.bias)[:, :l_filter]  # causal: truncation commutes
        nb = c.num_blocks if l_filter == c.seq_len else 1
        per = l_filter // nb
        # [B, blocks, pos, heads, (order + 1), head_size]
        uc = uc.reshape(B, nb, per, c.num_heads, c.order + 1, c.head_size)
        comps = uc.unbind(dim=4)
        v, x = comps[-1], comps[:-1]
        filters = self.filter_fn.generate_filters(per).reshape(per, c.order - 1, c.head_size)
        for o, x_i in enumerate(reversed(x[1:])):
            if c.outer_mixing:
                v = self.dropout(v.unsqueeze(-1) * x_i.unsqueeze(-2)).sum(dim=-2)
            else:
                v = self.dropout(v * x_i)
            # convolve along the position axis: move it next to the channel axis
            vt = v.permute(0, 1, 3, 2, 4)  # [B, blocks, heads, pos, head_size]
            vt = self.filter_fn(vt, filters[:, o, :])
            v = vt.permute(0, 1, 3, 2, 4)
        v = v * x[0]
        y = self.activation(v.reshape(B, l_filter, c.hidden_dim))
        return self.out_proj(y)
