"""Gated DeltaNet language model (Yang, Kautz & Hatamizadeh, "Gated Delta Networks", 2024): a decoder whose token mixer is
the gated delta rule, a linear-time recurrence with a matrix state per head,

    S_t = a_t * S_{t-1} (I - b_t k_t k_t^T) + b_t v_t k_t^T,        o_t = S_t q_t,

with decay ``a_t = exp(g_t) in (0, 1]`` and write strength ``b_t in (0, 1)``.  The reference framework has no such family;
parameter names follow the public implementations of the layer (``q_proj``/``k_proj``/``v_proj``, depthwise ``conv1d`` on
each, ``a_proj``/``b_proj``, ``A_log``, ``dt_bias``, gated output norm ``g_proj``/``o_norm``, ``o_proj``) so that converters
can be written against them.

Training uses the chunked form (:func:`delta_rule_chunked_scan`): inside a chunk of ``C`` tokens the recurrence is a
triangular system solved once (the WY representation), across chunks only the ``[d_k, d_v]`` state is carried, so the work
is batched matrix products of size ``C`` instead of ``L`` sequential rank-one updates.  :func:`delta_rule_recurrent` is the
step-by-step statement used for decoding and as the test oracle."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple, Type

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..layers.normalization import LayerNormConfigBase, RmsNormConfig
from ..nn import Embedding, Linear
from ..ops.delta_rule import chunk_state_scan
from ..ops.dwconv import causal_dwconv
from ..utils.activation import ActivationFunctionEnum
from ..utils.flop_utils import lm_flops_per_token
from ..utils.remat import should_recompute
from .llama import LlamaMlp
from .lm_model import LmConfig, LmHeadModel


def delta_rule_recurrent(q, k, v, g, beta, initial_state: Optional[torch.Tensor] = None):
    """Sequential gated delta rule.  ``q, k: [B, H, L, dk]``, ``v: [B, H, L, dv]``, ``g`` (log decay, <= 0) and ``beta``:
    ``[B, H, L]``.  Returns ``(o [B, H, L, dv], final state [B, H, dk, dv])`` in fp32."""
    B, H, L, dk = q.shape
    dv = v.shape[-1]
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    q = q * dk ** -0.5
    S = torch.zeros(B, H, dk, dv, device=q.device) if initial_state is None else initial_state.float().clone()
    out = torch.empty(B, H, L, dv, device=q.device)
    for t in range(L):
        S = S * g[:, :, t].exp()[..., None, None]
        kt, vt, bt = k[:, :, t], v[:, :, t], beta[:, :, t][..., None]
        pred = torch.einsum("bhk,bhkv->bhv", kt, S)  # what the memory currently returns for this key
        S = S + torch.einsum("bhk,bhv->bhkv", kt, (vt - pred) * bt)
        out[:, :, t] = torch.einsum("bhk,bhkv->bhv", q[:, :, t], S)
    return out, S


def delta_rule_chunked_scan(q, k, v, g, beta, chunk_size: int = 64, initial_state: Optional[torch.Tensor] = None):
    """Chunk-parallel gated delta rule with the same contract as :func:`delta_rule_recurrent`."""
    B, H, L, dk = q.shape
    dv = v.shape[-1]
    dtype = v.dtype
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    pad = (-L) % chunk_size
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    N, C = (L + pad) // chunk_size, chunk_size
    q = q * dk ** -0.5
    q, k, v = (t.reshape(B, H, N, C, -1) for t in (q, k, v))
    g = g.reshape(B, H, N, C).cumsum(-1)  # log decay from the chunk start up to and including each position
    beta = beta.reshape(B, H, N, C)
    kb, vb = k * beta[..., None], v * beta[..., None]
    # decay[i, j] = exp(g_i - g_j) for j <= i: how much of what was written at j survives until i
    diff = g[..., :, None] - g[..., None, :]
    lower = torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device))
    decay = torch.where(lower, diff, torch.full_like(diff, -float("inf"))).exp()
    # within a chunk the writes depend on one another through the predictions: (I + strict_lower(kb k^T * decay)) U = rhs
    A = torch.tril((kb @ k.transpose(-1, -2)) * decay, diagonal=-1)
    eye = torch.eye(C, device=q.device)
    T = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False)
    u = T @ vb  # values to write if the state entering the chunk were zero
    w = T @ (kb * g.exp()[..., None])  # what has to be corrected for the state entering the chunk
    # the loop over chunks only carries the state; everything it consumes is formed here for all chunks at once
    strict_upper = torch.triu(torch.ones(C, C, dtype=torch.bool, device=q.device), diagonal=1)
    scores = ((q @ k.transpose(-1, -2)) * decay).masked_fill(strict_upper, 0.0)
    qg = q * g.exp()[..., None]
    g_last = g[..., -1]
    kd = k * (g_last[..., None] - g).exp()[..., None]
    out, S = chunk_state_scan(w, qg, kd, scores, u, g_last.exp(), initial_state)
    out = out.reshape(B, H, N * C, dv)[:, :, :L]
    return out.to(dtype), S


@LmConfig.register_subclass("gated_deltanet")
@dataclass(frozen=True)
class GatedDeltaNetConfig(LmConfig):
    seq_len: int = 2048
    hidden_dim: int = 1024
    intermediate_dim: int = 2816
    num_layers: int = 24
    num_heads: int = 8  # value heads
    num_k_heads: Optional[int] = None  # key/query heads (value heads are grouped over them); default: num_heads
    head_k_dim: int = 128
    head_v_dim: int = 128
    conv_kernel: int = 4
    chunk_size: int = 64
    activation_function: ActivationFunctionEnum = ActivationFunctionEnum.silu
    initializer_range: float = 0.02
    layer_norm_epsilon: float = 1e-6
    tie_word_embeddings: bool = False
    use_bias: bool = False
    gradient_checkpointing: bool = True
    norm_config: LayerNormConfigBase = RmsNormConfig(use_weight=True, use_bias=False, eps=1e-6)
    cross_entropy_block_size: Optional[int] = None

    @property
    def model_type(self) -> Type["GatedDeltaNetLMHeadModel"]:
        return GatedDeltaNetLMHeadModel

    @property
    def k_heads(self) -> int:
        return self.num_k_heads or self.num_heads

    def mk_LayerNorm(self, dim: int):
        return self.norm_config.build(dim)

    def flops_per_token(self, vocab_size: int) -> Optional[float]:
        # projections + MLP like a transformer with no quadratic term; the scan adds ~ 4 * d_k * d_v per head per token
        e = self.hidden_dim
        kd, vd = self.k_heads * self.head_k_dim, self.num_heads * self.head_v_dim
        mixer = 2 * e * (2 * kd + 2 * vd) + 2 * vd * e + 4 * self.num_heads * self.head_k_dim * self.head_v_dim
        mlp = 2 * 3 * e * self.intermediate_dim
        return self.num_layers * (mixer + mlp) + 2 * e * vocab_size

    def total_trainable_params(self, vocab_size: int) -> int:
        e = self.hidden_dim
        kd, vd = self.k_heads * self.head_k_dim, self.num_heads * self.head_v_dim
        mixer = e * (2 * kd + 2 * vd) + vd * e + 2 * e * self.num_heads + (2 * kd + vd) * self.conv_kernel + 2 * self.num_heads + self.head_v_dim
        return self.num_layers * (mixer + 3 * e * self.intermediate_dim + 2 * e) + e + vocab_size * e * (1 if self.tie_word_embeddings else 2)


class GatedDeltaNetLayer(nn.Module):
    """The token mixer: projections, short causal convolutions, gates, the delta-rule scan, gated output norm."""

    def __init__(self, config: GatedDeltaNetConfig):
        super().__init__()
        c = config
        self.config = c
        kd, vd = c.k_heads * c.head_k_dim, c.num_heads * c.head_v_dim
        std = c.initializer_range
        self.q_proj = Linear(c.hidden_dim, kd, bias=False, init_std=std)
        self.k_proj = Linear(c.hidden_dim, kd, bias=False, init_std=std)
        self.v_proj = Linear(c.hidden_dim, vd, bias=False, init_std=std)
        self.a_proj = Linear(c.hidden_dim, c.num_heads, bias=False, init_std=std)
        self.b_proj = Linear(c.hidden_dim, c.num_heads, bias=False, init_std=std)
        self.g_proj = Linear(c.hidden_dim, vd, bias=False, init_std=std)
        self.o_proj = Linear(vd, c.hidden_dim, bias=False, init_std=std)
        self.q_conv1d = nn.Conv1d(kd, kd, c.conv_kernel, groups=kd, padding=c.conv_kernel - 1, bias=False)
        self.k_conv1d = nn.Conv1d(kd, kd, c.conv_kernel, groups=kd, padding=c.conv_kernel - 1, bias=False)
        self.v_conv1d = nn.Conv1d(vd, vd, c.conv_kernel, groups=vd, padding=c.conv_kernel - 1, bias=False)
        # decay rate a = exp(-exp(A_log) * softplus(a_proj(x) + dt_bias)): A in [1, 16], time steps log-uniform in [1e-3, 1e-1]
        self.A_log = nn.Parameter(torch.log(torch.empty(c.num_heads).uniform_(1.0, 16.0)))
        dt = torch.exp(torch.rand(c.num_heads) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus
        self.o_norm_weight = nn.Parameter(torch.ones(c.head_v_dim))
        for p in (self.A_log, self.dt_bias):
            p._no_weight_decay = True

    def _conv(self, conv: nn.Conv1d, x: torch.Tensor) -> torch.Tensor:
        # depthwise causal filter + SiLU over [B, L, C]; one kernel per direction on CUDA, conv1d between transposes elsewhere
        return causal_dwconv(x, conv.weight, conv.bias, silu=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.config
        B, L, _ = x.shape
        H, Hk, dk, dv = c.num_heads, c.k_heads, c.head_k_dim, c.head_v_dim
        q = self._conv(self.q_conv1d, self.q_proj(x)).view(B, L, Hk, dk)
        k = self._conv(self.k_conv1d, self.k_proj(x)).view(B, L, Hk, dk)
        v = self._conv(self.v_conv1d, self.v_proj(x)).view(B, L, H, dv)
        q = F.normalize(q.float(), dim=-1)
        k = F.normalize(k.float(), dim=-1)
        if Hk != H:
            q = q.repeat_interleave(H // Hk, dim=2)
            k = k.repeat_interleave(H // Hk, dim=2)
        beta = torch.sigmoid(self.b_proj(x).float())  # [B, L, H]
        g = -self.A_log.float().exp() * F.softplus(self.a_proj(x).float() + self.dt_bias.float())
        o, _ = delta_rule_chunked_scan(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2).float(), g.transpose(1, 2),
                                       beta.transpose(1, 2), chunk_size=c.chunk_size)
        o = o.transpose(1, 2)  # [B, L, H, dv]
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + c.layer_norm_epsilon) * self.o_norm_weight.float()
        o = o * F.silu(self.g_proj(x).float().view(B, L, H, dv))
        return self.o_proj(o.reshape(B, L, H * dv).to(x.dtype))


class GatedDeltaNetBlock(nn.Module):
    def __init__(self, config: GatedDeltaNetConfig):
        super().__init__()
        self.attn_norm = config.mk_LayerNorm(config.hidden_dim)
        self.attn = GatedDeltaNetLayer(config)
        self.mlp_norm = config.mk_LayerNorm(config.hidden_dim)
        self.mlp = LlamaMlp(config.hidden_dim, config.intermediate_dim, config.activation_function, use_bias=config.use_bias,
                            init_std=config.initializer_range)

    def forward(self, x):
        x = x + self.attn(self.attn_norm(x))
        return x + self.mlp(self.mlp_norm(x))


class GatedDeltaNetLMHeadModel(LmHeadModel):
    def __init__(self, vocab_size: int, config: GatedDeltaNetConfig):
        super().__init__()
        self.config = config
        self._vocab_size = vocab_size
        self.embeddings = Embedding(vocab_size, config.hidden_dim, init_std=config.initializer_range)
        self.layers = nn.ModuleList([GatedDeltaNetBlock(config) for _ in range(config.num_layers)])
        self.norm = config.mk_LayerNorm(config.hidden_dim)
        self.lm_head = None if config.tie_word_embeddings else Linear(config.hidden_dim, vocab_size, bias=False, init_std=config.initializer_range)

    @classmethod
    def init(cls, vocab_size: int, config: GatedDeltaNetConfig, *, tp=None) -> "GatedDeltaNetLMHeadModel":
        return cls(vocab_size, config)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def activations(self, input_ids, attn_mask=None, *, pos_ids=None):
        # the recurrence is causal by construction; segment masks are not supported (state flows across document ends)
        x = self.embeddings(input_ids)
        squeeze = x.dim() == 2
        if squeeze:
            x = x.unsqueeze(0)
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        for layer in self.layers:
            x = checkpoint(layer, x, use_reentrant=False) if remat else layer(x)
        x = self.norm(x)
        return x.squeeze(0) if squeeze else x

    def get_lm_head(self) -> torch.Tensor:
        return self.embeddings.weight if self.lm_head is None else self.lm_head.weight

    def resize_vocab(self, new_size: int):
        self.embeddings = self.embeddings.resize_embeddings(new_size, self.config.initializer_range)
        if self.lm_head is not None:
            old = self.lm_head
            new = Linear(self.config.hidden_dim, new_size, bias=False, init_std=self.config.initializer_range,
                         device=old.weight.device, dtype=old.weight.dtype)
            n = min(old.weight.shape[0], new_size)
            with torch.no_grad():
                new.weight[:n].copy_(old.weight[:n])
            self.lm_head = new
        self._vocab_size = new_size
        return self
