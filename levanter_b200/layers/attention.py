"""Attention: structured masks, the dispatching ``dot_product_attention``, the ``Attention`` module with
GQA / qk-norm / RoPE / sinks, multi-head latent attention, and the paged KV cache used by the inference engine.

Reference behaviour: src/levanter/layers/attention.py (mask :757-1003, dispatch :71-241, vanilla :329-378,
sink :244-326, module :1373-1635, KvPageCache :1638-1707, ragged paged attention :1710-1991, MLA :1994-2213).

Tensor layout here is ``q[B, Sq, Hq, D]``, ``k/v[B, Sk, Hkv, D]`` with ``Hq = Hkv * q_per_kv`` and query head
``h`` reading KV head ``h // q_per_kv`` (the reference's ``(kv_head, q_heads_per_group)`` articulation).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field, replace
from typing import Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from .normalization import LayerNormConfigBase, RmsNormConfig
from .rotary import DefaultRotaryEmbeddingsConfig, RotaryEmbeddings, RotaryEmbeddingsConfig


class AttentionBackend(str, enum.Enum):
    DEFAULT = "default"      # B200 flash kernel on a B200, blockwise PyTorch elsewhere
    B200 = "b200"            # hand-written sm_100a flash attention (ops.flash_attention)
    TORCH_FLASH = "torch_flash"  # blockwise FA-2 in PyTorch ops (counterpart of the reference's JAX_FLASH)
    SDPA = "sdpa"            # torch.nn.functional.scaled_dot_product_attention (library kernel; baseline/oracle)
    VANILLA = "vanilla"      # materialise the score matrix
    # names accepted from reference configs; they select DEFAULT here
    NVTE = "nvte"
    SPLASH = "splash"
    JAX_FLASH = "jax_flash"


# --------------------------------------------------------------------------------------------- masks
def _and(a, b):
    if a is None:
        return b
    if b is None:
        return a
    return a & b


def _or(a, b):
    if a is None or b is None:
        return None if (a is None and b is None) else (a if b is None else b)
    return a | b


def causal_mask(q_len: int, k_len: int, q_start=0, k_start=0, device=None) -> torch.Tensor:
    qp = torch.arange(q_len, device=device) + q_start
    kp = torch.arange(k_len, device=device) + k_start
    return qp[:, None] >= kp[None, :]


@dataclass(frozen=True)
class AttentionMask:
    """Conjunction of structured masks: causal (with an optional offset), explicit, sliding window, segment ids.

    ``materialize(q_len, k_len, q_slice, k_slice)`` returns the boolean mask of a block so block-wise kernels
    can skip or specialise blocks (src/levanter/layers/attention.py:795-846)."""

    is_causal: bool = False
    causal_offset: Union[None, int, torch.Tensor] = None
    explicit_mask: Optional[torch.Tensor] = None            # [..., Sq, Sk] bool
    segment_ids: Optional[Tuple[torch.Tensor, torch.Tensor]] = None  # ([B, Sq], [B, Sk])
    sliding_window: Optional[int] = None
    segments_sorted: bool = False
    """the segment ids are non-decreasing along the sequence with negative ids (padding) only at the end, as in packed
    batches: kernels may then skip every key block that lies before a query block's first sequence"""

    def __post_init__(self):
        if self.segment_ids is not None and not isinstance(self.segment_ids, tuple):
            object.__setattr__(self, "segment_ids", (self.segment_ids, self.segment_ids))

    @staticmethod
    def causal(*, sliding_window: Optional[int] = None, offset=None) -> "AttentionMask":
        return AttentionMask(is_causal=True, causal_offset=offset, sliding_window=sliding_window)

    @staticmethod
    def explicit(mask: torch.Tensor) -> "AttentionMask":
        return AttentionMask(is_causal=False, explicit_mask=mask)

    def with_segment_ids(self, segment_ids, kv_segment_ids=None, *, sorted: bool = False) -> "AttentionMask":
        return replace(self, segment_ids=(segment_ids, segment_ids if kv_segment_ids is None else kv_segment_ids),
                       segments_sorted=bool(sorted))

    def with_sliding_window(self, sliding_window: Optional[int]) -> "AttentionMask":
        return replace(self, sliding_window=sliding_window)

    def materialize(self, q_len: int, k_len: int, q_slice: Optional[Tuple[int, int]] = None,
                    k_slice: Optional[Tuple[int, int]] = None, device=None) -> Optional[torch.Tensor]:
        """Boolean mask broadcastable to ``[B, 1, q, k]`` for the block ``q_slice=(start,size)`` x ``k_slice``."""
        qs, qn = q_slice if q_slice is not None else (0, q_len)
        ks, kn = k_slice if k_slice is not None else (0, k_len)
        mask = None
        if self.is_causal:
            off = 0 if self.causal_offset is None else self.causal_offset
            if isinstance(off, torch.Tensor) and off.dim() > 0:
                qp = (torch.arange(qn, device=device) + qs)[None, :, None]
                kp = (torch.arange(kn, device=device) + ks)[None, None, :]
                mask = (qp + off.to(device).view(-1, 1, 1) >= kp).unsqueeze(1)
            else:
                off = int(off)
                mask = causal_mask(qn, kn, qs, ks - off, device)
        if self.explicit_mask is not None:
            em = self.explicit_mask[..., qs:qs + qn, ks:ks + kn]
            if em.dim() == 3:
                em = em.unsqueeze(1)
            mask = _and(mask, em.to(torch.bool))
        if self.sliding_window is not None:
            qp = torch.arange(qn, device=device) + qs
            kp = torch.arange(kn, device=device) + ks
            diff = qp[:, None] - kp[None, :]
            mask = _and(mask, (diff >= 0) & (diff < self.sliding_window))
        if self.segment_ids is not None:
            qseg, kseg = self.segment_ids
            sm = qseg[..., qs:qs + qn, None] == kseg[..., None, ks:ks + kn]
            if sm.dim() == 3:
                sm = sm.unsqueeze(1)
            mask = _and(mask, sm)
        return mask

    def __and__(self, other: "AttentionMask") -> "AttentionMask":
        if self.is_causal and other.is_causal:
            if self.causal_offset is not None and other.causal_offset is not None:
                same = self.causal_offset == other.causal_offset
                if isinstance(same, torch.Tensor):
                    same = bool(same.all())
                if not same:
                    raise ValueError("Mismatched causal offsets cannot be combined with &")
                offset = self.causal_offset
            else:
                offset = self.causal_offset if self.causal_offset is not None else other.causal_offset
            is_causal = True
        elif self.is_causal:
            is_causal, offset = True, self.causal_offset
        elif other.is_causal:
            is_causal, offset = True, other.causal_offset
        else:
            is_causal, offset = False, None
        if self.sliding_window is None:
            sw = other.sliding_window
        elif other.sliding_window is None:
            sw = self.sliding_window
        else:
            sw = min(self.sliding_window, other.sliding_window)
        return AttentionMask(is_causal, offset, _and(self.explicit_mask, other.explicit_mask), self._same_segments(other), sw)

    def __or__(self, other: "AttentionMask") -> "AttentionMask":
        def same_off():
            if self.causal_offset is None and other.causal_offset is None:
                return True
            if self.causal_offset is None or other.causal_offset is None:
                return False
            s = self.causal_offset == other.causal_offset
            return bool(s.all()) if isinstance(s, torch.Tensor) else bool(s)

        if self.is_causal and other.is_causal and same_off():
            is_causal, offset = True, self.causal_offset
        else:
            is_causal, offset = False, None
        if self.sliding_window is None or other.sliding_window is None:
            sw = None
        else:
            sw = max(self.sliding_window, other.sliding_window)
        return AttentionMask(is_causal, offset, _or(self.explicit_mask, other.explicit_mask), self._same_segments(other), sw)

    def _same_segments(self, other):
        a, b = self.segment_ids, other.segment_ids
        if a is not None and b is not None:
            if not (torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])):
                raise ValueError("Only one segment mask is allowed")
            return a
        return a if a is not None else b


def materialize_mask(mask: Union[None, torch.Tensor, AttentionMask], q_len: int, k_len: int, device=None,
                     q_slice=None, k_slice=None) -> Optional[torch.Tensor]:
    if mask is None:
        return None
    if isinstance(mask, AttentionMask):
        return mask.materialize(q_len, k_len, q_slice, k_slice, device=device)
    qs, qn = q_slice if q_slice is not None else (0, q_len)
    ks, kn = k_slice if k_slice is not None else (0, k_len)
    m = mask[..., qs:qs + qn, ks:ks + kn]
    if m.dim() == 3:
        m = m.unsqueeze(1)
    return m


# --------------------------------------------------------------------------------------------- attention functions
def _expand_kv(k: torch.Tensor, q_heads: int) -> torch.Tensor:
    kv = k.shape[2]
    if kv == q_heads:
        return k
    return k.repeat_interleave(q_heads // kv, dim=2)


def simple_attention_with_dropout(q, k, v, mask=None, bias=None, *, dropout: float = 0.0, inference: bool = True,
                                  attention_dtype: Optional[torch.dtype] = None, logits_soft_cap: Optional[float] = None,
                                  scaling_factor: Optional[float] = None) -> torch.Tensor:
    """Vanilla attention: scale q, QK^T, +bias, tanh soft-cap, mask -> -1e9, softmax in ``attention_dtype``, dropout, .V
    (src/levanter/layers/attention.py:329-378)."""
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    scale = scaling_factor if scaling_factor is not None else 1.0 / math.sqrt(D)
    orig = v.dtype
    kk = _expand_kv(k, H)
    vv = _expand_kv(v, H)
    if attention_dtype is not None:
        q, kk = q.to(attention_dtype), kk.to(attention_dtype)
    w = torch.einsum("bqhd,bkhd->bhqk", q * scale, kk)
    if bias is not None:
        w = w + bias
    if logits_soft_cap is not None:
        w = torch.tanh(w / logits_soft_cap) * logits_soft_cap
    m = materialize_mask(mask, Sq, Sk, device=q.device)
    if m is not None:
        w = torch.where(m, w, torch.full_like(w, -1e9))
    w = torch.softmax(w.float() if attention_dtype is None else w, dim=-1).to(orig)
    if dropout > 0.0 and not inference:
        w = F.dropout(w, dropout, training=True)
    return torch.einsum("bhqk,bkhd->bqhd", w, vv)


def _structured_only(mask) -> bool:
    """True when the mask has only the structures the fused kernels understand natively."""
    if mask is None:
        return True
    if not isinstance(mask, AttentionMask):
        return False
    if mask.explicit_mask is not None:
        return False
    if mask.causal_offset is not None and not (isinstance(mask.causal_offset, int) and mask.causal_offset == 0):
        off = mask.causal_offset
        if isinstance(off, torch.Tensor) and off.dim() == 0 and int(off) == 0:
            return True
        return False
    return True


def dot_product_attention(q, k, v, mask: Union[None, torch.Tensor, AttentionMask] = None, bias=None, *,
                          attention_dtype: Optional[torch.dtype] = None, dropout: float = 0.0, inference: bool = True,
                          use_flash: Optional[bool] = None, attn_backend: Optional[AttentionBackend] = None,
                          flash_block_size: Optional[int] = None, logits_soft_cap: Optional[float] = None,
                          scaling_factor: Optional[float] = None) -> torch.Tensor:
    """Dispatch to the best available attention implementation (src/levanter/layers/attention.py:71-241).

    On a B200 the default is the hand-written flash kernel whenever the mask is structured (causal / sliding
    window / segment ids), there is no bias and no dropout; anything else falls through to blockwise PyTorch
    flash attention and finally to the vanilla implementation."""
    from ..models import flash_attention as FA
    from ..ops import flash_attention as KFA

    backend = attn_backend or AttentionBackend.DEFAULT
    if isinstance(backend, str) and not isinstance(backend, AttentionBackend):
        backend = AttentionBackend(backend)
    if backend in (AttentionBackend.NVTE, AttentionBackend.SPLASH):
        backend = AttentionBackend.DEFAULT
    if backend == AttentionBackend.JAX_FLASH:
        backend = AttentionBackend.TORCH_FLASH
    if use_flash is False:
        backend = AttentionBackend.VANILLA
    no_drop = dropout == 0.0 or inference

    if backend in (AttentionBackend.DEFAULT, AttentionBackend.B200):
        if KFA.supported(q, k, v, mask, bias, no_drop, attention_dtype):
            return KFA.flash_attention(q, k, v, mask, logits_soft_cap=logits_soft_cap, scaling_factor=scaling_factor)
        if backend == AttentionBackend.B200:
            raise ValueError("the B200 flash-attention kernel does not support this call (bias, dropout, explicit mask, dtype or head size)")
        plain = mask is None or (isinstance(mask, AttentionMask) and mask.explicit_mask is None and mask.segment_ids is None
                                 and mask.sliding_window is None and _structured_only(mask))
        if q.is_cuda and plain and bias is None and no_drop and logits_soft_cap is None and q.dtype in (torch.bfloat16, torch.float16) \
                and q.shape[1] == k.shape[1]:
            # shapes the tcgen05 kernels do not cover (head sizes other than 64 and 128, cross attention): the library's fused
            # attention rather than the blockwise PyTorch loop
            backend = AttentionBackend.SDPA
        else:
            backend = AttentionBackend.TORCH_FLASH if q.shape[1] > 1 else AttentionBackend.VANILLA

    if backend == AttentionBackend.SDPA and bias is None and no_drop and logits_soft_cap is None:
        B, Sq, H, D = q.shape
        m = materialize_mask(mask, Sq, k.shape[1], device=q.device)
        is_causal = isinstance(mask, AttentionMask) and mask.is_causal and mask.explicit_mask is None and \
            mask.segment_ids is None and mask.sliding_window is None and _structured_only(mask)
        out = F.scaled_dot_product_attention(
            q.transpose(1, 2), _expand_kv(k, H).transpose(1, 2), _expand_kv(v, H).transpose(1, 2),
            attn_mask=None if is_causal else m, is_causal=is_causal, scale=scaling_factor)
        return out.transpose(1, 2)

    if backend == AttentionBackend.TORCH_FLASH and bias is None:
        block = flash_block_size or FA.BLOCK_SIZE
        if q.shape[1] >= block and k.shape[1] >= block and q.shape[1] % block == 0 and k.shape[1] % block == 0:
            return FA.flash_attention(q, k, v, mask, dropout=dropout, inference=inference, block_size=block,
                                      dtype=attention_dtype, logits_soft_cap=logits_soft_cap, scaling_factor=scaling_factor)
    return simple_attention_with_dropout(q, k, v, mask, bias, dropout=dropout, inference=inference,
                                         attention_dtype=attention_dtype, logits_soft_cap=logits_soft_cap,
                                         scaling_factor=scaling_factor)


def dot_product_attention_with_sink(q, k, v, sink: torch.Tensor, mask=None, bias=None, **kw) -> torch.Tensor:
    """Attention with a learned per-head sink logit: a zero K/V column is appended and the sink logit is placed in
    the bias at that column (src/levanter/layers/attention.py:244-326).  ``sink``: ``[Hq]``."""
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    from ..ops import flash_attention as KFA

    if (kw.get("dropout", 0.0) == 0.0 or kw.get("inference", False)) and KFA.supported(q, k, v, mask, bias, True, kw.get("attention_dtype")):
        # the fused kernel takes the sink as one more term of the softmax denominator
        return KFA.flash_attention(q, k, v, mask, logits_soft_cap=kw.get("logits_soft_cap"), scaling_factor=kw.get("scaling_factor"),
                                   sink=sink)
    zk = torch.zeros(B, 1, k.shape[2], D, dtype=k.dtype, device=k.device)
    k2 = torch.cat([k, zk], dim=1)
    v2 = torch.cat([v, torch.zeros_like(zk)], dim=1)
    b = torch.zeros(B, H, Sq, Sk + 1, dtype=torch.float32, device=q.device)
    if bias is not None:
        b[..., :Sk] = bias
    b[..., Sk] = sink.float().view(1, H, 1)
    m = materialize_mask(mask, Sq, Sk, device=q.device)
    if m is not None:
        m = m.expand(B, -1, Sq, Sk) if m.dim() == 4 else m.expand(Sq, Sk)[None, None].expand(B, 1, Sq, Sk)
        m = torch.cat([m, torch.ones(B, m.shape[1], Sq, 1, dtype=torch.bool, device=q.device)], dim=-1)
    kw.pop("attn_backend", None)
    return simple_attention_with_dropout(q, k2, v2, m, b, **{k_: v_ for k_, v_ in kw.items() if k_ in
                                          ("dropout", "inference", "attention_dtype", "logits_soft_cap", "scaling_factor")})


# --------------------------------------------------------------------------------------------- module
from ..nn import Linear, RmsNorm  # noqa: E402  (after function definitions to keep the file readable)


@dataclass(frozen=True)
class AttentionConfig:
    """Configuration of the shared attention module (src/levanter/layers/attention.py:1373-1447)."""

    hidden_dim: int
    num_heads: int
    num_kv_heads: int
    head_dim: Optional[int] = None
    use_bias: bool = False
    use_output_bias: Optional[bool] = None
    upcast_attn: bool = False
    attn_backend: Optional[AttentionBackend] = None
    flash_attention_block_size: Optional[int] = None
    rope: Optional[RotaryEmbeddingsConfig] = None
    scaling_factor: Optional[float] = None
    logits_soft_cap: Optional[float] = None
    qk_norm: Optional[LayerNormConfigBase] = None
    sliding_window: Optional[int] = None

    def __post_init__(self):
        assert self.num_heads % self.num_kv_heads == 0, "num_heads must be divisible by num_kv_heads"

    @property
    def head_size(self) -> int:
        return self.head_dim if self.head_dim is not None else self.hidden_dim // self.num_heads

    @property
    def q_heads_per_group(self) -> int:
        return self.num_heads // self.num_kv_heads

    @property
    def use_flash_attention(self) -> bool:
        return self.attn_backend != AttentionBackend.VANILLA


class Attention(nn.Module):
    """Multi-head / grouped-query attention with optional per-head qk-norm and RoPE.

    Parameter layouts for checkpoints: ``q_proj.weight [kv_head, q_heads_per_group, head_size, embed]``,
    ``k_proj/v_proj.weight [kv_head, head_size, embed]``, ``o_proj.weight [embed, heads, head_size]``
    (src/levanter/layers/attention.py:1473-1488).  In memory they are the 2-D ``[out, in]`` matrices the GEMM
    kernels consume; the articulated shape is a reshape."""

    def __init__(self, config: AttentionConfig, *, init_std: float = 0.02, tp=None):
        super().__init__()
        c = config
        self.config = c
        D = c.head_size
        self.tp = tp
        tp_size = tp.size if tp is not None else 1
        assert c.num_kv_heads % tp_size == 0 or tp_size == 1, "kv heads must divide the tensor-parallel size"
        self.local_heads = c.num_heads // tp_size
        self.local_kv = c.num_kv_heads // tp_size
        out_bias = c.use_output_bias if c.use_output_bias is not None else c.use_bias
        self.q_proj = Linear(c.hidden_dim, self.local_heads * D, bias=c.use_bias, init_std=init_std,
                             lev_out=(self.local_kv, c.q_heads_per_group, D), lev_in=(c.hidden_dim,), parallel=("column", tp))
        self.k_proj = Linear(c.hidden_dim, self.local_kv * D, bias=c.use_bias, init_std=init_std,
                             lev_out=(self.local_kv, D), lev_in=(c.hidden_dim,), parallel=("column", tp))
        self.v_proj = Linear(c.hidden_dim, self.local_kv * D, bias=c.use_bias, init_std=init_std,
                             lev_out=(self.local_kv, D), lev_in=(c.hidden_dim,), parallel=("column", tp))
        self.o_proj = Linear(self.local_heads * D, c.hidden_dim, bias=out_bias, init_std=init_std,
                             lev_out=(c.hidden_dim,), lev_in=(self.local_heads, D), parallel=("row", tp))
        if c.qk_norm is not None:
            self.q_norm = c.qk_norm.build(D)
            self.k_norm = c.qk_norm.build(D)
        else:
            self.q_norm = None
            self.k_norm = None
        self.rot: Optional[RotaryEmbeddings] = c.rope.build(D) if c.rope is not None else None

    # -- projections shared by training and paged decode (src/levanter/layers/attention.py:1606-1635)
    def _compute_qkv(self, x: torch.Tensor, pos_ids: Optional[torch.Tensor]):
        c = self.config
        D = c.head_size
        lead = x.shape[:-1]
        q = self.q_proj(x).view(*lead, self.local_heads, D)
        k = self.k_proj(x).view(*lead, self.local_kv, D)
        v = self.v_proj(x).view(*lead, self.local_kv, D)
        if self.q_norm is not None:
            q = self.q_norm(q)
            k = self.k_norm(k)
        if self.rot is not None:
            from ..ops import rope as rope_op

            q, k = rope_op.apply_rope(q, k, self.rot, pos_ids)
        return q, k, v

    def forward(self, x: torch.Tensor, mask: Union[None, AttentionMask, torch.Tensor] = None,
                pos_ids: Optional[torch.Tensor] = None, *, skip_out_bias: bool = False,
                residual: Optional[torch.Tensor] = None, row_parallel=None) -> torch.Tensor:
        """``row_parallel``: a ``TensorParallel`` whose ``row_linear`` applies the output projection and sums it over the model
        axis (the caller then adds the bias once)."""
        c = self.config
        q, k, v = self._compute_qkv(x, pos_ids)
        if c.sliding_window is not None and isinstance(mask, AttentionMask) and mask.is_causal:
            mask = mask & AttentionMask.causal(sliding_window=c.sliding_window)
        squeeze = q.dim() == 3
        if squeeze:
            q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
        attn = dot_product_attention(
            q, k, v, mask, attention_dtype=torch.float32 if c.upcast_attn else None, attn_backend=c.attn_backend,
            flash_block_size=c.flash_attention_block_size, logits_soft_cap=c.logits_soft_cap,
            scaling_factor=c.scaling_factor, inference=True)
        if squeeze:
            attn = attn.squeeze(0)
        attn = attn.reshape(*x.shape[:-1], self.local_heads * c.head_size).to(x.dtype)
        if residual is not None:
            if type(self.o_proj) is Linear:
                from ..ops.gemm import linear_residual

                return linear_residual(attn, self.o_proj.weight, None if skip_out_bias else self.o_proj.bias, residual)
            return self.o_proj(attn, skip_bias=skip_out_bias) + residual  # wrapped projections (LoRA, fp8) add it themselves
        if row_parallel is not None:
            return row_parallel.row_linear(attn, self.o_proj)
        return self.o_proj(attn, skip_bias=skip_out_bias)

    def forward_with_residual(self, x, mask, pos_ids, residual):
        """``residual + attention(x)`` with the add done in the output-projection GEMM epilogue."""
        return self.forward(x, mask, pos_ids, residual=residual)

    def paged_decode(self, x: torch.Tensor, kv_cache: "KvPageCache", batch_info, pos_ids: torch.Tensor,
                     residual: Optional[torch.Tensor] = None):
        """Decode/prefill step over packed tokens ``x[T, E]``; writes K/V into the page cache and attends over
        the pages of each sequence (src/levanter/layers/attention.py:1559-1604)."""
        from ..ops import paged_attention as PA

        c = self.config
        q, k, v = self._compute_qkv(x, pos_ids)
        kv_cache = kv_cache.update(batch_info, k, v)
        scale = c.scaling_factor if c.scaling_factor is not None else 1.0 / math.sqrt(c.head_size)
        seg = getattr(batch_info, "prefill_segment_ids", None)
        if seg is not None and x.is_cuda:
            # pure prefill: nothing to read from the cache, so this is causal attention over the packed tokens with one segment
            # per sequence (the flash kernel), instead of the decode kernel walking pages
            m = AttentionMask.causal(sliding_window=c.sliding_window).with_segment_ids(seg.unsqueeze(0), sorted=True)
            out = dot_product_attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), m, attn_backend=c.attn_backend,
                                        logits_soft_cap=c.logits_soft_cap, scaling_factor=c.scaling_factor, inference=True).squeeze(0)
        else:
            out = PA.ragged_paged_attention(q, kv_cache.kv_pages, batch_info.seq_lens, batch_info.page_indices,
                                            batch_info.cu_q_lens, batch_info.num_seqs, sm_scale=scale,
                                            soft_cap=c.logits_soft_cap)
        out = out.reshape(x.shape[0], self.local_heads * c.head_size).to(x.dtype)
        if residual is not None:
            if type(self.o_proj) is Linear:
                from ..ops.gemm import linear_residual

                return linear_residual(out, self.o_proj.weight, self.o_proj.bias, residual), kv_cache
            return self.o_proj(out) + residual, kv_cache
        return self.o_proj(out), kv_cache

    def empty_page_cache(self, max_pages: int, page_size: int, *, dtype=torch.bfloat16, device=None) -> "KvPageCache":
        return KvPageCache.init(max_pages, page_size, self.local_kv, self.config.head_size, dtype=dtype, device=device)


class AttentionWithSink(Attention):
    """Attention with learned sink logits ``sinks[kv_head, q_heads_per_group]``
    (src/levanter/layers/attention.py:2216-2295)."""

    def __init__(self, config: AttentionConfig, **kw):
        super().__init__(config, **kw)
        self.sinks = nn.Parameter(torch.zeros(self.local_kv, config.q_heads_per_group))
        self.sinks.lev_shape = tuple(self.sinks.shape)

    def forward(self, x, mask=None, pos_ids=None):
        c = self.config
        q, k, v = self._compute_qkv(x, pos_ids)
        squeeze = q.dim() == 3
        if squeeze:
            q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
        attn = dot_product_attention_with_sink(q, k, v, self.sinks.reshape(-1), mask,
                                               attention_dtype=torch.float32 if c.upcast_attn else None,
                                               logits_soft_cap=c.logits_soft_cap, scaling_factor=c.scaling_factor)
        if squeeze:
            attn = attn.squeeze(0)
        return self.o_proj(attn.reshape(*x.shape[:-1], -1).to(x.dtype))


# --------------------------------------------------------------------------------------------- MLA
@dataclass(frozen=True)
class MultiHeadLatentAttentionConfig:
    """DeepSeek-V3-style latent attention (src/levanter/layers/attention.py:1994-2060)."""

    hidden_dim: int
    num_heads: int
    kv_lora_rank: int
    q_lora_rank: Optional[int] = None
    qk_rope_head_dim: int = 64
    qk_nope_head_dim: int = 128
    v_head_dim: int = 128
    use_bias: bool = False
    upcast_attn: bool = False
    attn_backend: Optional[AttentionBackend] = None
    flash_attention_block_size: Optional[int] = None
    rope: Optional[RotaryEmbeddingsConfig] = None
    scaling_factor: Optional[float] = None
    logits_soft_cap: Optional[float] = None

    @property
    def qk_head_dim(self):
        return self.qk_nope_head_dim + self.qk_rope_head_dim


class MultiHeadLatentAttention(nn.Module):
    """K/V are reconstructed from a low-rank latent (``kv_lora_rank``) plus a decoupled RoPE key shared by all heads;
    queries optionally pass through their own low-rank bottleneck (src/levanter/layers/attention.py:2063-2213)."""

    def __init__(self, config: MultiHeadLatentAttentionConfig, init_std: float = 0.02):
        super().__init__()
        c = config
        self.config = c
        H = c.num_heads
        if c.q_lora_rank is None:
            self.q_proj = Linear(c.hidden_dim, H * c.qk_head_dim, bias=c.use_bias, init_std=init_std)
            self.q_a_proj = self.q_a_norm = self.q_b_proj = None
        else:
            self.q_proj = None
            self.q_a_proj = Linear(c.hidden_dim, c.q_lora_rank, bias=c.use_bias, init_std=init_std)
            self.q_a_norm = RmsNorm(c.q_lora_rank)
            self.q_b_proj = Linear(c.q_lora_rank, H * c.qk_head_dim, bias=c.use_bias, init_std=init_std)
        self.kv_a_proj = Linear(c.hidden_dim, c.kv_lora_rank + c.qk_rope_head_dim, bias=c.use_bias, init_std=init_std)
        self.kv_a_norm = RmsNorm(c.kv_lora_rank)
        self.kv_b_proj = Linear(c.kv_lora_rank, H * (c.qk_nope_head_dim + c.v_head_dim), bias=c.use_bias, init_std=init_std)
        self.o_proj = Linear(H * c.v_head_dim, c.hidden_dim, bias=c.use_bias, init_std=init_std)
        rope = c.rope if c.rope is not None else DefaultRotaryEmbeddingsConfig()
        self.rot = rope.build(c.qk_rope_head_dim)

    def forward(self, x, mask=None, pos_ids=None):
        c = self.config
        B, S, _ = x.shape
        H = c.num_heads
        if pos_ids is None:
            pos_ids = torch.arange(S, device=x.device)
        q = self.q_proj(x) if self.q_proj is not None else self.q_b_proj(self.q_a_norm(self.q_a_proj(x)))
        q = q.view(B, S, H, c.qk_head_dim)
        q_nope, q_rope = q.split([c.qk_nope_head_dim, c.qk_rope_head_dim], dim=-1)
        kv_a = self.kv_a_proj(x)
        latent, k_rope = kv_a.split([c.kv_lora_rank, c.qk_rope_head_dim], dim=-1)
        kv = self.kv_b_proj(self.kv_a_norm(latent)).view(B, S, H, c.qk_nope_head_dim + c.v_head_dim)
        k_nope, v = kv.split([c.qk_nope_head_dim, c.v_head_dim], dim=-1)
        q_rope = self.rot(q_rope, pos_ids)
        k_rope = self.rot(k_rope.unsqueeze(2), pos_ids).expand(B, S, H, c.qk_rope_head_dim)
        qf = torch.cat([q_nope, q_rope], dim=-1)
        kf = torch.cat([k_nope, k_rope], dim=-1)
        scale = c.scaling_factor if c.scaling_factor is not None else 1.0 / math.sqrt(c.qk_head_dim)
        # value head size differs from the qk head size, so pad V for the shared kernel interface
        out = simple_attention_with_dropout(qf, kf, F.pad(v, (0, c.qk_head_dim - c.v_head_dim)) if c.v_head_dim < c.qk_head_dim else v,
                                            mask, attention_dtype=torch.float32 if c.upcast_attn else None,
                                            logits_soft_cap=c.logits_soft_cap, scaling_factor=scale)
        out = out[..., : c.v_head_dim]
        return self.o_proj(out.reshape(B, S, H * c.v_head_dim).to(x.dtype))


# --------------------------------------------------------------------------------------------- paged KV cache
@dataclass
class KvPageCache:
    """Paged KV storage ``kv_pages[page, slot, 2 * kv_heads, head_size]`` with K at even and V at odd head index
    (src/levanter/layers/attention.py:1638-1707)."""

    kv_pages: torch.Tensor

    @staticmethod
    def init(max_pages: int, page_size: int, kv_heads: int, head_size: int, *, dtype=torch.bfloat16, device=None):
        return KvPageCache(torch.zeros(max_pages, page_size, 2 * kv_heads, head_size, dtype=dtype, device=device))

    @property
    def page_size(self) -> int:
        return self.kv_pages.shape[1]

    def update(self, batch_info, new_k: torch.Tensor, new_v: torch.Tensor) -> "KvPageCache":
        """Scatter ``new_k/new_v [T, kv_heads, D]`` to the (page, slot) destinations of ``batch_info``;
        destinations outside the table (padding tokens) are dropped."""
        from ..ops import paged_attention as PA

        PA.kv_page_write(self.kv_pages, new_k, new_v, batch_info.new_token_dests)
        return self

    def copy_page(self, src_page: int, dst_page: int) -> "KvPageCache":
        self.kv_pages[dst_page].copy_(self.kv_pages[src_page])
        return self


def default_ragged_paged_attention(q, kv_pages, kv_lens, page_indices, cu_q_lens, num_seqs, sm_scale: float = 1.0, soft_cap=None):
    """The plain statement of ragged paged attention (src/levanter/layers/attention.py:1856-1991): per sequence, causal by
    absolute position over the pages it owns.  The engine calls ``ops.paged_attention.ragged_paged_attention`` (the CUDA kernel
    on a B200); this is its oracle under the reference's name."""
    from ..ops.paged_attention import ragged_paged_attention_reference

    return ragged_paged_attention_reference(q, kv_pages, kv_lens, page_indices, cu_q_lens, num_seqs, sm_scale, soft_cap)
