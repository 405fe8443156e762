"""Flash attention on tcgen05 tensor cores (``csrc/flash_attn*.cu``): head sizes 64 and 128, causal (with sliding window) or
not, GQA, segment ids, any sequence length (padded to a multiple of 128 behind a segment id of its own).

Replaces the reference's fused-attention call sites (TransformerEngine/cuDNN on GPU, src/levanter/layers/attention.py:
533-544; pure-JAX flash attention, src/levanter/models/flash_attention.py:143-385)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import lib


def kernel_built() -> bool:
    try:
        return hasattr(lib.load(), "lvb_flash_attn_fwd")
    except Exception:
        return False


def supported(q, k, v, mask, bias, no_dropout: bool, attention_dtype) -> bool:
    from ..layers.attention import AttentionMask, _structured_only

    if not (q.is_cuda and lib.available() and kernel_built()):
        return False
    if bias is not None or not no_dropout:
        return False
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        return False
    if attention_dtype is not None and attention_dtype not in (torch.float32, torch.bfloat16):
        return False
    if q.shape[-1] not in (64, 128) or v.shape[-1] != q.shape[-1] or k.shape[-1] != q.shape[-1]:
        return False
    if mask is not None and not isinstance(mask, AttentionMask):
        return False
    if q.shape[1] != k.shape[1] and (q.shape[1] == 1 or (isinstance(mask, AttentionMask) and mask.is_causal)):
        return False  # different query and key lengths: cross attention only (no causal part); single-token decode steps stay off
    if isinstance(mask, AttentionMask) and not mask.is_causal and mask.sliding_window:
        return False
    return _structured_only(mask)


def flash_attention(q, k, v, mask, *, logits_soft_cap: Optional[float] = None, scaling_factor: Optional[float] = None, sink=None):
    from ._flash_impl import flash_attention_cuda

    return flash_attention_cuda(q, k, v, mask, logits_soft_cap=logits_soft_cap, scaling_factor=scaling_factor, sink=sink)
