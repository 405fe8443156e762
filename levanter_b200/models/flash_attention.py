"""Blockwise (FlashAttention-2 style) attention written with PyTorch ops and a hand-written backward.

The counterpart of the reference's pure-JAX flash attention (src/levanter/models/flash_attention.py:143-385):
the forward walks query blocks and, for each, key blocks (stopping at the diagonal for causal masks), keeping a
running max / sum, and saves ``(O, L = max + log sumexp)``; the backward walks key blocks outside and query blocks
inside with ``D = rowsum(dO * O)``, reducing dK/dV over the query heads of a KV group.  It is the memory-efficient
path on machines without a B200 and the oracle for the CUDA kernel tests.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

BLOCK_SIZE = 1024


def _block_mask(mask, Sq, Sk, qs, qn, ks, kn, device):
    from ..layers.attention import materialize_mask

    return materialize_mask(mask, Sq, Sk, device=device, q_slice=(qs, qn), k_slice=(ks, kn))


def _causal_limit(mask, q_end: int, Sk: int) -> int:
    """Last key index (exclusive) any query in a block ending at ``q_end`` can see under a plain causal mask."""
    from ..layers.attention import AttentionMask

    if isinstance(mask, AttentionMask) and mask.is_causal:
        off = mask.causal_offset
        if off is None or (isinstance(off, int)):
            return min(Sk, q_end + int(off or 0))
    return Sk


def _window_start(mask, q_start: int) -> int:
    from ..layers.attention import AttentionMask

    if isinstance(mask, AttentionMask) and mask.sliding_window is not None:
        return max(0, q_start - mask.sliding_window + 1)
    return 0


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, block, scale, soft_cap, dtype):
        B, Sq, H, D = q.shape
        Sk, KV = k.shape[1], k.shape[2]
        G = H // KV
        cd = dtype or torch.float32
        qg = q.view(B, Sq, KV, G, D)
        o = torch.zeros(B, Sq, KV, G, D, dtype=torch.float32, device=q.device)
        lse = torch.full((B, KV, G, Sq), -float("inf"), dtype=torch.float32, device=q.device)
        for qs in range(0, Sq, block):
            qn = min(block, Sq - qs)
            qb = qg[:, qs:qs + qn].to(cd) * scale
            m = torch.full((B, KV, G, qn), -float("inf"), dtype=torch.float32, device=q.device)
            l = torch.zeros(B, KV, G, qn, dtype=torch.float32, device=q.device)
            acc = torch.zeros(B, KV, G, qn, D, dtype=torch.float32, device=q.device)
            k_hi = _causal_limit(mask, qs + qn, Sk)
            k_lo = (_window_start(mask, qs) // block) * block
            for ks in range(k_lo, k_hi, block):
                kn = min(block, Sk - ks)
                kb = k[:, ks:ks + kn].to(cd)
                vb = v[:, ks:ks + kn].float()
                s = torch.einsum("bqkgd,bskd->bkgqs", qb, kb).float()
                if soft_cap is not None:
                    s = torch.tanh(s / soft_cap) * soft_cap
                bm = _block_mask(mask, Sq, Sk, qs, qn, ks, kn, q.device)
                if bm is not None:
                    bm = bm if bm.dim() == 2 else bm.reshape(bm.shape[0], 1, 1, qn, kn) if bm.dim() == 4 and bm.shape[1] == 1 else bm.unsqueeze(2)
                    s = torch.where(bm, s, torch.full_like(s, -float("inf")))
                m_new = torch.maximum(m, s.amax(-1))
                m_safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
                p = torch.exp(s - m_safe.unsqueeze(-1))
                alpha = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, -float("inf")), m) - m_safe)
                alpha = torch.where(torch.isinf(m), torch.zeros_like(alpha), alpha)
                l = l * alpha + p.sum(-1)
                acc = acc * alpha.unsqueeze(-1) + torch.einsum("bkgqs,bskd->bkgqd", p, vb)
                m = m_new
            l_safe = torch.where(l == 0, torch.ones_like(l), l)
            o[:, qs:qs + qn] = (acc / l_safe.unsqueeze(-1)).permute(0, 3, 1, 2, 4)
            lse[..., qs:qs + qn] = torch.where(l == 0, torch.full_like(m, -float("inf")), m + torch.log(l_safe))
        out = o.view(B, Sq, H, D).to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.mask, ctx.block, ctx.scale, ctx.soft_cap, ctx.cd = mask, block, scale, soft_cap, cd
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        mask, block, scale, soft_cap, cd = ctx.mask, ctx.block, ctx.scale, ctx.soft_cap, ctx.cd
        B, Sq, H, D = q.shape
        Sk, KV = k.shape[1], k.shape[2]
        G = H // KV
        qg = q.view(B, Sq, KV, G, D)
        dog = do.reshape(B, Sq, KV, G, D).float()
        og = out.view(B, Sq, KV, G, D).float()
        delta = (dog * og).sum(-1).permute(0, 2, 3, 1)  # [B, KV, G, Sq]
        dq = torch.zeros(B, Sq, KV, G, D, dtype=torch.float32, device=q.device)
        dk = torch.zeros(B, Sk, KV, D, dtype=torch.float32, device=q.device)
        dv = torch.zeros(B, Sk, KV, D, dtype=torch.float32, device=q.device)
        for ks in range(0, Sk, block):
            kn = min(block, Sk - ks)
            kb = k[:, ks:ks + kn].to(cd)
            vb = v[:, ks:ks + kn].float()
            for qs in range(0, Sq, block):
                qn = min(block, Sq - qs)
                if ks >= _causal_limit(mask, qs + qn, Sk):
                    continue
                if ks + kn <= _window_start(mask, qs):
                    continue
                qb = qg[:, qs:qs + qn].to(cd) * scale
                raw = torch.einsum("bqkgd,bskd->bkgqs", qb, kb).float()
                s = raw
                if soft_cap is not None:
                    th = torch.tanh(raw / soft_cap)
                    s = th * soft_cap
                bm = _block_mask(mask, Sq, Sk, qs, qn, ks, kn, q.device)
                if bm is not None:
                    bm = bm if bm.dim() == 2 else bm.reshape(bm.shape[0], 1, 1, qn, kn) if bm.dim() == 4 and bm.shape[1] == 1 else bm.unsqueeze(2)
                    s = torch.where(bm, s, torch.full_like(s, -float("inf")))
                L = lse[..., qs:qs + qn]
                L_safe = torch.where(torch.isinf(L), torch.zeros_like(L), L)
                p = torch.exp(s - L_safe.unsqueeze(-1))
                p = torch.where(torch.isinf(L).unsqueeze(-1), torch.zeros_like(p), p)
                dob = dog[:, qs:qs + qn]
                dv[:, ks:ks + kn] += torch.einsum("bkgqs,bqkgd->bskd", p, dob)
                dp = torch.einsum("bqkgd,bskd->bkgqs", dob, vb)
                ds = p * (dp - delta[..., qs:qs + qn].unsqueeze(-1))
                if soft_cap is not None:
                    ds = ds * (1 - th * th)
                dq[:, qs:qs + qn] += torch.einsum("bkgqs,bskd->bqkgd", ds, kb.float()) * scale
                dk[:, ks:ks + kn] += torch.einsum("bkgqs,bqkgd->bskd", ds, qb.float())
        return dq.view(B, Sq, H, D).to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None


def flash_attention(q, k, v, mask=None, *, dropout: float = 0.0, inference: bool = True, block_size: Optional[int] = None,
                    dtype: Optional[torch.dtype] = None, logits_soft_cap: Optional[float] = None,
                    scaling_factor: Optional[float] = None) -> torch.Tensor:
    """``q[B,Sq,H,D]``, ``k/v[B,Sk,KV,D]`` -> ``[B,Sq,H,D]``.  Falls back to vanilla attention for dropout."""
    if dropout > 0.0 and not inference:
        from ..layers.attention import simple_attention_with_dropout

        return simple_attention_with_dropout(q, k, v, mask, dropout=dropout, inference=False, attention_dtype=dtype,
                                             logits_soft_cap=logits_soft_cap, scaling_factor=scaling_factor)
    block = block_size or BLOCK_SIZE
    scale = scaling_factor if scaling_factor is not None else 1.0 / math.sqrt(q.shape[-1])
    return _FlashFn.apply(q, k, v, mask, block, scale, logits_soft_cap, dtype)
