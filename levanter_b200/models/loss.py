"""Next-token cross-entropy, optionally fused with the LM head so the ``[tokens, vocab]`` logits never exist.

API and semantics of the reference's ``maybe_fused_next_token_loss`` (src/levanter/models/loss.py:16-90): targets are
the tokens rolled left by one, the last position is masked out, the loss is ``logZ - logit[target]`` plus an optional
``logsumexp_weight * logZ^2`` z-loss, optional tanh ``logit_soft_cap``, and the default reduction is the masked mean
``sum(loss * mask) / sum(mask)`` (:159,212).
"""
from __future__ import annotations

from typing import Callable, Optional, Union

import torch

from ..ops import cross_entropy as CE

Reduction = Union[None, str, Callable]


def _reduce(loss: torch.Tensor, mask: Optional[torch.Tensor], reduction: Reduction, reduction_dim=None):
    if reduction is None:
        return loss if mask is None else loss * mask
    if callable(reduction):
        return reduction(loss, mask)
    if reduction == "mean":
        if mask is None:
            return loss.mean() if reduction_dim is None else loss.mean(reduction_dim)
        m = mask.to(loss.dtype)
        if reduction_dim is None:
            return (loss * m).sum() / m.sum()
        return (loss * m).sum(reduction_dim) / m.sum(reduction_dim)
    if reduction == "sum":
        l = loss if mask is None else loss * mask.to(loss.dtype)
        return l.sum() if reduction_dim is None else l.sum(reduction_dim)
    raise ValueError(f"unknown reduction {reduction!r}")


def cross_entropy_and_logsumexp_penalty(logits: torch.Tensor, targets: torch.Tensor, *, logsumexp_weight: Optional[float] = None,
                                        logit_soft_cap: Optional[float] = None):
    """Per-position loss from materialised logits (fp32 math). Returns ``(loss, logZ)``."""
    lf = logits.float()
    if logit_soft_cap is not None:
        lf = torch.tanh(lf / logit_soft_cap) * logit_soft_cap
    logz = torch.logsumexp(lf, dim=-1)
    tl = lf.gather(-1, targets.clamp(0, lf.shape[-1] - 1).unsqueeze(-1).long()).squeeze(-1)
    loss = logz - tl
    if logsumexp_weight:
        loss = loss + logsumexp_weight * logz * logz
    return loss, logz


class _BlockwiseCE(torch.autograd.Function):
    """Vocab-blocked CE in PyTorch ops: online logsumexp forward, block recompute backward
    (src/levanter/models/loss.py:251-507).  Used off-GPU and as the oracle of the fused kernel."""

    @staticmethod
    def forward(ctx, x, w, targets, block, soft_cap, dtype):
        T, E = x.shape
        V = w.shape[0]
        m = torch.full((T,), -float("inf"), dtype=torch.float32, device=x.device)
        s = torch.zeros(T, dtype=torch.float32, device=x.device)
        tl = torch.zeros(T, dtype=torch.float32, device=x.device)
        xd = x.to(dtype)
        for v0 in range(0, V, block):
            wb = w[v0:v0 + block].to(dtype)
            lg = (xd @ wb.t()).float()
            if soft_cap is not None:
                lg = torch.tanh(lg / soft_cap) * soft_cap
            bm = lg.amax(-1)
            nm = torch.maximum(m, bm)
            s = s * torch.exp(m - nm) + torch.exp(lg - nm.unsqueeze(-1)).sum(-1)
            m = nm
            inb = (targets >= v0) & (targets < v0 + wb.shape[0])
            idx = (targets - v0).clamp(0, wb.shape[0] - 1)
            tl = tl + torch.where(inb, lg.gather(-1, idx.unsqueeze(-1)).squeeze(-1), torch.zeros_like(tl))
        logz = m + torch.log(s)
        ctx.save_for_backward(x, w, targets, logz)
        ctx.block, ctx.soft_cap, ctx.dtype = block, soft_cap, dtype
        return logz - tl, logz

    @staticmethod
    def backward(ctx, g_loss, g_logz):
        x, w, targets, logz = ctx.saved_tensors
        block, soft_cap, dtype = ctx.block, ctx.soft_cap, ctx.dtype
        T, E = x.shape
        V = w.shape[0]
        g_loss = g_loss.float()
        g_tot = g_loss + (g_logz.float() if g_logz is not None else 0.0)
        dx = torch.zeros(T, E, dtype=torch.float32, device=x.device)
        dw = torch.zeros(V, E, dtype=torch.float32, device=x.device)
        xd = x.to(dtype)
        for v0 in range(0, V, block):
            wb = w[v0:v0 + block].to(dtype)
            raw = (xd @ wb.t()).float()
            lg = raw
            dcap = None
            if soft_cap is not None:
                th = torch.tanh(raw / soft_cap)
                lg = th * soft_cap
                dcap = 1 - th * th
            p = torch.exp(lg - logz.unsqueeze(-1))
            dl = g_tot.unsqueeze(-1) * p
            inb = (targets >= v0) & (targets < v0 + wb.shape[0])
            idx = (targets - v0).clamp(0, wb.shape[0] - 1)
            dl.scatter_add_(-1, idx.unsqueeze(-1), -(g_loss * inb.float()).unsqueeze(-1))
            if dcap is not None:
                dl = dl * dcap
            dx += dl @ wb.float()
            dw[v0:v0 + wb.shape[0]] = dl.t() @ xd.float()
        return dx.to(x.dtype), dw.to(w.dtype), None, None, None, None


def fused_cross_entropy_loss_and_logsumexp_penalty(pred_embeddings, pred_lm_head, target_ids, *, block_size: Optional[int],
                                                   logsumexp_weight: Optional[float] = None, dtype=torch.float32,
                                                   logit_soft_cap: Optional[float] = None):
    """Per-position loss of ``pred_embeddings[..., E] @ pred_lm_head[V, E].T`` vs ``target_ids`` without full logits."""
    lead = pred_embeddings.shape[:-1]
    x = pred_embeddings.reshape(-1, pred_embeddings.shape[-1])
    t = target_ids.reshape(-1)
    if CE.kernel_ok(x, pred_lm_head):
        loss, _ = CE.fused_linear_cross_entropy(x, pred_lm_head, t, soft_cap=logit_soft_cap, z_weight=logsumexp_weight)
        return loss.view(lead)
    block = block_size or pred_lm_head.shape[0]
    loss, logz = _BlockwiseCE.apply(x, pred_lm_head, t.long(), block, logit_soft_cap, dtype or torch.float32)
    if logsumexp_weight:
        loss = loss + logsumexp_weight * logz * logz
    return loss.view(lead)


def maybe_fused_next_token_loss(pred_embeddings: torch.Tensor, pred_lm_head: torch.Tensor, true_ids: torch.Tensor,
                                loss_mask: Optional[torch.Tensor] = None, reduction: Reduction = "mean", reduction_dim=None,
                                logsumexp_weight: Optional[float] = None, block_size: Optional[int] = None,
                                dtype: Optional[torch.dtype] = torch.float32, logit_soft_cap: Optional[float] = None):
    """Next-token loss from final hidden states ``[B, S, E]`` and the LM head ``[V, E]``.

    With ``block_size=None`` on a machine without the fused kernel the logits are materialised; otherwise the fused
    (never-materialising) path is taken."""
    S = true_ids.shape[-1]
    target = torch.roll(true_ids, shifts=-1, dims=-1)
    not_last = torch.ones(S, dtype=torch.float32, device=true_ids.device)
    not_last[-1] = 0.0
    mask = not_last if loss_mask is None else loss_mask.to(torch.float32) * not_last
    if mask.dim() < target.dim():
        mask = mask.expand(target.shape)
    x2 = pred_embeddings.reshape(-1, pred_embeddings.shape[-1])
    if block_size is None and not CE.kernel_ok(x2, pred_lm_head):
        logits = (pred_embeddings.to(dtype) @ pred_lm_head.to(dtype).t()) if dtype is not None else pred_embeddings @ pred_lm_head.t()
        loss, _ = cross_entropy_and_logsumexp_penalty(logits, target, logsumexp_weight=logsumexp_weight, logit_soft_cap=logit_soft_cap)
    else:
        loss = fused_cross_entropy_loss_and_logsumexp_penalty(pred_embeddings, pred_lm_head, target, block_size=block_size,
                                                              logsumexp_weight=logsumexp_weight, dtype=dtype,
                                                              logit_soft_cap=logit_soft_cap)
    return _reduce(loss, mask, reduction, reduction_dim)


def next_token_loss(logits: torch.Tensor, true_ids: torch.Tensor, loss_mask: Optional[torch.Tensor] = None,
                    reduction: Reduction = "mean", reduction_dim=None, logsumexp_weight: Optional[float] = None,
                    logit_soft_cap: Optional[float] = None):
    """Next-token loss from materialised logits ``[B, S, V]`` (src/levanter/models/loss.py:93-160)."""
    S = true_ids.shape[-1]
    target = torch.roll(true_ids, shifts=-1, dims=-1)
    not_last = torch.ones(S, dtype=torch.float32, device=true_ids.device)
    not_last[-1] = 0.0
    mask = not_last if loss_mask is None else loss_mask.to(torch.float32) * not_last
    if mask.dim() < target.dim():
        mask = mask.expand(target.shape)
    loss, _ = cross_entropy_and_logsumexp_penalty(logits, target, logsumexp_weight=logsumexp_weight, logit_soft_cap=logit_soft_cap)
    return _reduce(loss, mask, reduction, reduction_dim)
