"""Paged-KV attention for the inference engine: KV page write and ragged paged attention
(src/levanter/layers/attention.py:1694-1695 and :1856-1991).  PyTorch statement; the CUDA kernels plug in here."""
from __future__ import annotations

import math
from typing import Optional

import torch

INVALID = 2_000_000


def kv_page_write(kv_pages: torch.Tensor, new_k: torch.Tensor, new_v: torch.Tensor, dests: torch.Tensor) -> None:
    """Write ``new_k/new_v [T, KV, D]`` to flat slots ``dests[T]`` (= page * page_size + slot) of
    ``kv_pages[P, page_size, 2*KV, D]``; K goes to even head indices, V to odd.  Out-of-range slots are dropped."""
    P, ps, H2, D = kv_pages.shape
    flat = kv_pages.view(P * ps, H2, D)
    valid = (dests >= 0) & (dests < P * ps)
    idx = torch.where(valid, dests, torch.zeros_like(dests)).long()
    if bool(valid.all()):
        flat[idx, 0::2] = new_k.to(kv_pages.dtype)
        flat[idx, 1::2] = new_v.to(kv_pages.dtype)
    else:
        sel = valid.nonzero().squeeze(-1)
        flat[idx[sel], 0::2] = new_k[sel].to(kv_pages.dtype)
        flat[idx[sel], 1::2] = new_v[sel].to(kv_pages.dtype)


def ragged_paged_attention(q: torch.Tensor, kv_pages: torch.Tensor, kv_lens: torch.Tensor, page_indices: torch.Tensor,
                           cu_q_lens: torch.Tensor, num_seqs, sm_scale: float = 1.0, soft_cap: Optional[float] = None) -> torch.Tensor:
    """Causal attention of packed query tokens ``q[T, H, D]`` over each sequence's pages.

    Sequence ``i`` owns query rows ``cu_q_lens[i]:cu_q_lens[i+1]``; its keys are the first ``kv_lens[i]`` slots of pages
    ``page_indices[i]``; query ``j`` of the sequence sits at absolute position ``kv_lens[i] - q_len + j``."""
    T, H, D = q.shape
    P, ps, H2, _ = kv_pages.shape
    KV = H2 // 2
    G = H // KV
    out = torch.zeros_like(q)
    n = int(num_seqs)
    cu = cu_q_lens.tolist()
    lens = kv_lens.tolist()
    for i in range(n):
        q0, q1 = cu[i], cu[i + 1]
        ql = q1 - q0
        kl = lens[i]
        if ql <= 0 or kl <= 0:
            continue
        npages = (kl + ps - 1) // ps
        pages = page_indices[i, :npages].long()
        kv = kv_pages[pages].reshape(npages * ps, H2, D)[:kl]
        k = kv[:, 0::2].float()
        v = kv[:, 1::2].float()
        qi = q[q0:q1].float().view(ql, KV, G, D) * sm_scale
        s = torch.einsum("qkgd,skd->kgqs", qi, k)
        if soft_cap is not None:
            s = torch.tanh(s / soft_cap) * soft_cap
        qpos = torch.arange(ql, device=q.device) + (kl - ql)
        kpos = torch.arange(kl, device=q.device)
        s = s.masked_fill(~(qpos[:, None] >= kpos[None, :]), -float("inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("kgqs,skd->qkgd", p, v)
        out[q0:q1] = o.reshape(ql, H, D).to(q.dtype)
    return out
