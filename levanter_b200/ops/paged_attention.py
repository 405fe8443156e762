"""Paged-KV attention for the inference engine: KV page write and ragged paged attention
(src/levanter/layers/attention.py:1694-1695 and :1856-1991).

On a B200 both run as CUDA kernels (``csrc/paged_attention.cu``) that read sequence boundaries and lengths from device
arrays, so a decode step never synchronises with the host.  The PyTorch statements below are the CPU path and the test
oracle."""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import lib

INVALID = 2_000_000
_f = {}
_scratch = {}


def _use_kernel(*tensors) -> bool:
    return all(t.is_cuda for t in tensors) and lib.available()


def kv_page_write(kv_pages: torch.Tensor, new_k: torch.Tensor, new_v: torch.Tensor, dests: torch.Tensor) -> None:
    """Write ``new_k/new_v [T, KV, D]`` to flat slots ``dests[T]`` (= page * page_size + slot) of
    ``kv_pages[P, page_size, 2*KV, D]``; K goes to even head indices, V to odd.  Out-of-range slots are dropped."""
    P, ps, H2, D = kv_pages.shape
    if _use_kernel(kv_pages, new_k, new_v, dests) and kv_pages.dtype == torch.bfloat16 and D % 8 == 0:
        c = lib
        if "w" not in _f:
            _f["w"] = lib.fn("lvb_kv_page_write", [c.c_void_p] * 4 + [c.c_int] * 3 + [c.c_longlong, c.c_void_p])
        k = new_k.to(torch.bfloat16).contiguous()
        v = new_v.to(torch.bfloat16).contiguous()
        d = dests.to(torch.int32).contiguous()
        rc = _f["w"](kv_pages.data_ptr(), k.data_ptr(), v.data_ptr(), d.data_ptr(), k.shape[0], H2 // 2, D, P * ps, lib.stream_ptr())
        lib.check_rc(rc, "lvb_kv_page_write")
        return
    flat = kv_pages.view(P * ps, H2, D)
    valid = (dests >= 0) & (dests < P * ps)
    sel = valid.nonzero().squeeze(-1)
    idx = dests[sel].long()
    flat[idx, 0::2] = new_k[sel].to(kv_pages.dtype)
    flat[idx, 1::2] = new_v[sel].to(kv_pages.dtype)


def ragged_paged_attention(q: torch.Tensor, kv_pages: torch.Tensor, kv_lens: torch.Tensor, page_indices: torch.Tensor,
                           cu_q_lens: torch.Tensor, num_seqs, sm_scale: float = 1.0, soft_cap: Optional[float] = None) -> torch.Tensor:
    """Causal attention of packed query tokens ``q[T, H, D]`` over each sequence's pages.

    Sequence ``i`` owns query rows ``cu_q_lens[i]:cu_q_lens[i+1]``; its keys are the first ``kv_lens[i]`` slots of pages
    ``page_indices[i]``; query ``j`` of the sequence sits at absolute position ``kv_lens[i] - q_len + j``.  Rows past
    ``cu_q_lens[num_seqs]`` are padding and come back as zeros."""
    T, H, D = q.shape
    P, ps, H2, _ = kv_pages.shape
    KV = H2 // 2
    if _use_kernel(q, kv_pages) and q.dtype == torch.bfloat16 and kv_pages.dtype == torch.bfloat16 and D in (64, 128, 256) \
            and H // KV <= 16:
        return _paged_attention_cuda(q, kv_pages, kv_lens, page_indices, cu_q_lens, num_seqs, sm_scale, soft_cap)
    return ragged_paged_attention_reference(q, kv_pages, kv_lens, page_indices, cu_q_lens, num_seqs, sm_scale, soft_cap)


def _paged_attention_cuda(q, kv_pages, kv_lens, page_indices, cu_q_lens, num_seqs, sm_scale, soft_cap):
    c = lib
    if "a" not in _f:
        _f["a"] = lib.fn("lvb_paged_attention", [c.c_void_p] * 9 + [c.c_int] * 8 + [c.c_float, c.c_float, c.c_void_p], launches=2)
        _f["parts"] = lib.fn("lvb_paged_attention_parts", [c.c_int], launches=0)
    T, H, D = q.shape
    P, ps, H2, _ = kv_pages.shape
    S, PP = page_indices.shape
    dev = q.device
    i32 = lambda t: t.to(device=dev, dtype=torch.int32).contiguous()  # noqa: E731
    ns = num_seqs if isinstance(num_seqs, torch.Tensor) else torch.tensor(int(num_seqs), dtype=torch.int32)
    ns = i32(ns.reshape(1))
    parts = _f["parts"](PP * ps)
    key = (dev, T, H, parts, D)
    if parts > 1 and key not in _scratch:
        _scratch.clear()  # one live shape at a time: the engine calls with fixed T per phase
        _scratch[key] = (torch.empty(T * H * parts * D, dtype=torch.float32, device=dev),
                         torch.empty(T * H * parts * 2, dtype=torch.float32, device=dev))
    po, pml = _scratch.get(key, (None, None))
    qc = q.contiguous()
    out = torch.empty_like(qc)
    rc = _f["a"](qc.data_ptr(), kv_pages.data_ptr(), i32(kv_lens).data_ptr(), i32(page_indices).data_ptr(), i32(cu_q_lens).data_ptr(),
                 ns.data_ptr(), out.data_ptr(), lib.ptr(po), lib.ptr(pml), T, H, H2 // 2, D, S, PP, ps, P, float(sm_scale),
                 float(soft_cap or 0.0), lib.stream_ptr())
    lib.check_rc(rc, "lvb_paged_attention")
    return out


def ragged_paged_attention_reference(q, kv_pages, kv_lens, page_indices, cu_q_lens, num_seqs, sm_scale: float = 1.0,
                                     soft_cap: Optional[float] = None) -> torch.Tensor:
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
        if ql <= 0 or kl <= 0 or kl == INVALID:
            continue
        npages = (kl + ps - 1) // ps
        pages = page_indices[i, :npages].long()
        kv = kv_pages[pages].reshape(npages * ps, H2, D)[:kl]
        k = kv[:, 0::2].float()
        v = kv[:, 1::2].float()
        qi = q[q0:q1].float().view(ql, KV, G, D) * sm_scale
        s = torch.einsum("qkgd,skd->kgqs", qi, k)
        if soft_cap is not None and soft_cap > 0:
            s = torch.tanh(s / soft_cap) * soft_cap
        qpos = torch.arange(ql, device=q.device) + (kl - ql)
        kpos = torch.arange(kl, device=q.device)
        s = s.masked_fill(~(qpos[:, None] >= kpos[None, :]), -float("inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("kgqs,skd->qkgd", p, v)
        out[q0:q1] = o.reshape(ql, H, D).to(q.dtype)
    return out
