"""Autograd binding of the tcgen05 flash-attention kernels (``csrc/flash_attn.cu``)."""
from __future__ import annotations

import contextlib
import math
from typing import Optional

import torch

from . import lib

_f = {}
_FORCE_ONE_TILE = False  # tests flip this to exercise the one-tile forward kernel on every shape


def _fwd():
    if "f" not in _f:
        c = lib
        _f["f"] = lib.fn("lvb_flash_attn_fwd", [c.c_void_p] * 8 + [c.c_int] * 4 + [c.c_float, c.c_float, c.c_int, c.c_void_p, c.c_void_p])
    return _f["f"]


def _fwd2():
    if "f2" not in _f:
        c = lib
        _f["f2"] = lib.fn("lvb_flash_attn_fwd2", [c.c_void_p] * 8 + [c.c_int] * 4 + [c.c_float, c.c_float, c.c_int, c.c_void_p, c.c_void_p])
    return _f["f2"]


def _bwd():
    if "b" not in _f:
        c = lib
        _f["b"] = lib.fn("lvb_flash_attn_bwd", [c.c_void_p] * 12 + [c.c_int] * 4 + [c.c_float, c.c_float, c.c_int, c.c_void_p, c.c_void_p],
                         launches=2)
    return _f["b"]


def _fwd_hd():
    """Head size 64 or 128, causal or not (one query tile per CTA)."""
    if "fh" not in _f:
        c = lib
        _f["fh"] = lib.fn("lvb_flash_attn_fwd_hd", [c.c_void_p] * 9 + [c.c_int] * 7 + [c.c_float, c.c_float, c.c_int, c.c_void_p, c.c_void_p])
    return _f["fh"]


def _fwd2_hd():
    """Head size 64 or 128, causal or not, two query tiles per CTA (S a multiple of 256)."""
    if "f2h" not in _f:
        c = lib
        _f["f2h"] = lib.fn("lvb_flash_attn_fwd2_hd", [c.c_void_p] * 9 + [c.c_int] * 7 + [c.c_float, c.c_float, c.c_int, c.c_void_p, c.c_void_p])
    return _f["f2h"]


def _bwd_hd():
    if "bh" not in _f:
        c = lib
        _f["bh"] = lib.fn("lvb_flash_attn_bwd_hd", [c.c_void_p] * 12 + [c.c_int] * 7 + [c.c_float, c.c_float, c.c_int, c.c_void_p, c.c_void_p],
                          launches=2)
    return _f["bh"]


def _bwd2():
    if "b2" not in _f:
        c = lib
        _f["b2"] = lib.fn("lvb_flash_attn_bwd2", [c.c_void_p] * 12 + [c.c_int] * 4 + [c.c_float, c.c_float, c.c_int, c.c_void_p, c.c_void_p],
                          launches=2)
    return _f["b2"]


# The backward pass runs on the software-pipelined kernel (``csrc/flash_attn_bwd2.cu``); ``LEVANTER_B200_FLASH_BWD=serial`` selects
# the one-buffer kernel (``csrc/flash_attn_bwd.cu``).
import os as _os

BWD_PIPELINED = _os.environ.get("LEVANTER_B200_FLASH_BWD", "pipelined") != "serial"


# Activation checkpointing that keeps attention outputs (utils/remat.py:checkpoint_layer): during the first pass of a
# checkpointed layer the forward below appends (o, lse) to ``_keep``; during the recomputation it takes them back from
# ``_replay`` in the same order and launches nothing.
_keep: Optional[list] = None
_replay: Optional[list] = None


@contextlib.contextmanager
def keeping_outputs(store: list):
    global _keep
    prev, _keep = _keep, store
    try:
        yield store
    finally:
        _keep = prev


@contextlib.contextmanager
def replaying_outputs(store: list):
    global _replay
    prev, _replay = _replay, list(store)
    try:
        yield
    finally:
        _replay = prev


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_seg, k_seg, scale, soft_cap, window, kblock_lo=None, causal=True, sink=None):
        B, S, Hq, D = q.shape
        Sk = k.shape[1]  # differs from S only for cross attention (no causal part)
        general = D != 128 or not causal  # the kernels templated on the head size; the pipelined backward is causal, 128 only
        if sink is not None:
            sink = sink.detach().float().contiguous()
        Hkv = k.shape[2]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        if _replay:
            o, lse2 = _replay.pop(0)
            if o.shape != q.shape:
                raise RuntimeError("the recomputation of a checkpointed layer called attention in a different order than its first pass")
        else:
            o = torch.empty_like(q)
            lse2 = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
            # two query tiles per CTA when the sequence allows it; the one-tile kernel covers the remaining lengths
            if general or sink is not None:
                rc = (_fwd2_hd() if (S % 256 == 0 and not _FORCE_ONE_TILE) else _fwd_hd())(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse2.data_ptr(), lib.ptr(q_seg), lib.ptr(k_seg),
                               lib.ptr(kblock_lo) if causal else 0, lib.ptr(sink), B, S, Sk, Hq, Hkv, D, int(bool(causal)), float(scale),
                               float(soft_cap or 0.0), int(window or 0), lib.status_buffer().data_ptr(), lib.stream_ptr())
            else:
                fwd = _fwd2() if (S % 256 == 0 and not _FORCE_ONE_TILE) else _fwd()
                rc = fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse2.data_ptr(), lib.ptr(q_seg), lib.ptr(k_seg),
                         lib.ptr(kblock_lo), B, S, Hq, Hkv, float(scale), float(soft_cap or 0.0), int(window or 0),
                         lib.status_buffer().data_ptr(), lib.stream_ptr())
            lib.check_rc(rc, "lvb_flash_attn_fwd")
            if _keep is not None:
                _keep.append((o, lse2))
        ctx.save_for_backward(q, k, v, o, lse2, q_seg, k_seg, sink)
        ctx.args = (scale, soft_cap, window, causal, general)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse2, q_seg, k_seg, sink = ctx.saved_tensors
        scale, soft_cap, window, causal, general = ctx.args
        B, S, Hq, D = q.shape
        Hkv = k.shape[2]
        do = do.contiguous()
        if do.dtype != torch.bfloat16:
            do = do.to(torch.bfloat16)
        dq32 = torch.zeros(B, S, Hq, D, dtype=torch.float32, device=q.device)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        delta = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
        if general:
            rc = _bwd_hd()(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse2.data_ptr(), delta.data_ptr(),
                           dq32.data_ptr(), dk.data_ptr(), dv.data_ptr(), lib.ptr(q_seg), lib.ptr(k_seg), B, S, k.shape[1], Hq, Hkv, D, int(bool(causal)),
                           float(scale), float(soft_cap or 0.0), int(window or 0), lib.status_buffer().data_ptr(), lib.stream_ptr())
        else:
            rc = (_bwd2() if BWD_PIPELINED else _bwd())(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse2.data_ptr(), delta.data_ptr(),
                        dq32.data_ptr(), dk.data_ptr(), dv.data_ptr(), lib.ptr(q_seg), lib.ptr(k_seg), B, S, Hq, Hkv, float(scale),
                        float(soft_cap or 0.0), int(window or 0), lib.status_buffer().data_ptr(), lib.stream_ptr())
        lib.check_rc(rc, "lvb_flash_attn_bwd")
        dsink = None
        if sink is not None and ctx.needs_input_grad[10]:
            # the sink column's probability is 2^(sink log2 e - lse2); its value row is zero, so its logit's gradient is
            # -p_sink * delta summed over batch and queries (delta = rowsum(dO * O), left in the scratch by the kernel)
            dsink = -(torch.exp2(sink.view(1, Hq, 1) * 1.4426950408889634 - lse2) * delta).sum(dim=(0, 2))
        return dq32.to(torch.bfloat16), dk, dv, None, None, None, None, None, None, None, dsink


PAD_SEGMENT = -2  # segment id of the rows added to bring a sequence to a multiple of 256: they see only one another


def flash_attention_cuda(q, k, v, mask, *, logits_soft_cap: Optional[float] = None, scaling_factor: Optional[float] = None,
                         sink: Optional[torch.Tensor] = None):
    """``q[B,S,Hq,D]``, ``k/v[B,S,Hkv,D]`` bf16, D = 64 or 128; ``mask`` is ``None`` (every key visible) or an ``AttentionMask``
    made of causal / sliding-window / segment-id parts.  A sequence length that is not a multiple of 256 is padded, and the
    padding rows get a segment id of their own so that no real query sees them.  ``sink [Hq]``: a learned logit per head that
    joins the softmax denominator (a key column whose value row is zero)."""
    scale = scaling_factor if scaling_factor is not None else 1.0 / math.sqrt(q.shape[-1])
    q_seg = k_seg = None
    window = 0
    causal = False
    B, S, Sk = q.shape[0], q.shape[1], k.shape[1]
    if mask is not None:
        causal = bool(mask.is_causal)
        window = mask.sliding_window or 0
        if mask.segment_ids is not None:
            q_seg, k_seg = mask.segment_ids
            q_seg = q_seg.to(torch.int32).expand(B, S).contiguous()
            k_seg = k_seg.to(torch.int32).expand(B, Sk).contiguous()
    if causal and Sk != S:
        raise ValueError("a causal mask needs as many keys as queries")
    # queries to a multiple of 256 (the two-tile forward kernel; the one-tile kernel takes any multiple of 128 but is far slower),
    # keys to a multiple of 128, or of 256 with the queries when the lengths are tied by a causal mask
    pad = (-S) % 256
    pad_k = pad if Sk == S else (-Sk) % 128
    if pad or pad_k:
        if q_seg is None:
            q_seg = torch.zeros(B, S, dtype=torch.int32, device=q.device)
            k_seg = torch.zeros(B, Sk, dtype=torch.int32, device=q.device)
        q_seg = torch.nn.functional.pad(q_seg, (0, pad), value=PAD_SEGMENT)
        k_seg = torch.nn.functional.pad(k_seg, (0, pad_k), value=PAD_SEGMENT)
        q = torch.nn.functional.pad(q, (0, 0, 0, 0, 0, pad))
        k, v = (torch.nn.functional.pad(t, (0, 0, 0, 0, 0, pad_k)) for t in (k, v))
    kblock_lo = None
    if q_seg is not None and causal and not pad and getattr(mask, "segments_sorted", False) and not torch.is_grad_enabled():
        # packed sequences: per block of 128 queries, the first block of 128 keys of the first query's sequence (padding ids < 0
        # sort last); the forward kernels start their key loop there instead of at the beginning of the packed batch
        big = torch.iinfo(torch.int32).max
        ks = torch.where(k_seg < 0, torch.full_like(k_seg, big), k_seg)
        qs = torch.where(q_seg < 0, torch.full_like(q_seg, big), q_seg)[:, ::128].contiguous()
        kblock_lo = (torch.searchsorted(ks, qs) // 128).to(torch.int32).contiguous()
    o = _FlashFn.apply(q, k, v, q_seg, k_seg, scale, logits_soft_cap, window, kblock_lo, causal, sink)
    return o[:, :S] if pad else o
