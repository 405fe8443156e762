"""Rotary embedding application (``csrc/elementwise.cu``), in place on fresh q/k projections.

Reference: src/levanter/layers/rotary.py:34-46 (and the llama3 / yarn variants, which only change the table)."""
from __future__ import annotations

import torch

from . import lib
from ..layers.rotary import RotaryEmbeddings

_rope = None


def _fn():
    global _rope
    if _rope is None:
        c = lib
        _rope = lib.fn("lvb_rope", [c.c_void_p] * 4 + [c.c_int] * 3 + [c.c_longlong, c.c_int, c.c_int, c.c_float, c.c_void_p, c.c_void_p])
    return _rope


def _launch(x: torch.Tensor, cos, sin, pos32, seq_len, sign):
    # x: [..., tokens, heads, D] contiguous in (heads, D); flatten leading dims
    D = x.shape[-1]
    H = x.shape[-2]
    xt = x.view(-1, H, D)
    rc = _fn()(xt.data_ptr(), cos.data_ptr(), sin.data_ptr(), lib.ptr(pos32), xt.shape[0], H, D, xt.stride(0), seq_len,
               cos.shape[0], float(sign), lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_rope")


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin, pos32, seq_len):
        q = q.contiguous()
        k = k.contiguous()
        # q/k are fresh projection outputs; rotate in place and mark dirty
        _launch(q, cos, sin, pos32, seq_len, 1.0)
        _launch(k, cos, sin, pos32, seq_len, 1.0)
        ctx.save_for_backward(cos, sin, pos32)
        ctx.seq_len = seq_len
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin, pos32 = ctx.saved_tensors
        dq = dq.contiguous().clone() if not dq.is_contiguous() else dq.clone()
        dk = dk.contiguous().clone() if not dk.is_contiguous() else dk.clone()
        _launch(dq, cos, sin, pos32, ctx.seq_len, -1.0)
        _launch(dk, cos, sin, pos32, ctx.seq_len, -1.0)
        return dq, dk, None, None, None, None


_last_cos_sin = None  # (key, position tensor kept alive, cos, sin)


def _cos_sin_once(rot: RotaryEmbeddings, pos_ids: torch.Tensor):
    """cos/sin rows for explicit positions, computed once per forward pass instead of once per layer: every layer of a model
    passes the same position tensor.  The entry holds a reference to that tensor (so its address cannot be reused while the
    entry lives) and is keyed on its version counter (in-place updates invalidate it) and on whether a CUDA graph is being
    captured (tables made before a capture must not be baked into the graph as constants)."""
    global _last_cos_sin
    capturing = torch.cuda.is_current_stream_capturing() if pos_ids.is_cuda else False
    sig = getattr(rot, "_value_signature", None)
    if sig is None:  # layers build their own embedding objects from the same config: compare them by value
        f = rot.inv_freq
        sig = rot._value_signature = (rot.head_dim, rot.position_scale, rot.temperature, f.numel(), float(f[0]), float(f[-1]), float(f.sum()))
    key = (pos_ids.data_ptr(), pos_ids._version, pos_ids.numel(), capturing, sig)
    hit = _last_cos_sin
    if hit is not None and hit[0] == key:
        return hit[2], hit[3]
    cos, sin = rot.cos_sin(pos_ids.reshape(-1))
    cos, sin = cos.contiguous(), sin.contiguous()
    _last_cos_sin = (key, pos_ids, cos, sin)
    return cos, sin


def apply_rope(q: torch.Tensor, k: torch.Tensor, rot: RotaryEmbeddings, pos_ids=None):
    """Rotate ``q[..., S, H, D]`` and ``k[..., S, KV, D]``.

    ``pos_ids`` is None (positions ``0..S-1``), a ``[S]`` tensor shared by every batch row, or a tensor with one
    position per token (``[B, S]`` / ``[T]``)."""
    D = q.shape[-1]
    S = q.shape[-3]
    if q.is_cuda and lib.available() and q.dtype == torch.bfloat16 and D % 16 == 0:
        tokens = q.numel() // (q.shape[-2] * D)
        if pos_ids is None:
            cos, sin = rot.table(S, q.device)
            period = S
        elif pos_ids.numel() == S and tokens % S == 0:
            cos, sin = _cos_sin_once(rot, pos_ids)
            period = S
        elif pos_ids.numel() == tokens:
            cos, sin = _cos_sin_once(rot, pos_ids)
            period = tokens
        else:
            raise ValueError(f"pos_ids of shape {tuple(pos_ids.shape)} does not match q {tuple(q.shape)}")
        # the kernel looks the row up as (token index mod period), so no index tensor is needed
        return _RopeFn.apply(q, k, cos.contiguous(), sin.contiguous(), None, period)
    if pos_ids is None:
        pos_ids = torch.arange(S, device=q.device)
    return rot(q, pos_ids), rot(k, pos_ids)
