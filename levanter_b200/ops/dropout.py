"""Dropout on a counter-based generator (``csrc/dropout.cu``), optionally fused with the residual add that follows it.

``dropout(x, p, residual=r)`` is ``r + mask * x / (1 - p)`` in one pass; the mask is a function of a 64-bit seed drawn from the
ambient PyTorch generator and the element index, so the backward pass regenerates it instead of storing it.  Replaces
``hnn.Dropout`` (src/levanter/models/gpt2.py:232,297) and its separate residual add."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

from . import lib

_f = {}


def _fn():
    if "f" not in _f:
        c = lib
        _f["f"] = lib.fn("lvb_dropout", [c.c_void_p, c.c_void_p, c.c_void_p, c.c_longlong, c.c_float, lib.ctypes.c_uint, lib.ctypes.c_uint, c.c_void_p])
    return _f["f"]


def _apply(x: torch.Tensor, residual: Optional[torch.Tensor], p: float, seed: int) -> torch.Tensor:
    out = torch.empty_like(x)
    rc = _fn()(x.data_ptr(), lib.ptr(residual), out.data_ptr(), x.numel(), float(p), seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, lib.stream_ptr())
    lib.check_rc(rc, "lvb_dropout")
    return out


def philox_keep_mask(n: int, p: float, seed: int) -> np.ndarray:
    """The kernel's keep-mask for ``n`` elements (a NumPy restatement of Philox4x32-10, for tests and CPU use)."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    n8 = (n + 7) // 8
    idx = np.arange(n8, dtype=np.uint64)
    draws = []
    for sub in (0, 1):
        c = [idx & 0xFFFFFFFF, idx >> np.uint64(32), np.full(n8, sub, dtype=np.uint64), np.zeros(n8, dtype=np.uint64)]
        k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
        for _ in range(10):
            p0, p1 = c[0] * np.uint64(M0), c[2] * np.uint64(M1)
            hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & np.uint64(0xFFFFFFFF), p1 >> np.uint64(32), p1 & np.uint64(0xFFFFFFFF)
            c = [(hi1 ^ c[1] ^ np.uint64(k0)) & np.uint64(0xFFFFFFFF), lo1, (hi0 ^ c[3] ^ np.uint64(k1)) & np.uint64(0xFFFFFFFF), lo0]
            k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
        draws.extend(c)
    r = np.stack(draws, axis=1).reshape(-1)[:n]  # 8 draws per index: (x, y, z, w) of the first call, then of the second
    thr = min(int(p * 4294967296.0), 4294967295)
    return r >= np.uint64(thr)


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, p, seed):
        ctx.p, ctx.seed, ctx.has_res = p, seed, residual is not None
        return _apply(x.contiguous(), residual.contiguous() if residual is not None else None, p, seed)

    @staticmethod
    def backward(ctx, dy):
        dx = _apply(dy.contiguous(), None, ctx.p, ctx.seed)
        return dx, (dy if ctx.has_res else None), None, None


def dropout(x: torch.Tensor, p: float, training: bool = True, residual: Optional[torch.Tensor] = None, seed: Optional[int] = None) -> torch.Tensor:
    """``residual + dropout(x)`` (``residual`` optional).  ``seed`` defaults to a draw from PyTorch's CPU generator, so a seeded
    region (the trainer seeds every micro-batch) reproduces its masks."""
    if p == 0.0 or not training:
        return x if residual is None else x + residual
    if x.is_cuda and lib.available() and x.dtype == torch.bfloat16 and x.numel() % 8 == 0 and (residual is None or residual.shape == x.shape):
        if seed is None:
            seed = int(torch.empty((), dtype=torch.int64).random_().item())
        return _DropoutFn.apply(x, residual, float(p), int(seed))
    y = F.dropout(x, p, training=True)
    return y if residual is None else y + residual
