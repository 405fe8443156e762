"""Depthwise causal convolution over ``[B, L, C]`` activations with an optional SiLU (``csrc/dwconv.cu``): the short filters of
the Hyena operator (src/levanter/models/hyena.py:474-482) and of the gated delta-rule layer, without the transposes around a
library ``conv1d``.  ``weight`` has the ``nn.Conv1d`` depthwise shape ``[C, 1, K]``."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import lib

_f = {}


def _bind():
    if not _f:
        P, I = lib.c_void_p, lib.c_int
        _f["fwd"] = lib.fn("lvb_dwconv_fwd", [P, P, P, P, I, I, I, I, I, I, I, P])
        _f["prep"] = lib.fn("lvb_dwconv_bwd_prep", [P] * 8 + [I] * 6 + [P], launches=2)
        _f["floats"] = lib.fn("lvb_dwconv_partial_floats", [I, I, I, I], restype=lib.c_longlong, launches=0)


def causal_dwconv_reference(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], silu: bool) -> torch.Tensor:
    """``conv1d`` padded by ``K - 1`` on both sides and truncated to the input length, computed in the weight's dtype."""
    L, K = x.shape[1], weight.shape[-1]
    y = F.conv1d(x.transpose(1, 2).to(weight.dtype), weight, bias, padding=K - 1, groups=weight.shape[0])[..., :L].transpose(1, 2)
    return (F.silu(y) if silu else y).to(x.dtype)


def _kernel_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    K = weight.shape[-1]
    return (x.is_cuda and lib.available() and x.dim() == 3 and x.dtype in (torch.bfloat16, torch.float32) and 2 <= K <= 4
            and x.shape[-1] % (8 if x.dtype == torch.bfloat16 else 4) == 0 and weight.shape[0] == x.shape[-1] and weight.shape[1] == 1)


class _CausalDwConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, silu):
        _bind()
        B, L, C = x.shape
        K = weight.shape[-1]
        x = x.contiguous()
        w32 = weight.detach().reshape(C, K).float().contiguous()
        b32 = None if bias is None else bias.detach().float().contiguous()
        y = torch.empty_like(x)
        bf = 1 if x.dtype == torch.bfloat16 else 0
        lib.check_rc(_f["fwd"](x.data_ptr(), w32.data_ptr(), lib.ptr(b32), y.data_ptr(), B, L, C, K, bf, int(silu), 0, lib.stream_ptr()),
                     "lvb_dwconv_fwd")
        ctx.save_for_backward(x, w32, b32 if b32 is not None else x.new_empty(0))
        ctx.meta = (bool(silu), bias is not None, weight.shape, weight.dtype, None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w32, b32 = ctx.saved_tensors
        silu, has_bias, w_shape, w_dtype, b_dtype = ctx.meta
        b32 = b32 if has_bias else None
        B, L, C = x.shape
        K = w32.shape[1]
        dy = dy.to(x.dtype).contiguous()
        bf = 1 if x.dtype == torch.bfloat16 else 0
        dev = x.device
        partial = torch.empty(_f["floats"](B, L, C, K), dtype=torch.float32, device=dev)
        dw = torch.empty(C, K, dtype=torch.float32, device=dev)
        db = torch.empty(C, dtype=torch.float32, device=dev) if has_bias else None
        dpre = torch.empty_like(x) if silu else None
        lib.check_rc(_f["prep"](x.data_ptr(), dy.data_ptr(), w32.data_ptr(), lib.ptr(b32), lib.ptr(dpre), partial.data_ptr(), dw.data_ptr(),
                                lib.ptr(db), B, L, C, K, bf, int(silu), lib.stream_ptr()), "lvb_dwconv_bwd_prep")
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            src = dpre if silu else dy
            lib.check_rc(_f["fwd"](src.data_ptr(), w32.data_ptr(), 0, dx.data_ptr(), B, L, C, K, bf, 0, 1, lib.stream_ptr()), "lvb_dwconv_fwd")
        return dx, dw.view(w_shape).to(w_dtype), None if db is None else db.to(b_dtype), None


def causal_dwconv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, silu: bool = False) -> torch.Tensor:
    """``y[b, l, c] = act(bias[c] + sum_j weight[c, 0, j] * x[b, l - (K - 1) + j, c])`` for ``x[B, L, C]``."""
    if _kernel_ok(x, weight):
        return _CausalDwConv.apply(x, weight, bias, silu)
    return causal_dwconv_reference(x, weight, bias, silu)
