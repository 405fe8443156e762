"""Causal long convolution with one filter per channel (``csrc/long_conv.cu``) and its gradients: the Hyena operator's long
filter as a direct sum in shared memory instead of zero-padded FFTs (src/levanter/models/hyena.py:326-339).  ``L <= 4096``
runs on the kernel (bf16 data, fp32 sums); anything else takes the FFT statement, which is also the oracle of the tests."""
from __future__ import annotations

from typing import Optional

import torch

from . import lib

_f = {}
MAX_KERNEL_LEN = 4096


def fft_conv_reference(u: torch.Tensor, k: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``u[..., L, C]`` with ``k[L, C]``: zero-padded FFT of size 2L in fp32."""
    L = u.shape[-2]
    n = 2 * L
    u_f = torch.fft.rfft(u.float(), n=n, dim=-2)
    k_f = torch.fft.rfft(k.float(), n=n, dim=-2)
    y = torch.fft.irfft(u_f * k_f, n=n, dim=-2)[..., :L, :]
    if bias is not None:
        y = y + bias.float()
    return y.to(u.dtype)


def _fns():
    if not _f:
        c = lib
        _f["conv"] = lib.fn("lvb_long_conv", [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_void_p])
        _f["dk"] = lib.fn("lvb_long_conv_filter_grad", [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_void_p])
    return _f


def _conv(u3: torch.Tensor, k: torch.Tensor, bias, reverse: bool) -> torch.Tensor:
    N, L, C = u3.shape
    y = torch.empty_like(u3)
    rc = _fns()["conv"](u3.data_ptr(), k.data_ptr(), lib.ptr(bias), y.data_ptr(), N, L, C, int(reverse), 0, lib.stream_ptr())
    lib.check_rc(rc, "lvb_long_conv")
    return y


class _LongConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, k, bias):
        shp = u.shape
        u3 = u.reshape(-1, shp[-2], shp[-1]).contiguous()
        kb = k.to(torch.bfloat16).contiguous()
        bf = bias.float().contiguous() if bias is not None else None
        ctx.save_for_backward(u3, kb)
        ctx.shape, ctx.k_dtype, ctx.has_bias = shp, k.dtype, bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return _conv(u3, kb, bf, False).view(shp)

    @staticmethod
    def backward(ctx, dy):
        u3, kb = ctx.saved_tensors
        N, L, C = u3.shape
        dy3 = dy.reshape(N, L, C).to(torch.bfloat16).contiguous()
        du = dk = db = None
        if ctx.needs_input_grad[0]:
            du = _conv(dy3, kb, None, True).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            part = torch.empty(N, L, C, dtype=torch.float32, device=u3.device)
            rc = _fns()["dk"](u3.data_ptr(), dy3.data_ptr(), part.data_ptr(), N, L, C, lib.stream_ptr())
            lib.check_rc(rc, "lvb_long_conv_filter_grad")
            dk = part.sum(0).to(ctx.k_dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy3.float().sum((0, 1)).to(ctx.bias_dtype)
        return du, dk, db


def long_conv(u: torch.Tensor, k: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[..., t, c] = sum_{s <= t} k[s, c] u[..., t - s, c] (+ bias[c])``."""
    L = u.shape[-2]
    if u.is_cuda and lib.available() and u.dtype == torch.bfloat16 and L <= MAX_KERNEL_LEN and k.shape == (L, u.shape[-1]):
        return _LongConvFn.apply(u, k, bias)
    return fft_conv_reference(u, k, bias)
