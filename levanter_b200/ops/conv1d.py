"""Dense 1-D convolution with a 3-tap kernel as one tensor-core GEMM over a channels-last, zero-padded input: the two stem
convolutions of the Whisper encoder (src/levanter/models/whisper.py:316-335: ``conv1d(n_mels -> d, k3, p1)``,
``conv1d(d -> d, k3, s2, p1)``).

With the input stored as ``xp[B, T + 2, C]`` (one zero row before and after every sequence) and flattened to rows of ``C``
channels, the three taps that output position ``t`` reads are ``3 C`` *contiguous* elements starting at row ``stride * t``.
The im2col matrix is therefore a view of the input itself -- shape ``[rows, 3 C]``, row stride ``stride * C`` -- that a TMA
tensor map describes directly, and the convolution is ``view @ W'^T`` with ``W'[o, k C + c] = W[o, c, k]``: one launch of
the library's GEMM, no unfolded copy.  Rows that straddle two sequences are computed and discarded (2 per sequence at stride
1, 1 at stride 2).  The input gradient folds the ``[rows, 3 C]`` product back with three strided adds; the weight gradient
is a second GEMM over the same view."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import gemm as G
from . import lib


def pad_channels_last(x_bct: torch.Tensor) -> torch.Tensor:
    """``x[B, C, T]`` -> ``xp[B, T + 2, C]`` with zero rows at positions 0 and T + 1."""
    B, C, T = x_bct.shape
    xp = x_bct.new_zeros(B, T + 2, C)
    xp[:, 1 : T + 1] = x_bct.transpose(1, 2)
    return xp


def kernel_ok(xp: torch.Tensor, weight: torch.Tensor, stride: int) -> bool:
    return (xp.is_cuda and lib.available() and xp.dtype == torch.bfloat16 and xp.dim() == 3 and xp.is_contiguous()
            and weight.dim() == 3 and weight.shape[-1] == 3 and weight.shape[1] == xp.shape[-1] and xp.shape[-1] % 8 == 0
            and stride in (1, 2) and (stride == 1 or xp.shape[1] % 2 == 0))


def _window_view(xp: torch.Tensor, stride: int) -> torch.Tensor:
    B, Tp, C = xp.shape
    R = B * Tp
    rows = R - 2 if stride == 1 else (R - 2) // 2
    return torch.as_strided(xp, (rows, 3 * C), (stride * C, 1), xp.storage_offset())


class _Conv3(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xp, weight, bias, stride):
        B, Tp, C = xp.shape
        wp = weight.permute(0, 2, 1).reshape(weight.shape[0], 3 * C).to(torch.bfloat16).contiguous()
        view = _window_view(xp, stride)
        out = G.gemm(view, wp, bias=bias)
        ctx.save_for_backward(xp, wp)
        ctx.stride, ctx.has_bias, ctx.w_dtype, ctx.needs_x = stride, bias is not None, weight.dtype, xp.requires_grad
        return out

    @staticmethod
    def backward(ctx, gy):
        xp, wp = ctx.saved_tensors
        B, Tp, C = xp.shape
        s = ctx.stride
        gy = gy.to(torch.bfloat16).contiguous()
        rows = gy.shape[0]
        view = _window_view(xp, s)
        dwp = G.gemm(gy, view, a_mn=True, b_mn=True, out_dtype=torch.float32)  # [Cout, 3 C] = gy^T view
        dw = dwp.view(-1, 3, C).permute(0, 2, 1).to(ctx.w_dtype)
        db = gy.float().sum(0).to(ctx.w_dtype) if ctx.has_bias else None
        dx = None
        if ctx.needs_x:
            dcols = G.gemm(gy, wp, b_mn=True, out_dtype=torch.float32)  # [rows, 3 C]
            dxf = torch.zeros(B * Tp, C, dtype=torch.float32, device=xp.device)
            for k in range(3):
                dxf[k : k + s * rows : s] += dcols[:, k * C : (k + 1) * C]
            dx = dxf.view(B, Tp, C).to(xp.dtype)
        return dx, dw, db, None


def conv1d_k3(xp: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], stride: int = 1) -> torch.Tensor:
    """``conv1d(kernel 3, padding 1, stride)`` of the sequences stored in ``xp[B, T + 2, C_in]`` (zero rows at 0 and T + 1).
    Returns ``[B, T_out, C_out]`` (``T_out = T`` at stride 1, ``T / 2`` at stride 2; ``T`` even), a view into a slightly
    larger product.  ``weight`` is ``[C_out, C_in, 3]`` as in ``torch.nn.Conv1d``."""
    B, Tp, C = xp.shape
    T = Tp - 2
    if not kernel_ok(xp, weight, stride):
        y = F.conv1d(xp[:, 1 : T + 1].transpose(1, 2).to(weight.dtype), weight, bias, stride=stride, padding=1)
        return y.transpose(1, 2).to(xp.dtype)
    out = _Conv3.apply(xp, weight, bias, stride)  # [rows, C_out]; row r <-> (b, t) with r = b * per_seq + t
    per_seq = Tp // stride
    t_out = T // stride if stride == 2 else T
    Cout = out.shape[-1]
    full = torch.as_strided(out, (B, t_out, Cout), (per_seq * Cout, Cout, 1), out.storage_offset())
    return full
