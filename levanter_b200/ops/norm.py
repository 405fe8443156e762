"""RMSNorm / LayerNorm (``csrc/norm.cu``) with PyTorch fp32 fallbacks.

Reference call sites: ``hnn.RmsNorm`` / ``hnn.LayerNorm`` via src/levanter/layers/normalization.py:38-48 and Gemma's
fp32 ``(1 + w)`` variant, src/levanter/models/gemma.py:279-291."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import lib

_f = {}


def _fn(name, argtypes, launches=1):
    if name not in _f:
        _f[name] = lib.fn(name, argtypes, launches=launches)
    return _f[name]


def _fwd():
    c = lib
    return _fn("lvb_norm_fwd", [c.c_void_p] * 4 + [c.c_int] + [c.c_void_p] * 4 + [c.c_int, c.c_int, c.c_float, c.c_float, c.c_int, c.c_void_p])


def _bwd():
    c = lib
    return _fn("lvb_norm_bwd", [c.c_void_p] * 3 + [c.c_int] + [c.c_void_p] * 7 + [c.c_int, c.c_int, c.c_float, c.c_int, c.c_int, c.c_void_p])


def _parts():
    c = lib
    return _fn("lvb_norm_bwd_parts", [c.c_int, c.c_int], launches=0)  # host-side size query


def norm_reference(x, weight, bias, eps, *, layer_norm=False, w_offset=0.0, residual=None):
    xf = x.float()
    if residual is not None:
        xf = (xf + residual.float()).to(x.dtype).float()
    if layer_norm:
        mean = xf.mean(-1, keepdim=True)
        var = xf.var(-1, keepdim=True, unbiased=False)
        y = (xf - mean) * torch.rsqrt(var + eps)
    else:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * (weight.float() + w_offset)
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def _kernel_ok(x, weight, bias) -> bool:
    if not (x.is_cuda and lib.available() and x.dtype == torch.bfloat16):
        return False
    dim = x.shape[-1]
    if dim % 8 != 0 or dim > 16384:
        return False
    for p in (weight, bias):
        if p is not None and (p.dtype not in (torch.float32, torch.bfloat16) or not p.is_contiguous() or p.data_ptr() % 16 != 0):
            return False  # the kernels read weights with 16-byte loads
    if weight is not None and bias is not None and weight.dtype != bias.dtype:
        return False
    return True


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, bias, eps, layer_norm, w_offset):
        dim = x.shape[-1]
        x2 = x.reshape(-1, dim)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        r2 = None
        h = None
        if residual is not None:
            r2 = residual.reshape(-1, dim).contiguous()
            h = torch.empty_like(x2)
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device) if layer_norm else None
        wf32 = int((weight if weight is not None else bias).dtype == torch.float32) if (weight is not None or bias is not None) else 0
        rc = _fwd()(x2.data_ptr(), lib.ptr(r2), lib.ptr(weight), lib.ptr(bias), wf32, y.data_ptr(), lib.ptr(h),
                    rstd.data_ptr(), lib.ptr(mean), rows, dim, float(eps), float(w_offset), int(layer_norm), lib.stream_ptr())
        lib.check_rc(rc, "lvb_norm_fwd")
        xin = h if h is not None else x2
        ctx.save_for_backward(xin, weight, rstd, mean)
        ctx.layer_norm = layer_norm
        ctx.w_offset = w_offset
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        ctx.wf32 = wf32
        if residual is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dh):
        xin, weight, rstd, mean = ctx.saved_tensors
        dim = xin.shape[-1]
        rows = xin.shape[0]
        dy2 = dy.reshape(-1, dim)
        if dy2.dtype != torch.bfloat16 or not dy2.is_contiguous():
            dy2 = dy2.to(torch.bfloat16).contiguous()
        dres = None
        if dh is not None:
            dres = dh.reshape(-1, dim)
            if dres.dtype != torch.bfloat16 or not dres.is_contiguous():
                dres = dres.to(torch.bfloat16).contiguous()
        dx = torch.empty_like(xin)
        need_dw = weight is not None and ctx.needs_input_grad[2]
        need_db = ctx.has_bias and ctx.needs_input_grad[3]
        nparts = _parts()(rows, dim)
        scratch = torch.empty(2 * nparts * dim, dtype=torch.float32, device=xin.device) if (need_dw or need_db) else None
        dw = torch.empty(dim, dtype=torch.float32, device=xin.device) if need_dw else None
        db = torch.empty(dim, dtype=torch.float32, device=xin.device) if need_db else None
        rc = _bwd()(dy2.data_ptr(), xin.data_ptr(), lib.ptr(weight), ctx.wf32, rstd.data_ptr(), lib.ptr(mean), lib.ptr(dres),
                    dx.data_ptr(), lib.ptr(dw), lib.ptr(db), lib.ptr(scratch), rows, dim, float(ctx.w_offset),
                    int(ctx.layer_norm), 0, lib.stream_ptr())
        lib.check_rc(rc, "lvb_norm_bwd")
        dxv = dx.view(ctx.shape)
        if dw is not None and weight.dtype != torch.float32:
            dw = dw.to(weight.dtype)
        if db is not None and weight is not None and weight.dtype != torch.float32:
            db = db.to(weight.dtype)
        return dxv, (dxv if ctx.has_res else None), dw, db, None, None, None


def fused_norm(x, weight, bias, eps, *, layer_norm=False, w_offset=0.0, residual=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns ``(norm(x + residual), x + residual)`` (second item None when there is no residual)."""
    if _kernel_ok(x, weight, bias) and (residual is None or residual.dtype == torch.bfloat16):
        return _NormFn.apply(x, residual, weight, bias, eps, layer_norm, w_offset)
    h = None
    if residual is not None:
        h = (x.float() + residual.float()).to(x.dtype)
        return norm_reference(h, weight, bias, eps, layer_norm=layer_norm, w_offset=w_offset), h
    return norm_reference(x, weight, bias, eps, layer_norm=layer_norm, w_offset=w_offset), None


def rms_norm(x, weight, bias=None, eps: float = 1e-6, w_offset: float = 0.0) -> torch.Tensor:
    return fused_norm(x, weight, bias, eps, layer_norm=False, w_offset=w_offset)[0]


def layer_norm(x, weight, bias, eps: float = 1e-5) -> torch.Tensor:
    return fused_norm(x, weight, bias, eps, layer_norm=True)[0]
