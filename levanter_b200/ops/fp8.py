"""fp8 training of Linear layers (the reference's ``QuantizationConfig(fp8=True)``: Haliax ``Fp8DotGeneralOp`` with per-tensor
delayed scaling, src/levanter/trainer.py:648, config/gpt2_small_fast_fp8.yaml:17-18).

Forward operands are quantised to e4m3, output gradients to e5m2, each with one scale per tensor taken from a rolling
history of absolute maxima (delayed scaling: the scale used now is the maximum over earlier steps' recorded maxima, so
quantisation needs no pass over the tensor beforehand; values that outgrow it saturate, and a tensor's very first use
takes its current maximum).  On a B200 one kernel (``csrc/fp8_quant.cu``) reads the bf16 tensor once and writes its fp8
copy, the transposed fp8 copy and the tensor's absolute maximum into the history.  The three GEMMs of a layer run on the
tcgen05 fp8 path (``kind::f8f6f4``, ``csrc/gemm_bf16.cu``), fp32 accumulation, with the product of the two
de-quantisation scales applied in the epilogue from a device scalar.  The GEMM takes K-contiguous operands only, which
is what the transposed copies are for.  Master weights, optimizer state and checkpoints are unchanged:
``Fp8Linear`` owns the same ``weight`` / ``bias`` parameters as the ``Linear`` it replaces."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import lib

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2
_FMAX = {E4M3: 448.0, E5M2: 57344.0}
_FMT = {E4M3: 0, E5M2: 1}
_f = {}


def quantize(x: torch.Tensor, dtype: torch.dtype, amax: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(x_q, inv_scale)``: ``x ~= x_q.float() * inv_scale``.  ``amax`` (device scalar) picks the scale; default: of ``x``."""
    if amax is None:
        amax = x.detach().abs().amax().float()
    scale = _FMAX[dtype] / torch.clamp(amax, min=1e-12)
    xq = (x.float() * scale).clamp_(-_FMAX[dtype], _FMAX[dtype]).to(dtype)
    return xq, (1.0 / scale).reshape(1)


def _t(xq: torch.Tensor) -> torch.Tensor:
    """Transposed contiguous copy of a 2-D fp8 tensor (done on the byte view)."""
    return xq.view(torch.uint8).t().contiguous().view(xq.dtype)


def fp8_gemm(a: torch.Tensor, b: torch.Tensor, scale: torch.Tensor, *, out: Optional[torch.Tensor] = None,
             out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``scale * a[M,K] @ b[N,K]^T`` (+ bias) for fp8 ``a``/``b``; fp32 accumulation."""
    M, K = a.shape
    N = b.shape[0]
    use = a.is_cuda and lib.available() and K % 16 == 0 and a.is_contiguous() and b.is_contiguous()
    if not use:
        res = (a.float() @ b.float().t()) * scale.float()
        if bias is not None:
            res = res + bias.float()
        if out is not None:
            out.copy_(out.float() + res if accumulate else res)
            return out
        return res.to(out_dtype)
    c = lib
    if "g" not in _f:
        _f["g"] = lib.fn("lvb_gemm_fp8", [c.c_void_p] * 3 + [c.c_int] * 9 + [c.c_float] + [c.c_void_p] * 3 + [c.c_int, c.c_int, c.c_void_p, c.c_void_p])
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    flags = (1 if out.dtype == torch.float32 else 0) | (2 if accumulate else 0)
    if bias is not None:
        flags |= 4 | (16 if bias.dtype == torch.float32 else 0)
    rc = _f["g"](a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, K, K, out.stride(0), _FMT[a.dtype], _FMT[b.dtype], flags, 1.0,
                 scale.data_ptr(), lib.ptr(bias), 0, 0, 0, lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_gemm_fp8")
    return out


def quantize_with_history(x2: torch.Tensor, dtype: torch.dtype, hist: torch.Tensor, seen: bool, want_t: bool):
    """Quantise ``x2 [R, C]`` with the scale its history gives and record its own maximum as the newest history entry.
    Returns ``(q, q_t or None, inv_scale)``.  One pass over ``x2`` on a B200; PyTorch ops elsewhere."""
    src = hist.max().reshape(1) if seen else x2.detach().abs().amax().float().reshape(1)
    hist.copy_(torch.roll(hist, 1))
    hist[0] = 0.0
    if x2.is_cuda and lib.available() and x2.dtype == torch.bfloat16 and x2.stride(1) == 1:
        R, C = x2.shape
        q = torch.empty(R, C, dtype=dtype, device=x2.device)
        qt = torch.empty(C, R, dtype=dtype, device=x2.device) if want_t else None
        inv = torch.empty(1, dtype=torch.float32, device=x2.device)
        c = lib
        if "q" not in _f:
            _f["q"] = lib.fn("lvb_fp8_quantize", [c.c_void_p, c.c_longlong, c.c_int, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_void_p,
                                                  c.c_void_p, c.c_void_p, c.c_void_p])
        rc = _f["q"](x2.data_ptr(), x2.stride(0), R, C, src.data_ptr(), _FMT[dtype], q.data_ptr(), lib.ptr(qt), inv.data_ptr(),
                     hist.data_ptr(), lib.stream_ptr())  # hist[0] (just cleared) receives the maximum: a non-negative float's bits order as integers
        lib.check_rc(rc, "lvb_fp8_quantize")
        return q, qt, inv
    hist[0] = x2.detach().abs().amax().float()
    q, inv = quantize(x2, dtype, src.reshape(()))
    return q, (_t(q) if want_t else None), inv


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, mod):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        train = torch.is_grad_enabled() or mod.training
        xq, xq_t, sx = quantize_with_history(x2, E4M3, mod.amax_hist_x, mod._seen["x"], train)
        wq, wq_t, sw = quantize_with_history(weight, E4M3, mod.amax_hist_w, mod._seen["w"], train)
        mod._seen["x"] = mod._seen["w"] = True
        y = fp8_gemm(xq, wq, sx * sw, out_dtype=x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16, bias=bias)
        ctx.save_for_backward(xq_t if xq_t is not None else xq, sx, wq_t if wq_t is not None else wq, sw)
        ctx.has_t = xq_t is not None
        ctx.has_bias = bias is not None
        ctx.weight = weight
        ctx.mod = mod
        ctx.x_dtype = x.dtype
        ctx.in_features = x.shape[-1]
        return y.reshape(*lead, weight.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        xs, sx, ws, sw = ctx.saved_tensors
        xq_t, wq_t = (xs, ws) if ctx.has_t else (_t(xs), _t(ws))
        mod = ctx.mod
        g2 = gy.reshape(-1, gy.shape[-1])
        gq, gq_t, sg = quantize_with_history(g2, E5M2, mod.amax_hist_g, mod._seen["g"], True)
        mod._seen["g"] = True
        dx = fp8_gemm(gq, wq_t, sg * sw, out_dtype=torch.bfloat16 if gy.dtype == torch.bfloat16 else torch.float32)
        w = ctx.weight
        main = getattr(w, "main_grad", None)
        if main is not None:
            fp8_gemm(gq_t, xq_t, sg * sx, out=main, accumulate=True)  # straight into the fp32 gradient accumulator
            dw = None
        else:
            dw = fp8_gemm(gq_t, xq_t, sg * sx, out_dtype=torch.float32).to(w.dtype)
        db = g2.float().sum(0).to(gy.dtype) if ctx.has_bias else None
        return dx.reshape(*gy.shape[:-1], ctx.in_features).to(ctx.x_dtype), dw, db, None


class Fp8Linear(nn.Module):
    """Drop-in for :class:`levanter_b200.nn.Linear` with fp8 GEMMs and delayed per-tensor scaling (one scale per tensor; a
    ``block`` argument is accepted for configs that name a block size and is not used)."""

    def __init__(self, weight: nn.Parameter, bias: Optional[nn.Parameter], amax_history_length: int = 1024):
        super().__init__()
        self.weight, self.bias = weight, bias
        self.in_features, self.out_features = weight.shape[1], weight.shape[0]
        h = max(int(amax_history_length), 1)
        for name in ("x", "w", "g"):
            self.register_buffer(f"amax_hist_{name}", torch.zeros(h, device=weight.device), persistent=False)
        self._seen = {"x": False, "w": False, "g": False}

    @staticmethod
    def from_linear(linear: nn.Module, block: int = 128, amax_history_length: int = 16) -> "Fp8Linear":
        return Fp8Linear(linear.weight, getattr(linear, "bias", None), amax_history_length)

    def forward(self, x: torch.Tensor, *, skip_bias: bool = False) -> torch.Tensor:
        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)
        if w is not self.weight and hasattr(self.weight, "main_grad"):
            w.main_grad = self.weight.main_grad
        return _Fp8LinearFn.apply(x, w, None if skip_bias else self.bias, self)
