"""fp8 training of Linear layers (the reference's ``QuantizationConfig(fp8=True)``: Haliax ``Fp8DotGeneralOp`` with per-tensor
delayed scaling, src/levanter/trainer.py:648, config/gpt2_small_fast_fp8.yaml:17-18).

Forward operands are quantised to e4m3, output gradients to e5m2, each with one scale per tensor taken from a rolling
history of absolute maxima (delayed scaling: the scale used now comes from earlier steps, so quantisation needs no extra
pass over the tensor; the first step uses the current maximum).  The three GEMMs of a layer run on the tcgen05 fp8 path
(``kind::f8f6f4``, ``csrc/gemm_bf16.cu``), fp32 accumulation, with the product of the two de-quantisation scales applied in
the epilogue from a device scalar.  The kernel takes K-contiguous operands only, so the backward pass quantises transposed
copies of the weight, the input and the output gradient.  Master weights, optimizer state and checkpoints are unchanged:
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


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, amax_x, amax_w, amax_g):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        xq, sx = quantize(x2, E4M3, amax_x)
        wq, sw = quantize(weight, E4M3, amax_w)
        y = fp8_gemm(xq, wq, sx * sw, out_dtype=x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16, bias=bias)
        ctx.save_for_backward(xq, sx, wq, sw, amax_g if amax_g is not None else torch.empty(0))
        ctx.has_bias = bias is not None
        ctx.weight = weight
        ctx.x_dtype = x.dtype
        return y.reshape(*lead, weight.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        xq, sx, wq, sw, amax_g = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        gq, sg = quantize(g2, E5M2, amax_g if amax_g.numel() else None)
        dx = fp8_gemm(gq, _t(wq), sg * sw, out_dtype=torch.bfloat16 if gy.dtype == torch.bfloat16 else torch.float32)
        w = ctx.weight
        main = getattr(w, "main_grad", None)
        if main is not None:
            fp8_gemm(_t(gq), _t(xq), sg * sx, out=main, accumulate=True)  # straight into the fp32 gradient accumulator
            dw = None
        else:
            dw = fp8_gemm(_t(gq), _t(xq), sg * sx, out_dtype=torch.float32).to(w.dtype)
        db = g2.float().sum(0).to(gy.dtype) if ctx.has_bias else None
        return dx.reshape(*gy.shape[:-1], xq.shape[1]).to(ctx.x_dtype), dw, db, None, None, None


class Fp8Linear(nn.Module):
    """Drop-in for :class:`levanter_b200.nn.Linear` with fp8 GEMMs and delayed per-tensor scaling."""

    def __init__(self, weight: nn.Parameter, bias: Optional[nn.Parameter], amax_history_length: int = 1024):
        super().__init__()
        self.weight, self.bias = weight, bias
        self.in_features, self.out_features = weight.shape[1], weight.shape[0]
        h = max(int(amax_history_length), 1)
        for name in ("x", "w", "g"):
            self.register_buffer(f"amax_hist_{name}", torch.zeros(h, device=weight.device), persistent=False)
        self._seen = False

    @staticmethod
    def from_linear(linear: nn.Module, block: int = 128, amax_history_length: int = 16) -> "Fp8Linear":
        return Fp8Linear(linear.weight, getattr(linear, "bias", None), amax_history_length)

    def _delayed(self, name: str, current: torch.Tensor) -> torch.Tensor:
        """Scale source for this step: the maximum over the history (the current value on the first step), then push."""
        hist = getattr(self, f"amax_hist_{name}")
        cur = current.detach().abs().amax().float()
        use = torch.where(hist.max() > 0, hist.max(), cur)
        hist.copy_(torch.roll(hist, 1))
        hist[0] = cur
        # a tensor that outgrew its history would saturate: never use a scale below the current maximum's
        return torch.maximum(use, cur)

    def forward(self, x: torch.Tensor, *, skip_bias: bool = False) -> torch.Tensor:
        ax = self._delayed("x", x)
        aw = self._delayed("w", self.weight)
        ag = self.amax_hist_g.max() if self.training and bool(self._seen) else None
        return _Fp8LinearFn.apply(x, self.weight, None if skip_bias else self.bias, ax, aw, None)
