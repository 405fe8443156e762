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
``Fp8Linear`` owns the same ``weight`` / ``bias`` parameters as the ``Linear`` it replaces.

Block scaling (``Fp8Linear(block_scaled=True)``, ``QuantizationConfig(scaling="block")``): every run of 32 values along the
contraction dimension has its own power-of-two scale (the OCP MX format), computed from the block itself, so there is no
history and no saturation, and an outlier costs precision only inside its block.  ``csrc/mxfp8_quant.cu`` writes the fp8
values and the scale bytes in one pass, for the tensor as it is and for its transpose (a backward product contracts over the
other dimension and needs its own blocks); ``csrc/gemm_mxfp8.cu`` runs ``tcgen05.mma kind::mxf8f6f4.block_scale``, where
the tensor core applies the scales from tensor memory.  Shapes whose three dimensions are not multiples of 128 take the
bf16 path for that call."""
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


# ------------------------------------------------------------------------------------------------ block scaling (MX)
MX_BLOCK = 32


def _sf_chunks(sf2d: torch.Tensor) -> torch.Tensor:
    """``[rows, K / 32]`` scale bytes -> the chunked layout of the GEMM (rows padded to 128 and K to 128 with 127)."""
    R, KB = sf2d.shape
    Rp, KBp = -(-R // 128) * 128, -(-KB // 4) * 4
    full = torch.full((Rp, KBp), 127, dtype=torch.uint8, device=sf2d.device)
    full[:R, :KB] = sf2d
    return full.view(Rp // 128, 4, 32, KBp // 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)


def _sf_rows(chunks: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """Inverse of :func:`_sf_chunks`: ``[rows, K / 32]`` scale bytes."""
    Rp, KBp = -(-rows // 128) * 128, -(-(K // 32) // 4) * 4
    full = chunks.view(Rp // 128, KBp // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(Rp, KBp)
    return full[:rows, : K // 32]


def _mx_quantize_rows_reference(x2: torch.Tensor, dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """PyTorch statement of the kernel: blocks of 32 along the last dimension, scale ``2^ceil(log2(amax / fmax))``."""
    R, C = x2.shape
    xb = x2.float().view(R, C // MX_BLOCK, MX_BLOCK)
    amax = xb.abs().amax(-1)
    m, ex = torch.frexp(amax / _FMAX[dtype])  # amax / fmax = m 2^ex, m in [0.5, 1): ceil(log2) is ex, or ex - 1 at a power of two
    e = torch.where(amax > 0, (ex - (m == 0.5).to(ex.dtype)).float(), torch.full_like(amax, -127.0)).clamp_(-127, 126)
    q = (xb * torch.exp2(-e.clamp(min=-126)).unsqueeze(-1)).clamp_(-_FMAX[dtype], _FMAX[dtype]).to(dtype).view(R, C)
    return q, _sf_chunks((e + 127).to(torch.uint8))


def mx_quantize(x2: torch.Tensor, dtype: torch.dtype, want_row: bool = True, want_col: bool = False):
    """``x2 [R, C]`` -> ``(q_row [R, C], sf_row, q_col [C, R], sf_col)`` (``None`` for what was not asked): fp8 values with
    one scale per 32 values along C (``q_row``) or along R (``q_col``, the transpose).  One kernel on a B200."""
    R, C = x2.shape
    if (x2.is_cuda and lib.available() and x2.dtype == torch.bfloat16 and x2.stride(1) == 1 and x2.stride(0) % 8 == 0 and C % 8 == 0
            and x2.data_ptr() % 16 == 0):
        c = lib
        if "mxq" not in _f:
            _f["mxq"] = lib.fn("lvb_mxfp8_quantize", [c.c_void_p, c.c_longlong, c.c_int, c.c_int, c.c_int] + [c.c_void_p] * 5)
            _f["mxsf"] = lib.fn("lvb_mxfp8_sf_bytes", [c.c_int, c.c_int], restype=c.c_longlong, launches=0)
        dev = x2.device
        q_row = torch.empty(R, C, dtype=dtype, device=dev) if want_row else None
        sf_row = torch.empty(_f["mxsf"](R, -(-C // 128) * 128), dtype=torch.uint8, device=dev) if want_row else None
        q_col = torch.empty(C, R, dtype=dtype, device=dev) if want_col else None
        sf_col = torch.empty(_f["mxsf"](C, -(-R // 128) * 128), dtype=torch.uint8, device=dev) if want_col else None
        rc = _f["mxq"](x2.data_ptr(), x2.stride(0), R, C, _FMT[dtype], lib.ptr(q_row), lib.ptr(sf_row), lib.ptr(q_col), lib.ptr(sf_col),
                       lib.stream_ptr())
        lib.check_rc(rc, "lvb_mxfp8_quantize")
        return q_row, sf_row, q_col, sf_col
    q_row, sf_row = _mx_quantize_rows_reference(x2, dtype) if want_row else (None, None)
    q_col, sf_col = _mx_quantize_rows_reference(x2.t().contiguous(), dtype) if want_col else (None, None)
    return q_row, sf_row, q_col, sf_col


def mx_dequantize(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    """fp32 values of a block-scaled operand ``q [rows, K]`` with its chunked scale bytes."""
    rows, K = q.shape
    e = _sf_rows(sf, rows, K).float() - 127.0
    return (q.float().view(rows, K // MX_BLOCK, MX_BLOCK) * torch.exp2(e).unsqueeze(-1)).view(rows, K)


def mx_gemm(a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor, sfb: torch.Tensor, *, out: Optional[torch.Tensor] = None,
            out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, bias: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
    """``a[M,K] @ b[N,K]^T`` (+ bias) for block-scaled fp8 operands; fp32 accumulation; ``K % 128 == 0``."""
    M, K = a.shape
    N = b.shape[0]
    if not (a.is_cuda and lib.available() and K % 128 == 0 and a.is_contiguous() and b.is_contiguous()):
        res = mx_dequantize(a, sfa) @ mx_dequantize(b, sfb).t()
        if bias is not None:
            res = res + bias.float()
        if out is not None:
            out.copy_(out.float() + res if accumulate else res)
            return out
        return res.to(out_dtype)
    c = lib
    if "mxg" not in _f:
        _f["mxg"] = lib.fn("lvb_gemm_mxfp8", [c.c_void_p] * 5 + [c.c_int] * 9 + [c.c_float, c.c_void_p, c.c_int, c.c_void_p, c.c_void_p])
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    flags = (1 if out.dtype == torch.float32 else 0) | (2 if accumulate else 0)
    if bias is not None:
        flags |= 4 | (16 if bias.dtype == torch.float32 else 0)
        bias = bias.contiguous()
    rc = _f["mxg"](a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), out.data_ptr(), M, N, K, K, K, out.stride(0),
                   _FMT[a.dtype], _FMT[b.dtype], flags, 1.0, lib.ptr(bias), bn, lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_gemm_mxfp8")
    return out


class _MxFp8LinearFn(torch.autograd.Function):
    """``y = x W^T (+ b)`` with the three products of the layer in block-scaled fp8 (forward operands e4m3, output gradients
    e5m2).  Each tensor is quantised twice, with blocks along either dimension, because each product contracts over a
    different one: forward over ``in``, dX over ``out``, dW over the tokens."""

    @staticmethod
    def forward(ctx, x, weight, bias, train):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        xq, sx, xq_t, sx_t = mx_quantize(x2, E4M3, True, train)
        wq, sw, wq_t, sw_t = mx_quantize(weight, E4M3, True, train)
        y = mx_gemm(xq, sx, wq, sw, out_dtype=torch.bfloat16, bias=bias)
        if train:
            ctx.save_for_backward(xq_t, sx_t, wq_t, sw_t)
        ctx.has_bias = bias is not None
        ctx.weight = weight
        ctx.x_dtype = x.dtype
        ctx.in_features = x.shape[-1]
        return y.reshape(*lead, weight.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        xq_t, sx_t, wq_t, sw_t = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        if g2.dtype != torch.bfloat16 or g2.stride(1) != 1:
            g2 = g2.to(torch.bfloat16).contiguous()
        gq, sg, gq_t, sg_t = mx_quantize(g2, E5M2, True, True)
        dx = mx_gemm(gq, sg, wq_t, sw_t, out_dtype=torch.bfloat16)  # [T, in]: contraction over out
        w = ctx.weight
        main = getattr(w, "main_grad", None)
        if main is not None:
            mx_gemm(gq_t, sg_t, xq_t, sx_t, out=main, accumulate=True)  # [out, in] += , contraction over the tokens
            dw = None
        else:
            dw = mx_gemm(gq_t, sg_t, xq_t, sx_t, out_dtype=torch.float32).to(w.dtype)
        db = g2.float().sum(0).to(gy.dtype) if ctx.has_bias else None
        return dx.reshape(*gy.shape[:-1], ctx.in_features).to(ctx.x_dtype), dw, db, None


def mx_shapes_ok(tokens: int, in_features: int, out_features: int) -> bool:
    return tokens % 128 == 0 and in_features % 128 == 0 and out_features % 128 == 0


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
    """Drop-in for :class:`levanter_b200.nn.Linear` with fp8 GEMMs: delayed per-tensor scaling by default, one scale per 32
    values (the tensor core's block-scaled format) with ``block_scaled=True``.  A ``block`` argument is accepted for configs
    that name a block size; the hardware block is 32."""

    def __init__(self, weight: nn.Parameter, bias: Optional[nn.Parameter], amax_history_length: int = 1024, block_scaled: bool = False):
        super().__init__()
        self.weight, self.bias = weight, bias
        self.block_scaled = block_scaled
        self.in_features, self.out_features = weight.shape[1], weight.shape[0]
        h = max(int(amax_history_length), 1)
        for name in ("x", "w", "g"):
            self.register_buffer(f"amax_hist_{name}", torch.zeros(h, device=weight.device), persistent=False)
        self._seen = {"x": False, "w": False, "g": False}

    @staticmethod
    def from_linear(linear: nn.Module, block: int = 128, amax_history_length: int = 16, block_scaled: bool = False) -> "Fp8Linear":
        return Fp8Linear(linear.weight, getattr(linear, "bias", None), amax_history_length, block_scaled)

    def forward(self, x: torch.Tensor, *, skip_bias: bool = False) -> torch.Tensor:
        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)
        if w is not self.weight and hasattr(self.weight, "main_grad"):
            w.main_grad = self.weight.main_grad
        bias = None if skip_bias else self.bias
        if self.block_scaled:
            tokens = x.numel() // x.shape[-1]
            if mx_shapes_ok(tokens, self.in_features, self.out_features) and x.dtype == torch.bfloat16:
                return _MxFp8LinearFn.apply(x, w, bias, torch.is_grad_enabled() and (x.requires_grad or w.requires_grad))
            from .gemm import linear as _bf16_linear

            return _bf16_linear(x, w, bias)
        return _Fp8LinearFn.apply(x, w, bias, self)
