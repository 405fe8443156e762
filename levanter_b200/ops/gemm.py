"""bf16 GEMM on tcgen05 tensor cores (see ``csrc/gemm_bf16.cu``) and the ``linear`` autograd op on top of it.

Replaces the dense projections that the reference lowers through ``hnn.Linear`` /
``hax.dot`` (src/levanter/layers/attention.py:1606-1635, src/levanter/models/llama.py:273-280).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import lib

F_OUT_F32 = 1
F_ACCUMULATE = 2
F_BIAS = 4
F_RESIDUAL = 8
F_BIAS_F32 = 16

_gemm_fn = None


def _fn():
    global _gemm_fn
    if _gemm_fn is None:
        c = lib
        _gemm_fn = lib.fn(
            "lvb_gemm_bf16",
            [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
             c.c_int, c.c_int, c.c_float, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_void_p],
        )
    return _gemm_fn


def _rowmajor_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError(f"expected a 2-D tensor, got {tuple(t.shape)}")
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def gemm_reference(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=torch.bfloat16, accumulate=False,
                   bias=None, residual=None, alpha=1.0):
    """PyTorch fp32 statement of :func:`gemm` (used on CPU and as the test oracle)."""
    af = (a.t() if a_mn else a).float()
    bf = (b if b_mn else b.t()).float()
    c = alpha * (af @ bf)
    if bias is not None:
        c = c + bias.float()
    if residual is not None:
        c = c + residual.float()
    if out is not None:
        if accumulate:
            c = c + out.float()
        out.copy_(c.to(out.dtype))
        return out
    return c.to(out_dtype)


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    accumulate: bool = False,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    alpha: float = 1.0,
    max_ctas: int = 0,
) -> torch.Tensor:
    """``C[M,N] = alpha * op(A) @ op(B)^T (+bias) (+residual) (+C)``.

    ``a`` is ``[M,K]`` (``a_mn=False``) or ``[K,M]`` (``a_mn=True``); ``b`` is ``[N,K]`` or ``[K,N]``.
    Inputs are bf16; the accumulator is fp32; ``out`` may be bf16 or fp32.
    """
    if not (a.is_cuda and lib.available()):
        return gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out=out, out_dtype=out_dtype, accumulate=accumulate,
                              bias=bias, residual=residual, alpha=alpha)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm expects bf16 operands")
    a = _rowmajor_2d(a)
    b = _rowmajor_2d(b)
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"reduction dims differ: {K} vs {Kb}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        if accumulate:
            raise ValueError("accumulate=True needs out=")
    else:
        if out.shape != (M, N) or out.stride(1) != 1:
            raise ValueError("out has the wrong shape or is not row-major")
    flags = 0
    if out.dtype == torch.float32:
        flags |= F_OUT_F32
    elif out.dtype != torch.bfloat16:
        raise TypeError("out must be bf16 or fp32")
    if accumulate:
        flags |= F_ACCUMULATE
    if bias is not None:
        flags |= F_BIAS
        if bias.dtype == torch.float32:
            flags |= F_BIAS_F32
        bias = bias.contiguous()
    ldr = 0
    if residual is not None:
        flags |= F_RESIDUAL
        if residual.dtype != torch.bfloat16 or residual.stride(-1) != 1:
            residual = residual.to(torch.bfloat16).contiguous()
        residual = residual.view(M, N) if residual.dim() != 2 else residual
        ldr = residual.stride(0)
    if _use_skinny(M, N) and not a_mn and not b_mn and not accumulate and max_ctas == 0:
        # a few row blocks (decode steps, small batches): the weight-streaming kernel
        rc = _skinny_fn()(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), flags, float(alpha),
            lib.ptr(bias), lib.ptr(residual), ldr, 0, 0, _skinny_workspace(a.device, M, N),
            lib.status_buffer().data_ptr(), lib.stream_ptr(),
        )
        lib.check_rc(rc, "lvb_gemm_skinny")
        return out
    if _copy_job_provider is not None and N > 128 and max_ctas == 0:
        job = _copy_job_provider(2.0 * M * N * K)
        if job is not None:
            table, u0, u1, srcs, n_srcs, dst = job
            rc = (_cj_pair_fn() if (PAIR_ENABLED and M > 128) else _cj_fn())(
                a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                int(a_mn), int(b_mn), flags, float(alpha), lib.ptr(bias), lib.ptr(residual), ldr,
                table, u0, u1, srcs, n_srcs, dst, lib.status_buffer().data_ptr(), lib.stream_ptr(),
            )
            lib.check_rc(rc, "lvb_gemm_bf16_copy_job")
            return out
    pair = PAIR_ENABLED and N > 128 and M > 128
    if pair and not a_mn and not b_mn and not accumulate and max_ctas == 0 and _use_pair_splitk(M, N, K):
        rc = _pair_splitk_fn()(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), flags, float(alpha),
            lib.ptr(bias), lib.ptr(residual), ldr, 0, _splitk_workspace(a.device), lib.status_buffer().data_ptr(), lib.stream_ptr(),
        )
        lib.check_rc(rc, "lvb_gemm_bf16_pair_splitk")
        return out
    rc = (_pair_fn() if pair else _fn())(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn), int(b_mn), flags, float(alpha), lib.ptr(bias), lib.ptr(residual), ldr, int(max_ctas),
        lib.status_buffer().data_ptr(), lib.stream_ptr(),
    )
    lib.check_rc(rc, "lvb_gemm_bf16_pair" if pair else "lvb_gemm_bf16")
    return out


# Large products run on CTA pairs (``csrc/gemm_pair.cu``: 256 x 256 tiles, tcgen05 cta_group::2); ``LEVANTER_B200_GEMM_PAIR=0``
# keeps everything on the one-CTA kernel.
import os as _os

PAIR_ENABLED = _os.environ.get("LEVANTER_B200_GEMM_PAIR", "1") != "0"
_pair = None


def _pair_fn():
    global _pair
    if _pair is None:
        c = lib
        _pair = lib.fn(
            "lvb_gemm_bf16_pair",
            [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
             c.c_int, c.c_int, c.c_float, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_void_p],
        )
    return _pair


_pair_splitk = None
SPLITK_MODE = _os.environ.get("LEVANTER_B200_SMALL_M", "splitk")  # what 128 < M products with few tiles run on: splitk | stream | general


def _pair_splitk_fn():
    global _pair_splitk
    if _pair_splitk is None:
        c = lib
        _pair_splitk = lib.fn("lvb_gemm_bf16_pair_splitk",
                              [c.c_void_p, c.c_void_p, c.c_void_p] + [c.c_int] * 7 + [c.c_float, c.c_void_p, c.c_void_p, c.c_int, c.c_int,
                                                                                       c.c_void_p, c.c_void_p, c.c_void_p], launches=2)
    return _pair_splitk


def _use_pair_splitk(M: int, N: int, K: int) -> bool:
    """Few 256 x 256 tiles (at most half the 74 SM pairs) and a K long enough to split, N % 4 == 0: the decode-size
    projections, where whole-K tiles would leave most SMs idle."""
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    return SPLITK_MODE == "splitk" and tiles <= 37 and K >= 1024 and N % 4 == 0


def _splitk_workspace(device) -> int:
    """The split-K scratch shared with the streaming kernel (tiles x splits <= 74 pieces of 256 x 256 fp32 fit in it)."""
    ws = _skinny_ws.get(device)
    if ws is None:
        ws = _skinny_ws[device] = torch.empty(8 * _SKINNY_SPLIT_MAX_TILES * 128 * 128 * 4, dtype=torch.uint8, device=device)
    return ws.data_ptr()


# A provider of copy jobs (``flops -> (table_ptr, u0, u1, src_ptr_array, n_srcs, dst_ptr) | None``): when one is set, dense
# GEMMs ask it before every launch and, given a job, run the kernel variant whose extra warp carries out the copies beside
# the tensor cores (the next layer's weight gather of fully sharded training, ``parallel/zero3.py``).
_copy_job_provider = None
_cj = None


def set_copy_job_provider(fn) -> None:
    global _copy_job_provider
    _copy_job_provider = fn


_cj_pair = None


def _cj_pair_fn():
    global _cj_pair
    if _cj_pair is None:
        c = lib
        _cj_pair = lib.fn("lvb_gemm_bf16_pair_copy_job",
                          [c.c_void_p, c.c_void_p, c.c_void_p] + [c.c_int] * 9 + [c.c_float, c.c_void_p, c.c_void_p, c.c_int,
                                                                                   c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_int, c.c_void_p,
                                                                                   c.c_void_p, c.c_void_p])
    return _cj_pair


def _cj_fn():
    global _cj
    if _cj is None:
        c = lib
        _cj = lib.fn("lvb_gemm_bf16_copy_job",
                     [c.c_void_p, c.c_void_p, c.c_void_p] + [c.c_int] * 9 + [c.c_float, c.c_void_p, c.c_void_p, c.c_int,
                                                                              c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_int, c.c_void_p,
                                                                              c.c_void_p, c.c_void_p])
    return _cj


SKINNY_MAX_ROWS = 128          # up to here the weight-streaming kernel always runs
SKINNY_MAX_ROWS_NARROW = 512   # up to here it runs when the general kernel's 256 x 256 tiles would leave most SMs idle
_SKINNY_NARROW_TILES = int(_os.environ.get("LEVANTER_B200_SKINNY_NARROW_TILES", "48"))
_skinny = None


def _use_skinny(M: int, N: int) -> bool:
    if M <= SKINNY_MAX_ROWS:
        return True
    if M > SKINNY_MAX_ROWS_NARROW or SPLITK_MODE != "stream":
        return False
    return ((M + 255) // 256) * ((N + 255) // 256) <= _SKINNY_NARROW_TILES


def _skinny_fn():
    global _skinny
    if _skinny is None:
        c = lib
        _skinny = lib.fn("lvb_gemm_skinny", [c.c_void_p, c.c_void_p, c.c_void_p] + [c.c_int] * 7 + [c.c_float, c.c_void_p, c.c_void_p,
                                                                                                  c.c_int, c.c_int, c.c_int, c.c_void_p, c.c_void_p,
                                                                                                  c.c_void_p], launches=2)
    return _skinny


_skinny_ws = {}


def _skinny_workspace(device, M: int, N: int) -> int:
    """Address of the per-device scratch for the split-K partials of the streaming kernel, or 0 when the launcher will not
    split (wide outputs already give every SM a tile).  Successive GEMMs on a stream reuse the scratch safely: each one's
    second kernel has consumed it before the next one's first kernel writes it."""
    if ((M + 127) // 128) * ((N + 127) // 128) > _SKINNY_SPLIT_MAX_TILES:
        return 0
    ws = _skinny_ws.get(device)
    if ws is None:
        ws = _skinny_ws[device] = torch.empty(8 * _SKINNY_SPLIT_MAX_TILES * 128 * 128 * 4, dtype=torch.uint8, device=device)
    return ws.data_ptr()


_SKINNY_SPLIT_MAX_TILES = 74  # more 128 x 128 tiles than half the SMs: the launcher does not split K


class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ b).  ``weight`` is ``[out, in]``.

    If ``weight`` carries a ``main_grad`` attribute (an fp32 buffer of the same shape, owned by the
    sharded-gradient engine) the weight gradient is accumulated straight into it by the GEMM
    epilogue and autograd sees no dense weight gradient.  If it carries a ``grad_sink`` (weights that exist only as
    row slices per rank, ``parallel/zero3.py``) the two operands of the weight-gradient product are handed to it.
    """

    @staticmethod
    def forward(ctx, x, weight, bias, residual=None):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        r2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
        y = gemm(x2, weight, bias=bias, residual=r2)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.x_shape = shp
        ctx.weight_ref = weight
        return y.view(*shp[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(ctx.weight_ref, "main_grad", None)
            sink = getattr(ctx.weight_ref, "grad_sink", None)
            if sink is not None:
                sink(dy2, x2)  # fully sharded weights: the product is reduce-scattered to the rows' owners as it is computed
                dw = None
            elif main_grad is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype if weight.dtype in (torch.bfloat16, torch.float32) else torch.float32)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0)
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres


def _tma_shapes_ok(weight: torch.Tensor) -> bool:
    """Forward, input-gradient and weight-gradient GEMMs each read ``weight`` or the activations with one of the two feature
    sizes as the row stride, and a TMA row stride must be a multiple of 16 bytes: both sizes must be multiples of 8 (a
    router with 4 experts, for one, goes to the library GEMM)."""
    return weight.dim() == 2 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Linear layer on the tcgen05 GEMM when running bf16 on a B200; ``F.linear`` otherwise."""
    if x.is_cuda and lib.available() and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and _tma_shapes_ok(weight):
        return _LinearFn.apply(x, weight, bias, None)
    return torch.nn.functional.linear(x, weight, bias)


def linear_residual(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], residual: Optional[torch.Tensor]) -> torch.Tensor:
    """``x W^T + b + residual`` with the residual added in the GEMM epilogue (one pass over the output)."""
    if residual is None:
        return linear(x, weight, bias)
    if weight.dtype != x.dtype:
        weight = weight.to(x.dtype)
        bias = bias.to(x.dtype) if bias is not None else None
    if x.is_cuda and lib.available() and x.dtype == torch.bfloat16 and residual.dtype == torch.bfloat16 and _tma_shapes_ok(weight):
        return _LinearFn.apply(x, weight, bias, residual)
    return torch.nn.functional.linear(x, weight, bias) + residual
