"""LM-head GEMM + cross-entropy without ever holding ``[tokens, vocab]``.

Tokens are processed in chunks: the tcgen05 GEMM writes a chunk of fp32 logits into a reusable buffer,
``lvb_ce_stats`` reduces every row to (logsumexp, target logit); the backward pass recomputes the chunk,
``lvb_ce_grad`` writes bf16 dlogits and two more GEMMs produce dX and accumulate dW.  Same mathematics as the
reference's vocab-blockwise loss (src/levanter/models/loss.py:251-507: online logsumexp forward, recompute in
backward, ``dlogits = (g_loss + g_logz) * p - g_loss * onehot``), tiled over tokens instead of vocab because the
GEMM wants long K-major rows of the head matrix.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import lib
from .gemm import gemm

_f = {}
_buffers: dict = {}


def _stats():
    if "s" not in _f:
        c = lib
        _f["s"] = lib.fn("lvb_ce_stats", [c.c_void_p, c.c_longlong, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_float, c.c_void_p, c.c_void_p])
    return _f["s"]


def _grad():
    if "g" not in _f:
        c = lib
        _f["g"] = lib.fn("lvb_ce_grad", [c.c_void_p, c.c_longlong] + [c.c_void_p] * 5 + [c.c_longlong, c.c_int, c.c_int, c.c_float, c.c_void_p])
    return _f["g"]


def _buffer(key, shape, dtype, device):
    k = (key, torch.cuda.current_device())
    b = _buffers.get(k)
    n = 1
    for s in shape:
        n *= s
    if b is None or b.numel() < n or b.dtype != dtype:
        b = torch.empty(n, dtype=dtype, device=device)
        _buffers[k] = b
    return b[:n].view(*shape)


def chunk_rows_for(vocab: int, budget_bytes: int = 1 << 30) -> int:
    rows = budget_bytes // (vocab * 4)
    rows = max(256, (rows // 256) * 256)
    return min(rows, 16384)


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, targets, soft_cap, z_weight, chunk_rows):
        T, E = x.shape
        V = weight.shape[0]
        x = x.contiguous()
        tg = targets.to(torch.int32).contiguous()
        lse = torch.empty(T, dtype=torch.float32, device=x.device)
        tl = torch.empty(T, dtype=torch.float32, device=x.device)
        chunk = chunk_rows or chunk_rows_for(V)
        Vp = (V + 3) // 4 * 4
        logits = _buffer("logits", (min(chunk, T), Vp), torch.float32, x.device)
        cap = float(soft_cap) if soft_cap is not None else 0.0
        st = lib.status_buffer().data_ptr()
        for r0 in range(0, T, chunk):
            n = min(chunk, T - r0)
            lg = logits[:n, :V] if Vp != V else logits[:n]
            gemm(x[r0:r0 + n], weight, out=lg)
            rc = _stats()(lg.data_ptr(), lg.stride(0), tg[r0:].data_ptr(), lse[r0:].data_ptr(), tl[r0:].data_ptr(), n, V, cap,
                          st, lib.stream_ptr())
            lib.check_rc(rc, "lvb_ce_stats")
        ctx.save_for_backward(x, weight, tg, lse)
        ctx.cap, ctx.z, ctx.chunk = cap, float(z_weight or 0.0), chunk
        ctx.weight_ref = weight
        loss = lse - tl
        if ctx.z != 0.0:
            loss = loss + ctx.z * lse * lse
        ctx.mark_non_differentiable(lse)
        return loss, lse

    @staticmethod
    def backward(ctx, dloss, _dlse):
        x, weight, tg, lse = ctx.saved_tensors
        T, E = x.shape
        V = weight.shape[0]
        chunk = ctx.chunk
        Vp = (V + 3) // 4 * 4
        Vd = (V + 7) // 8 * 8
        logits = _buffer("logits", (min(chunk, T), Vp), torch.float32, x.device)
        dlog = _buffer("dlogits", (min(chunk, T), Vd), torch.bfloat16, x.device)
        g_loss = dloss.float().contiguous()
        g_logz = (g_loss * (2.0 * ctx.z) * lse).contiguous() if ctx.z != 0.0 else None
        dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
        need_dw = ctx.needs_input_grad[1]
        main_grad = getattr(ctx.weight_ref, "main_grad", None) if need_dw else None
        dw = None
        if need_dw and main_grad is None:
            dw = torch.zeros(V, E, dtype=torch.float32, device=x.device)
        acc = main_grad if main_grad is not None else dw
        for r0 in range(0, T, chunk):
            n = min(chunk, T - r0)
            lg = logits[:n, :V] if Vp != V else logits[:n]
            gemm(x[r0:r0 + n], weight, out=lg)
            dl = dlog[:n, :V] if Vd != V else dlog[:n]
            rc = _grad()(lg.data_ptr(), lg.stride(0), tg[r0:].data_ptr(), lse[r0:].data_ptr(), g_loss[r0:].data_ptr(),
                         g_logz[r0:].data_ptr() if g_logz is not None else 0, dl.data_ptr(), dl.stride(0), n, V, ctx.cap,
                         lib.stream_ptr())
            lib.check_rc(rc, "lvb_ce_grad")
            if dx is not None:
                gemm(dl, weight, b_mn=True, out=dx[r0:r0 + n])
            if need_dw:
                gemm(dl, x[r0:r0 + n], a_mn=True, b_mn=True, out=acc, accumulate=True)
        if dw is not None:
            dw = dw.to(weight.dtype)
        return dx, dw, None, None, None, None


def fused_linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, *, soft_cap: Optional[float] = None,
                               z_weight: Optional[float] = None, chunk_rows: Optional[int] = None):
    """Per-token ``(loss, logsumexp)`` of ``softmax(x @ weight.T)`` against ``targets``; ``x[T,E]`` bf16, ``weight[V,E]`` bf16."""
    return _FusedLinearCE.apply(x, weight, targets, soft_cap, z_weight, chunk_rows)


def kernel_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.is_cuda and lib.available() and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0)
