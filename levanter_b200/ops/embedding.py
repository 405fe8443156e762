"""Token-embedding gather and its gradient on this library's kernels (``csrc/embedding.cu``).

Forward is a row gather; backward adds the output gradient into the rows of the fp32 gradient accumulator (``main_grad``)
in a fixed order, so the result is bitwise reproducible.  Without an accumulator (a bare parameter) the dense gradient is
formed the same way into a zero matrix.  Replaces ``hnn.Embedding`` (src/levanter/models/llama.py:460-468)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import lib

_f = {}


def _fwd():
    if "f" not in _f:
        c = lib
        _f["f"] = lib.fn("lvb_embedding_fwd", [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_void_p, c.c_void_p])
    return _f["f"]


def _bwd():
    if "b" not in _f:
        c = lib
        _f["b"] = lib.fn("lvb_embedding_bwd", [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_float,
                                               c.c_void_p, c.c_void_p])
    return _f["b"]


def scatter_add_rows(ids: torch.Tensor, dy: torch.Tensor, grad: torch.Tensor, scale: float = 1.0) -> None:
    """``grad[ids[t]] += scale * dy[t]`` for bf16 ``dy [T, D]`` into fp32 ``grad [V, D]``, deterministically."""
    flat = ids.reshape(-1).to(torch.int32)
    sorted_ids, order = torch.sort(flat, stable=True)
    order = order.to(torch.int32)
    dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
    rc = _bwd()(sorted_ids.data_ptr(), order.data_ptr(), dy2.data_ptr(), grad.data_ptr(), flat.numel(), dy2.shape[1], grad.shape[0],
                float(scale), lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_embedding_bwd")


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        flat = ids.reshape(-1).to(torch.int32).contiguous()
        out = torch.empty(flat.numel(), weight.shape[1], dtype=weight.dtype, device=weight.device)
        rc = _fwd()(flat.data_ptr(), weight.data_ptr(), out.data_ptr(), flat.numel(), weight.shape[1], weight.shape[0],
                    lib.status_buffer().data_ptr(), lib.stream_ptr())
        lib.check_rc(rc, "lvb_embedding_fwd")
        ctx.save_for_backward(flat)
        ctx.weight_ref = weight
        return out.view(*ids.shape, weight.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        w = ctx.weight_ref
        if dy.dtype != torch.bfloat16:
            dy = dy.to(torch.bfloat16)
        main = getattr(w, "main_grad", None)
        if main is not None:
            scatter_add_rows(flat, dy, main)
            return None, None
        g = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        scatter_add_rows(flat, dy, g)
        return None, g.to(w.dtype)


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if (weight.is_cuda and lib.available() and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
            and weight.is_contiguous()):
        return _EmbeddingFn.apply(ids, weight)
    return F.embedding(ids, weight)
