"""Bindings of the one-pass analysis kernels (``csrc/analysis.cu``): tensor summary + histogram and per-row entropy / top-2
gap of logits.  Each has a PyTorch statement of the same computation for CPU tensors, which is also the test oracle."""
from __future__ import annotations

from typing import Tuple

import torch

from . import lib

_f = {}


def _bind():
    if not _f:
        P, I, L = lib.c_void_p, lib.c_int, lib.c_longlong
        _f["summary"] = lib.fn("lvb_tensor_summary", [P, L, I, P, P, P], launches=2)
        _f["hist"] = lib.fn("lvb_histogram", [P, L, I, P, I, P, P])
        _f["ent"] = lib.fn("lvb_entropy_top2", [P, I, I, L, I, P, P, P, P])


def _kernel_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and lib.available() and x.dtype in (torch.float32, torch.bfloat16) and x.numel() > 0


def summary_and_histogram(x: torch.Tensor, bins: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(summary[4] = min, max, sum, sum of squares; counts[bins] int32)`` of all elements of ``x``, binned over
    ``[min, max]``, in two reads of ``x`` and without a host synchronisation in between.  CUDA fp32/bf16 tensors only."""
    assert _kernel_ok(x) and bins <= 256
    _bind()
    x = x.detach().contiguous()
    dev = x.device
    scratch = torch.empty(4096, dtype=torch.float32, device=dev)
    summary = torch.empty(4, dtype=torch.float32, device=dev)
    counts = torch.zeros(bins, dtype=torch.int32, device=dev)
    bf = 1 if x.dtype == torch.bfloat16 else 0
    lib.check_rc(_f["summary"](x.data_ptr(), x.numel(), bf, scratch.data_ptr(), summary.data_ptr(), lib.stream_ptr()), "lvb_tensor_summary")
    lib.check_rc(_f["hist"](x.data_ptr(), x.numel(), bf, summary.data_ptr(), bins, counts.data_ptr(), lib.stream_ptr()), "lvb_histogram")
    return summary, counts


def histogram_counts(x: torch.Tensor, lo: float, hi: float, bins: int) -> torch.Tensor:
    """Bin counts (int32) of ``x`` over a range the caller already knows (shared edges of a sharded tensor)."""
    assert _kernel_ok(x) and bins <= 256
    _bind()
    x = x.detach().contiguous()
    rng = torch.tensor([lo, hi], dtype=torch.float32, device=x.device)
    counts = torch.zeros(bins, dtype=torch.int32, device=x.device)
    lib.check_rc(_f["hist"](x.data_ptr(), x.numel(), 1 if x.dtype == torch.bfloat16 else 0, rng.data_ptr(), bins, counts.data_ptr(),
                            lib.stream_ptr()), "lvb_histogram")
    return counts


def entropy_top2_reference(logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    z = logits.float()
    lse = torch.logsumexp(z, dim=-1)
    p = torch.exp(z - lse.unsqueeze(-1))
    ent = lse - torch.where(p > 0, p * z, torch.zeros_like(z)).sum(-1)
    top = torch.topk(z, 2, dim=-1).values
    return ent, top[..., 0] - top[..., 1], lse


def entropy_top2(logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per row of ``logits[..., V]``: predictive entropy, gap between the two largest logits, log-sum-exp (fp32), from one
    streaming read of the logits on a B200; the PyTorch statement elsewhere."""
    if not _kernel_ok(logits) or logits.shape[-1] < 2:
        return entropy_top2_reference(logits)
    _bind()
    V = logits.shape[-1]
    z = logits.detach().reshape(-1, V)
    if z.stride(-1) != 1:
        z = z.contiguous()
    rows = z.shape[0]
    ent, gap, lse = (torch.empty(rows, dtype=torch.float32, device=z.device) for _ in range(3))
    rc = _f["ent"](z.data_ptr(), rows, V, z.stride(0), 1 if z.dtype == torch.bfloat16 else 0, ent.data_ptr(), gap.data_ptr(), lse.data_ptr(),
                   lib.stream_ptr())
    lib.check_rc(rc, "lvb_entropy_top2")
    shape = logits.shape[:-1]
    return ent.view(shape), gap.view(shape), lse.view(shape)
