"""Optimizer utilities: Gaussian trees, norm logging, block-RMS clipping, Hessian-vector products
(src/levanter/optim/util.py)."""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from . import transforms as T
from .transforms import GradientTransformation, Tree


def tree_gaussian_like(tree: Tree, generator: Optional[torch.Generator] = None) -> Tree:
    """Standard-normal noise with the structure of ``tree`` (None for non-float leaves)."""
    out = {}
    for k, v in tree.items():
        if v is None or not v.is_floating_point():
            out[k] = None
        else:
            out[k] = torch.randn(v.shape, dtype=torch.float32, device=v.device, generator=generator).to(v.dtype)
    return out


def log_norm_passthrough(desc: str) -> GradientTransformation:
    def update(updates, state, params=None, **extra):
        try:
            from .. import tracker

            tracker.jit_log({desc: float(T.global_norm(updates))})
        except Exception:
            pass
        return updates, state

    return GradientTransformation(lambda p: T.EmptyState(), update)


def scan_aware_clip_by_block_rms(threshold: float) -> GradientTransformation:
    """Per-tensor RMS clip: ``u / max(1, rms(u) / threshold)``.  Parameters are per-layer tensors here, so this is
    already "scan aware" (the reference vmaps over the stacked layer axis, src/levanter/optim/util.py:62-77)."""

    def update(updates, state, params=None, **extra):
        def clip(u):
            rms = torch.sqrt(torch.mean(u.float() * u.float()))
            return u / torch.clamp(rms / threshold, min=1.0).to(u.dtype)

        return T.tree_map(clip, updates), state

    return GradientTransformation(lambda p: T.EmptyState(), update)


scale_by_update_rms_clipping = scan_aware_clip_by_block_rms


def hvp(f: Callable[[Dict[str, torch.Tensor]], torch.Tensor], params: Dict[str, torch.Tensor], v: Tree) -> Tree:
    """Hessian-vector product of scalar ``f(params)`` along ``v`` by double backward."""
    names = [k for k, p in params.items() if p is not None and v.get(k) is not None]
    # leaves that do not require gradients (plain tensors handed in by a caller) are differentiated through a detached alias
    params = {k: (p if (p is None or p.requires_grad) else p.detach().requires_grad_()) for k, p in params.items()}
    ps = [params[k] for k in names]
    with torch.enable_grad():
        loss = f(params)
    grads = torch.autograd.grad(loss, ps, create_graph=True, allow_unused=True)
    dot = sum((g * v[k].to(g.dtype)).sum() for g, k in zip(grads, names) if g is not None)
    hv = torch.autograd.grad(dot, ps, allow_unused=True)
    return {k: (h if h is not None else torch.zeros_like(params[k])) for k, h in zip(names, hv)}
