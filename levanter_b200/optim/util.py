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


# ------------------------------------------------------------------------------------------ linear layers as matrices
# The reference articulates a linear layer's weight over several named axes (heads, head size, ...) and flattens it to a
# matrix before matrix-valued optimizers see it (src/levanter/optim/util.py:83-212).  Here a linear weight is stored as the
# matrix ``[out, in]`` already; what can have more axes is a stacked (per-layer or per-expert) leaf, whose leading axes index
# independent matrices.  These helpers give matrix-valued transformations one view of all of them.
def flatten_linear_layers(tree: Dict[str, torch.Tensor], is_linear: Optional[Callable[[str, torch.Tensor], bool]] = None) -> Dict[str, torch.Tensor]:
    """Every linear weight as a stack of matrices ``[..., out, in]`` -> ``[n, out, in]`` (``n = 1`` for a plain matrix);
    other leaves are returned unchanged.  ``is_linear`` defaults to "at least two axes"."""
    pick = is_linear or (lambda name, t: t is not None and t.dim() >= 2)
    return {k: (v.reshape(-1, v.shape[-2], v.shape[-1]) if pick(k, v) else v) for k, v in tree.items()}


def unflatten_linear_layers(template: Dict[str, torch.Tensor], flat: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Inverse of :func:`flatten_linear_layers`: every leaf takes the shape of the same leaf in ``template``."""
    return {k: (v.reshape(template[k].shape) if v is not None and template.get(k) is not None else v) for k, v in flat.items()}


def map_flattened_linear_layers(f: Callable[[torch.Tensor], torch.Tensor], params: Dict[str, torch.Tensor], *,
                                or_else: Optional[Callable[[torch.Tensor], torch.Tensor]] = None,
                                is_linear: Optional[Callable[[str, torch.Tensor], bool]] = None) -> Dict[str, torch.Tensor]:
    """Apply ``f`` to every matrix of every linear weight (stacked leaves are mapped matrix by matrix, the reference's vmap
    over scan layers) and ``or_else`` (default: identity) to the other leaves; shapes are preserved."""
    pick = is_linear or (lambda name, t: t is not None and t.dim() >= 2)
    out = {}
    for k, v in params.items():
        if v is not None and pick(k, v):
            mats = v.reshape(-1, v.shape[-2], v.shape[-1])
            out[k] = torch.stack([f(m) for m in mats]).reshape(v.shape)
        else:
            out[k] = or_else(v) if (or_else is not None and v is not None) else v
    return out
