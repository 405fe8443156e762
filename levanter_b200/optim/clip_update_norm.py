"""Clip the update's global norm to ``mean + sigma_factor * std`` of its own rolling history
(src/levanter/optim/clip_update_norm.py:20-115).  The history stores the *unclipped* norm."""
from __future__ import annotations

from dataclasses import dataclass
from typing import NamedTuple

import torch

from . import transforms as T
from .skipstep import _masked_mean_std
from .transforms import GradientTransformation


class ClipUpdateNormState(NamedTuple):
    update_norms: torch.Tensor
    valid_mask: torch.Tensor
    current_idx: int
    count: int


@dataclass(frozen=True)
class ClipUpdateNormConfig:
    rolling_interval_length: int = 128
    sigma_factor: float = 3.0

    def build(self) -> GradientTransformation:
        return clip_update_by_historical_norm(self.rolling_interval_length, self.sigma_factor)


def clip_update_by_historical_norm(rolling_interval_length: int = 128, sigma_factor: float = 3.0) -> GradientTransformation:
    n = rolling_interval_length

    def init(params):
        return ClipUpdateNormState(torch.zeros(n), torch.zeros(n, dtype=torch.bool), 0, 0)

    def update(updates, state: ClipUpdateNormState, params=None, **extra):
        gnorm = float(T.global_norm(updates))
        can_clip = state.count >= max(2, n // 2)
        mean, std = _masked_mean_std(state.update_norms, state.valid_mask)
        std = max(std, 1e-6) if std == std else std
        thr = mean + sigma_factor * std
        max_norm = thr if can_clip else float("inf")
        factor = max_norm / max(gnorm, 1e-6) if gnorm > max_norm else 1.0
        if factor != 1.0:
            keys = T.tree_keys(updates)
            torch._foreach_mul_([updates[k] for k in keys], factor)
        try:
            from .. import tracker

            tracker.jit_log({"optim/clip_update/did_clip": float(factor < 1.0), "optim/clip_update/pre_clip_norm": gnorm,
                             "optim/clip_update/update_norm_threshold": thr,
                             "optim/clip_update/post_clip_norm": min(max_norm, gnorm)})
        except Exception:
            pass
        norms = state.update_norms.clone()
        vm = state.valid_mask.clone()
        norms[state.current_idx] = gnorm
        vm[state.current_idx] = True
        return updates, ClipUpdateNormState(norms, vm, (state.current_idx + 1) % n, min(state.count + 1, n))

    return GradientTransformation(init, update)
