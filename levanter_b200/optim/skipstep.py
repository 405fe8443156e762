"""Skip-step wrapper: drop an update whose loss or gradient norm is an outlier against a rolling window
(src/levanter/optim/skipstep.py:64-199).

The step is skipped (zero update, inner state kept) when either value exceeds ``mean + sigma_factor * std`` of the
last ``rolling_interval_length`` steps, once at least half a window (>= 2 points) has been seen.  The state keeps the
inner optimizer state *flattened in place* next to ``_skipstep_*`` leaves so that a skip-step run can resume from a
checkpoint written without skip-step (:20-61)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, NamedTuple, Optional, Union

import torch

from . import transforms as T
from .transforms import GradientTransformation


_SKIP_FIELDS = ("losses", "grad_norms", "valid_mask", "current_idx", "count")


class SkipStepState(NamedTuple):
    inner_opt_state: Any
    losses: torch.Tensor
    grad_norms: torch.Tensor
    valid_mask: torch.Tensor
    current_idx: int
    count: int

    # Checkpoint layout: the children of the inner state keep the key paths they have without this wrapper and the window
    # sits beside them as ``_skipstep_*`` leaves, so either kind of run can start from the other kind's checkpoint.
    def checkpoint_children(self):
        from ..tensorstore_serialization import keyed_children

        inner = keyed_children(self.inner_opt_state)
        if inner is None:  # the inner state is one leaf (or nothing): it has no children to splice in
            inner = [("inner_opt_state", self.inner_opt_state)]
        return list(inner) + [(f"_skipstep_{f}", getattr(self, f)) for f in _SKIP_FIELDS]

    def with_checkpoint_children(self, values):
        from ..tensorstore_serialization import keyed_children, rebuild_from_children

        values = list(values)
        n = len(values) - len(_SKIP_FIELDS)
        inner = values[0] if keyed_children(self.inner_opt_state) is None else rebuild_from_children(self.inner_opt_state, values[:n])
        return SkipStepState(inner, *values[n:])


def _masked_mean_std(x: torch.Tensor, mask: torch.Tensor):
    n = int(mask.sum())
    if n == 0:
        return float("nan"), float("nan")
    v = x[mask]
    mean = float(v.mean())
    std = float(v.std(unbiased=False))
    return mean, std


@dataclass(frozen=True)
class SkipStepConfig:
    rolling_interval_length: int = 128
    sigma_factor: float = 6.0

    @staticmethod
    def from_bool_int_or_config(config: Union[bool, int, "SkipStepConfig"]) -> Optional["SkipStepConfig"]:
        if isinstance(config, SkipStepConfig):
            return config
        if config is True:
            return SkipStepConfig()
        if config is False:
            return None
        if isinstance(config, int):
            return SkipStepConfig(rolling_interval_length=config)
        raise ValueError(f"Invalid type for SkipStepConfig: {type(config)}")

    @staticmethod
    def from_config_value(v):
        return SkipStepConfig.from_bool_int_or_config(v)

    def wrap(self, inner: GradientTransformation) -> GradientTransformation:
        n = self.rolling_interval_length

        def init(params):
            return SkipStepState(inner.init(params), torch.zeros(n), torch.zeros(n), torch.zeros(n, dtype=torch.bool), 0, 0)

        def update(updates, state: SkipStepState, params=None, *, loss=None, **extra):
            if loss is None:
                raise ValueError("Loss must be provided as a keyword argument to the update function when using SkipStepOptimizer.")
            loss_v = float(loss)
            gnorm = float(T.global_norm(updates))
            min_points = max(2, n // 2)
            can_skip = state.count >= min_points
            lm, ls = _masked_mean_std(state.losses, state.valid_mask)
            gm, gs = _masked_mean_std(state.grad_norms, state.valid_mask)
            ls = max(ls, 1e-6) if ls == ls else ls
            gs = max(gs, 1e-6) if gs == gs else gs
            loss_thr = lm + self.sigma_factor * ls
            g_thr = gm + self.sigma_factor * gs
            loss_ok = loss_v <= loss_thr
            g_ok = gnorm <= g_thr
            should_skip = not (loss_ok and g_ok)
            skip = bool(can_skip and should_skip)
            losses = state.losses.clone()
            gns = state.grad_norms.clone()
            vm = state.valid_mask.clone()
            losses[state.current_idx] = loss_v
            gns[state.current_idx] = gnorm
            vm[state.current_idx] = True
            try:
                from .. import tracker

                tracker.jit_log({
                    "optim/skipped_step": float(skip), "optim/skip_step/loss_threshold": loss_thr,
                    "optim/skip_step/loss": loss_v, "optim/skip_step/loss_std": ls,
                    "optim/skip_step/grad_norm_threshold": g_thr, "optim/skip_step/grad_norm": gnorm,
                    "optim/skip_step/grad_norm_std": gs})
            except Exception:
                pass
            if skip:
                new_updates = T.tree_map(torch.zeros_like, updates)
                new_inner = state.inner_opt_state
            else:
                new_updates, new_inner = inner.update(updates, state.inner_opt_state, params, loss=loss, **extra) \
                    if _accepts_loss(inner) else inner.update(updates, state.inner_opt_state, params, **extra)
            return new_updates, SkipStepState(new_inner, losses, gns, vm, (state.current_idx + 1) % n, min(state.count + 1, n))

        return GradientTransformation(init, update)


def _accepts_loss(t: GradientTransformation) -> bool:
    return False
