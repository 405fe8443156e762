"""Cautious Adam (src/levanter/optim/cautious.py): Adam update masked to the coordinates whose sign agrees with the
gradient, rescaled by the kept fraction ``u * m / (mean(m) + eps)`` (mean over each parameter tensor)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, NamedTuple, Optional

import torch

from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .transforms import GradientTransformation, Tree


class ScaleByCautiousState(NamedTuple):
    count: int
    mu: Tree
    nu: Tree


def scale_by_cautious(b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, eps_root: float = 0.0) -> GradientTransformation:
    def init(params):
        return ScaleByCautiousState(0, T.tree_zeros_like(params), T.tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        keys = T.tree_keys(updates)
        count = state.count + 1
        out = dict(updates)
        for k in keys:
            g = updates[k]
            mu, nu = state.mu[k], state.nu[k]
            mu.mul_(b1).add_(g, alpha=1 - b1)
            nu.mul_(b2).addcmul_(g, g, value=1 - b2)
            u = (mu / (1 - b1 ** count)) / (torch.sqrt(nu / (1 - b2 ** count) + eps_root) + eps)
            m = ((g * u) > 0).to(u.dtype)
            out[k] = u * m / (m.mean() + eps)
        return out, ScaleByCautiousState(count, state.mu, state.nu)

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("cautious")
@dataclass(frozen=True)
class CautiousConfig(OptimizerConfig):
    beta1: float = 0.95
    beta2: float = 0.95
    gamma: float = 0.025
    epsilon: float = 1e-8
    max_grad_norm: Optional[float] = 1.0
    adamc_weight_decay: bool = False
    needs_full_tensors = True  # the kept-fraction mean is per whole parameter tensor

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        cache: Dict = {}
        max_lr = self.learning_rate

        def _optimizer(learning_rate):
            comps = []
            if self.max_grad_norm:
                comps.append(T.clip_by_global_norm(self.max_grad_norm))
            comps.append(scale_by_cautious(self.beta1, self.beta2, self.epsilon))
            if self.weight_decay > 0:
                wd = self.weight_decay * (learning_rate / max_lr) if (self.adamc_weight_decay and max_lr > 0) else self.weight_decay
                comps.append(_decay(wd, mask_fn, cache))
            comps.append(T.scale(-learning_rate))
            return T.chain(*comps)

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
