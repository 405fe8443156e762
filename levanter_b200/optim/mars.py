"""MARS (src/levanter/optim/mars.py): Adam on the variance-reduced gradient ``c = g + gamma * b1 / (1 - b1) * (g - g_prev)``,
clipped to ``max_grad_norm`` before the moments are updated."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, NamedTuple, Optional

import torch

from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .transforms import GradientTransformation, Tree


class ScaleByMarsState(NamedTuple):
    count: int
    mu: Tree
    nu: Tree
    mog: Tree


def scale_by_mars(b1: float = 0.9, b2: float = 0.999, gamma: float = 0.05, eps: float = 1e-8, eps_root: float = 0.0,
                  max_grad_norm: float = 0.0) -> GradientTransformation:
    def init(params):
        return ScaleByMarsState(0, T.tree_zeros_like(params), T.tree_zeros_like(params), T.tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        keys = T.tree_keys(updates)
        coef = gamma * b1 / (1 - b1)
        c = {k: updates[k] + coef * (updates[k] - state.mog[k]) for k in keys}
        if max_grad_norm:
            gn = T.global_norm(c)
            s = torch.clamp(max_grad_norm / (gn + 1e-6), max=1.0)
            c = {k: v * s.to(v.device) for k, v in c.items()}
        count = state.count + 1
        out = dict(updates)
        for k in keys:
            mu, nu = state.mu[k], state.nu[k]
            mu.mul_(b1).add_(c[k], alpha=1 - b1)
            nu.mul_(b2).addcmul_(c[k], c[k], value=1 - b2)
            out[k] = (mu / (1 - b1 ** count)) / (torch.sqrt(nu / (1 - b2 ** count) + eps_root) + eps)
            state.mog[k].copy_(updates[k])
        return out, ScaleByMarsState(count, state.mu, state.nu, state.mog)

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("mars")
@dataclass(frozen=True)
class MarsConfig(OptimizerConfig):
    weight_decay: float = 0.1
    beta1: float = 0.95
    beta2: float = 0.99
    gamma: float = 0.025
    epsilon: float = 1e-8
    max_grad_norm: Optional[float] = 1.0

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        cache: Dict = {}

        def _optimizer(learning_rate):
            comps = [scale_by_mars(self.beta1, self.beta2, self.gamma, self.epsilon, max_grad_norm=self.max_grad_norm or 0.0)]
            if self.weight_decay > 0:
                comps.append(_decay(self.weight_decay, mask_fn, cache))
            comps.append(T.scale(-learning_rate))
            return T.chain(*comps)

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
