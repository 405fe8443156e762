"""ADOPT (src/levanter/optim/adopt.py): Adam variant that normalises the gradient by the *previous* second moment and
applies momentum afterwards; the first step produces a zero update."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, NamedTuple, Optional

import torch

from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .transforms import GradientTransformation, Tree


class ScaleByAdoptState(NamedTuple):
    count: int
    mu: Tree
    nu: Tree


def scale_by_adopt(b1: float = 0.9, b2: float = 0.999, eps: float = 1e-6, eps_root: float = 0.0) -> GradientTransformation:
    def init(params):
        return ScaleByAdoptState(0, T.tree_zeros_like(params), T.tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        keys = T.tree_keys(updates)
        g = [updates[k] for k in keys]
        mu = [state.mu[k] for k in keys]
        nu = [state.nu[k] for k in keys]
        if state.count == 0:
            normed = [torch.zeros_like(x) for x in g]
        else:
            bc = 1.0 - b2 ** state.count
            denom = torch._foreach_div(nu, bc)
            if eps_root:
                torch._foreach_add_(denom, eps_root)
            torch._foreach_sqrt_(denom)
            torch._foreach_add_(denom, eps)
            normed = torch._foreach_div(g, denom)
        torch._foreach_mul_(mu, b1)
        torch._foreach_add_(mu, normed, alpha=1 - b1)
        torch._foreach_mul_(nu, b2)
        torch._foreach_addcmul_(nu, g, g, value=1 - b2)
        count = state.count + 1
        mu_hat = torch._foreach_div(mu, 1.0 - b1 ** count)
        out = dict(updates)
        for k, u in zip(keys, mu_hat):
            out[k] = u
        return out, ScaleByAdoptState(count, state.mu, state.nu)

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("adopt")
@dataclass(frozen=True)
class AdoptConfig(OptimizerConfig):
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    epsilon: float = 1e-6
    max_grad_norm: Optional[float] = 1.0
    schedule_list: Optional[List[str]] = None

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        cache: Dict = {}

        def _optimizer(learning_rate):
            comps = []
            if self.max_grad_norm:
                comps.append(T.clip_by_global_norm(self.max_grad_norm))
            comps.append(scale_by_adopt(self.beta1, self.beta2, self.epsilon))
            if self.weight_decay > 0:
                comps.append(_decay(self.weight_decay, mask_fn, cache))
            comps.append(T.scale(-learning_rate))
            return T.chain(*comps)

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
