"""RMSProp with momentum (src/levanter/optim/rmsprop.py): gradient divided by the bias-corrected RMS, then an EMA
momentum with bias correction."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, NamedTuple, Optional

import torch

from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .transforms import GradientTransformation, Tree


class ScaleByRMSPropMomState(NamedTuple):
    count: int
    mean_square: Tree
    momentum: Tree


def scale_by_rmsprop_momentum(beta1: float = 0.9, beta2: float = 0.99, eps: float = 1e-30) -> GradientTransformation:
    def init(params):
        return ScaleByRMSPropMomState(0, T.tree_zeros_like(params), T.tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        keys = T.tree_keys(updates)
        count = state.count + 1
        out = dict(updates)
        for k in keys:
            g = updates[k]
            ms, mom = state.mean_square[k], state.momentum[k]
            ms.mul_(beta2).addcmul_(g, g, value=1 - beta2)
            scaled = g / (torch.sqrt(ms / (1 - beta2 ** count)) + eps)
            mom.mul_(beta1).add_(scaled, alpha=1 - beta1)
            out[k] = mom / (1 - beta1 ** count)
        return out, ScaleByRMSPropMomState(count, state.mean_square, state.momentum)

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("rmsprop")
@dataclass(frozen=True)
class RMSPropMomentumConfig(OptimizerConfig):
    beta1: float = 0.9
    beta2: float = 0.99
    eps: float = 1e-30
    max_grad_norm: Optional[float] = 1.0
    weight_decay: float = 0.1

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        cache: Dict = {}

        def _optimizer(learning_rate):
            comps = []
            if self.max_grad_norm:
                comps.append(T.clip_by_global_norm(self.max_grad_norm))
            comps.append(scale_by_rmsprop_momentum(self.beta1, self.beta2, self.eps))
            if self.weight_decay > 0:
                comps.append(_decay(self.weight_decay, mask_fn, cache))
            comps.append(T.scale(-learning_rate))
            return T.chain(*comps)

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
