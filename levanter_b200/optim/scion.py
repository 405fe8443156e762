"""Scion (src/levanter/optim/scion.py): EMA momentum ``(1 - beta) g`` orthogonalised by ten Newton-Schulz steps for Linear
weights (scaled by ``sqrt(max(1, out/in))``); Signum (sign of an EMA of gradients) for all other parameters at
``scion_to_signum_lr`` times the learning rate."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, NamedTuple, Optional

import torch

from ..ops.newton_schulz import orthogonalize_tree
from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .muon import linear_weight_labels
from .transforms import GradientTransformation, Tree


class ScaleByScionState(NamedTuple):
    momentum_buffer: Tree


def scale_by_signum(momentum: float = 0.95) -> GradientTransformation:
    def init(params):
        return ScaleByScionState(T.tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        out = dict(updates)
        for k in T.tree_keys(updates):
            buf = state.momentum_buffer[k]
            buf.mul_(momentum).add_(updates[k], alpha=1 - momentum)
            out[k] = torch.sign(buf)
        return out, state

    return GradientTransformation(init, update)


def scale_with_scion(momentum: float = 0.95, steps: int = 5, scion_eps: float = 1e-8) -> GradientTransformation:
    def init(params):
        return ScaleByScionState(T.tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        out = dict(updates)
        for k in T.tree_keys(updates):
            buf = state.momentum_buffer[k]
            buf.mul_(momentum).add_(updates[k], alpha=1 - momentum)
            out[k] = buf if buf.dim() == 2 else buf.clone()
        ortho = orthogonalize_tree({k: u for k, u in out.items() if u is not None and u.dim() == 2}, steps=steps, eps=scion_eps)
        for k, o in ortho.items():
            out[k] = o * math.sqrt(max(1.0, o.shape[0] / o.shape[1]))
        return out, state

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("scion")
@dataclass(frozen=True)
class ScionConfig(OptimizerConfig):
    lr: float = 0.02
    scion_to_signum_lr: float = 0.25
    momentum: float = 0.95
    backend_steps: int = 10
    weight_decay: float = 0.0
    beta1: float = 0.9
    scion_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    needs_full_tensors = True

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        c1: Dict = {}
        c2: Dict = {}
        label_fn = linear_weight_labels(param_info, "scion", "signum")

        def optimizer(learning_rate):
            signum_lr = learning_rate * self.scion_to_signum_lr
            scion = [scale_with_scion(self.momentum, self.backend_steps, self.scion_epsilon)]
            if self.weight_decay > 0:
                scion.append(_decay(self.weight_decay, mask_fn, c1))
            scion.append(T.scale(-learning_rate))
            signum = []
            if self.max_grad_norm:
                signum.append(T.clip_by_global_norm(self.max_grad_norm))
            signum.append(scale_by_signum(self.beta1))
            if self.weight_decay > 0:
                signum.append(_decay(self.weight_decay, mask_fn, c2))
            signum.append(T.scale(-signum_lr))
            return T.multi_transform({"scion": T.chain(*scion), "signum": T.chain(*signum)}, label_fn)

        return T.inject_hyperparams(optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
