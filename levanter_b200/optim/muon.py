"""Muon: momentum orthogonalised by Newton-Schulz for Linear weights, AdamW for everything else
(src/levanter/optim/muon.py).

Linear weights (2-D ``[out, in]``; never embeddings or the LM head) get ``momentum(0.95, nesterov)`` -> five Newton-Schulz
iterations -> scale ``sqrt(max(1, out/in))`` (or Kimi's ``0.2 sqrt(max(out, in))``) -> weight decay -> ``-lr``.  Biases, norms,
embeddings and the LM head use AdamW with its own ``adam_lr`` (:91-111).  Muon needs whole matrices, so the engine runs it
unsharded (gradients all-reduced, momentum on every rank); the Newton-Schulz iterations, which are nearly all of the
optimizer's arithmetic, are dealt out matrix by matrix over the data ranks (``ops/newton_schulz.py:orthogonalize_tree``)
where the reference reshards every matrix over the mesh (:186-194)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, NamedTuple, Optional

import torch

from ..ops.newton_schulz import orthogonalize_tree
from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .transforms import GradientTransformation, Tree


class ScaleByMuonState(NamedTuple):
    momentum_buffer: Tree


def scale_with_muon(momentum: float = 0.95, nesterov: bool = True, steps: int = 5, muon_eps: float = 1e-8,
                    use_kimi_scaling: bool = False) -> GradientTransformation:
    steps = int(steps)

    def init(params):
        return ScaleByMuonState(T.tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        out = dict(updates)
        for k in T.tree_keys(updates):
            g = updates[k]
            buf = state.momentum_buffer[k]
            buf.mul_(momentum).add_(g)
            out[k] = momentum * buf + g if nesterov else buf
        # the matrices of the step are orthogonalised together: on several ranks each one is iterated by one rank only
        ortho = orthogonalize_tree({k: u for k, u in out.items() if u is not None and u.dim() == 2}, steps=steps, eps=muon_eps)
        for k, o in ortho.items():
            if not use_kimi_scaling:
                o = o * math.sqrt(max(1.0, o.shape[0] / o.shape[1]))
            else:
                o = o * (0.2 * math.sqrt(max(o.shape[0], o.shape[1])))
            out[k] = o
        return out, state

    return GradientTransformation(init, update)


def linear_weight_labels(param_info: Optional[ParamInfo], matrix_label: str, other_label: str):
    """Label function for ``multi_transform``: 2-D Linear weights outside embeddings / lm_head -> ``matrix_label``."""

    def labels(params) -> Dict[str, str]:
        out = {}
        for name, p in params.items():
            cls_path = (param_info.class_path(name) if param_info is not None else None) or ""
            is_linear = (param_info.is_linear_weight(name) if param_info is not None and name in param_info.module_types
                         else (p is not None and p.dim() == 2 and name.endswith("weight")))
            if "Embedding" in cls_path or "lm_head" in name or "embeddings" in name:
                out[name] = other_label
            elif is_linear and p is not None and p.dim() == 2:
                out[name] = matrix_label
            else:
                out[name] = other_label
        return out

    return labels


@OptimizerConfig.register_subclass("muon")
@dataclass(frozen=True)
class MuonConfig(OptimizerConfig):
    lr: float = 0.02
    adam_lr: float = 6e-4
    momentum: float = 0.95
    nesterov: bool = True
    backend_steps: int = 5
    weight_decay: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.95
    epsilon: float = 1e-8
    muon_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    use_kimi_scaling: bool = False
    needs_full_tensors = True

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        c1: Dict = {}
        c2: Dict = {}
        label_fn = linear_weight_labels(param_info, "muon", "adamw")

        def optimizer(learning_rate, adam_lr):
            muon = [scale_with_muon(self.momentum, self.nesterov, self.backend_steps, self.muon_epsilon, self.use_kimi_scaling)]
            if self.weight_decay > 0:
                muon.append(_decay(self.weight_decay, mask_fn, c1))
            muon.append(T.scale(-learning_rate))
            adam = []
            if self.max_grad_norm:
                adam.append(T.clip_by_global_norm(self.max_grad_norm))
            adam.append(T.scale_by_adam(self.beta1, self.beta2, self.epsilon))
            if self.weight_decay > 0:
                adam.append(_decay(self.weight_decay, mask_fn, c2))
            adam.append(T.scale(-adam_lr))
            return T.multi_transform({"muon": T.chain(*muon), "adamw": T.chain(*adam)}, label_fn)

        return T.inject_hyperparams(optimizer)(learning_rate=self.lr_scheduler(num_train_steps),
                                               adam_lr=self.lr_scheduler(num_train_steps, override_lr=self.adam_lr))
