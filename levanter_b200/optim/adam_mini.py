"""Adam-mini (src/levanter/optim/adam_mini.py): momentum per element, but one second-moment scalar per parameter *group*
chosen by role: per KV-head for q/k projections, per output neuron for v/o/other Linear weights, per token row for the
embedding and LM head (:58-113); everything else is plain AdamW.  As in the reference the second-moment buffer keeps the
full shape and holds the group mean broadcast over the group."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, NamedTuple, Optional, Tuple

import torch

from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .transforms import GradientTransformation, Tree


class ScaleByMiniState(NamedTuple):
    count: int
    momentum_buffer: Tree
    second_moment_buffer: Tree


def _group_mean(sq: torch.Tensor, role: str, lev_shape: Optional[Tuple[int, ...]]) -> torch.Tensor:
    """Mean of ``sq`` over the axes that make up one group, broadcast back to ``sq``'s shape."""
    if sq.dim() < 2:
        return sq
    if role in ("query", "key") and lev_shape is not None and len(lev_shape) >= 3:
        kv = lev_shape[0]
        v = sq.reshape(kv, -1)
        return v.mean(1, keepdim=True).expand_as(v).reshape(sq.shape)
    return sq.mean(dim=tuple(range(1, sq.dim())), keepdim=True).expand_as(sq)


def scale_with_mini(beta1: float, beta2: float, epsilon: float, role: str, shapes: Dict[str, Tuple[int, ...]]) -> GradientTransformation:
    def init(params):
        return ScaleByMiniState(0, T.tree_zeros_like(params), T.tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        count = state.count + 1
        out = dict(updates)
        for k in T.tree_keys(updates):
            g = updates[k]
            m, v = state.momentum_buffer[k], state.second_moment_buffer[k]
            m.mul_(beta1).add_(g, alpha=1 - beta1)
            v.mul_(beta2).add_(_group_mean(g * g, role, shapes.get(k)), alpha=1 - beta2)
            out[k] = (m / (1 - beta1 ** count)) / (torch.sqrt(v / (1 - beta2 ** count)) + epsilon)
        return out, ScaleByMiniState(count, state.momentum_buffer, state.second_moment_buffer)

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("mini")
@dataclass(frozen=True)
class MiniConfig(OptimizerConfig):
    lr: float = 0.02
    weight_decay: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.95
    epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    nesterov: bool = False
    needs_full_tensors = True

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        caches: Dict[str, Dict] = {}
        lev_shapes: Dict[str, Tuple[int, ...]] = {}
        if param_info is not None:
            lev_shapes = dict(getattr(param_info, "lev_shapes", {}))

        def labels(params) -> Dict[str, str]:
            out = {}
            for name, p in params.items():
                if "embedding" in name:
                    out[name] = "embedding"
                elif "q_proj" in name and name.endswith("weight"):
                    out[name] = "query"
                elif "k_proj" in name and name.endswith("weight"):
                    out[name] = "key"
                elif "v_proj" in name and name.endswith("weight"):
                    out[name] = "value"
                elif "o_proj" in name and name.endswith("weight"):
                    out[name] = "output"
                elif "lm_head" in name:
                    out[name] = "lm_head"
                elif p is not None and p.dim() == 2 and name.endswith("weight") and (
                        param_info is None or param_info.is_linear_weight(name)):
                    out[name] = "linear"
                else:
                    out[name] = "adamw"
            return out

        def optimizer(learning_rate):
            def mini(role):
                comps = [scale_with_mini(self.beta1, self.beta2, self.epsilon, role, lev_shapes)]
                if self.weight_decay > 0:
                    comps.append(_decay(self.weight_decay, mask_fn, caches.setdefault(role, {})))
                comps.append(T.scale(-learning_rate))
                return T.chain(*comps)

            adam = []
            if self.max_grad_norm:
                adam.append(T.clip_by_global_norm(self.max_grad_norm))
            adam.append(T.scale_by_adam(self.beta1, self.beta2, self.epsilon))
            if self.weight_decay > 0:
                adam.append(_decay(self.weight_decay, mask_fn, caches.setdefault("adamw", {})))
            adam.append(T.scale(-learning_rate))
            tx = {r: mini(r) for r in ("embedding", "lm_head", "query", "key", "value", "output", "linear")}
            tx["adamw"] = T.chain(*adam)
            return T.multi_transform(tx, labels)

        return T.inject_hyperparams(optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
