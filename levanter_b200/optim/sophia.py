"""Sophia-H (src/levanter/optim/sophia.py): clipped Newton-like steps with a Hutchinson estimate of the Hessian diagonal.

update = ``clip(m_hat / max(gamma * h, eps), +-clip_threshold)`` then decoupled weight decay and ``-lr`` (:341-353);
every ``update_interval`` steps ``h <- b2 h + (1 - b2) * g * (H g)`` with ``g ~ N(0, 1)`` and the Hessian-vector product taken
on the *same batch objective* the step used (passed as ``obj_fn``, :367-388, 428-446).  Logs ``optim/param_norm``,
``optim/momentum_norm``, ``optim/hessian_norm`` and ``optim/unclipped_fraction``.

The Hessian-vector product is an exact double backward.  The hand-written CUDA ops define first derivatives only, so the
trainer evaluates ``obj_fn`` with the PyTorch reference implementations of the ops for that one pass every
``update_interval`` steps; the regular steps stay on the kernels.  Sophia-G is not implemented (as in the reference, :394-406)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, NamedTuple, Optional

import torch

from .. import tracker as trk
from . import transforms as T
from .config import HessianOptConfig, OptimizerConfig, ParamInfo, _decay
from .transforms import GradientTransformation, Tree
from .util import hvp, tree_gaussian_like

GAMMA_SOPHIA_G = 0.05
GAMMA_SOPHIA_H = 0.01


class ScaleBySophiaState(NamedTuple):
    count: int
    hessian_count: int
    mu: Tree
    h: Tree
    hess_key: int


def stochastic_hessian_diagonal(fn: Callable[[Dict[str, torch.Tensor]], torch.Tensor], params: Dict[str, torch.Tensor], hess_key: int) -> Tree:
    """Hutchinson estimator ``g * (H g)`` of the Hessian diagonal (Algorithm 1 of the Sophia paper)."""
    dev = next(iter(params.values())).device
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(hess_key) & 0x7FFFFFFF)
    g = tree_gaussian_like(params, generator=gen)
    product = hvp(fn, params, g)
    return {k: product[k] * g[k].to(product[k].dtype) for k in product}


def _fused_update_available(updates, state, keys) -> bool:
    from ..ops import lib

    if not keys:
        return False
    t = updates[keys[0]]
    return bool(t.is_cuda and lib.available() and all(updates[k].dtype == torch.float32 and state.mu[k].dtype == torch.float32
                                                       and state.h[k].dtype == torch.float32 and updates[k].is_contiguous() for k in keys))


_sophia_fn = {}


def _fused_update(g, mu, h, param, b1, bc1, gamma, eps, clip, stats):
    """One pass of ``csrc/sophia.cu`` over a leaf: momentum update, preconditioned and clipped step, statistics."""
    from ..ops import lib

    if "f" not in _sophia_fn:
        c = lib
        _sophia_fn["f"] = lib.fn("lvb_sophia_update", [c.c_void_p] * 5 + [c.c_longlong] + [c.c_float] * 5 + [c.c_void_p, c.c_void_p])
    u = torch.empty_like(g)
    pp = param if (param is not None and param.dtype == torch.float32 and param.is_contiguous()) else None
    rc = _sophia_fn["f"](g.data_ptr(), mu.data_ptr(), h.data_ptr(), lib.ptr(pp), u.data_ptr(), g.numel(), float(b1), float(bc1), float(gamma),
                         float(eps), float(clip) if clip is not None else 0.0, stats.data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_sophia_update")
    return u


def _sophia_gradient_transform(sophia_hess_fn, update_interval: int, b1: float, b2: float, eps: float, gamma: float,
                               clip_threshold: Optional[float], initial_key: int) -> GradientTransformation:
    def init(params):
        return ScaleBySophiaState(0, 0, T.tree_zeros_like(params), T.tree_zeros_like(params), int(initial_key))

    def update(updates, state, params=None, *, obj_fn=None, **kwargs):
        if obj_fn is None:
            raise ValueError("Sophia needs the batch objective: pass obj_fn= to update()")
        keys = T.tree_keys(updates)
        count = state.count + 1
        out = dict(updates)
        unclipped = 0.0
        total = 0
        mom_sq = torch.zeros((), device=updates[keys[0]].device)
        hess_sq = torch.zeros((), device=updates[keys[0]].device)
        par_sq = torch.zeros((), device=updates[keys[0]].device)
        fused = _fused_update_available(updates, state, keys)
        if fused:
            stats_dev = torch.zeros(4, dtype=torch.float32, device=updates[keys[0]].device)
            for k in keys:
                p_k = params.get(k) if params is not None else None
                out[k] = _fused_update(updates[k], state.mu[k], state.h[k], p_k, b1, 1 - b1 ** count, gamma, eps, clip_threshold, stats_dev)
                total += updates[k].numel()
            mom_sq, hess_sq, par_sq, unclipped = stats_dev[0], stats_dev[1], stats_dev[2], stats_dev[3]
            keys_loop = []
        else:
            keys_loop = keys
        for k in keys_loop:
            mu = state.mu[k]
            mu.mul_(b1).add_(updates[k], alpha=1 - b1)
            mu_hat = mu / (1 - b1 ** count)
            h = state.h[k]
            u = mu_hat / torch.clamp(gamma * h, min=eps)
            if clip_threshold is not None:
                unclipped = unclipped + (u.abs() < clip_threshold).float().sum()
                total += u.numel()
                u = torch.clamp(u, -clip_threshold, clip_threshold)
            out[k] = u
            mom_sq += (mu_hat.float() ** 2).sum()
            hess_sq += (h.float() ** 2).sum()
            if params is not None and params.get(k) is not None:
                par_sq += (params[k].float() ** 2).sum()
        stats = {"optim/param_norm": torch.sqrt(par_sq), "optim/momentum_norm": torch.sqrt(mom_sq),
                 "optim/hessian_norm": torch.sqrt(hess_sq)}
        if clip_threshold is not None and total:
            stats["optim/unclipped_fraction"] = unclipped / float(total)
        trk.jit_log(stats)
        hessian_count, key = state.hessian_count, state.hess_key
        if count % update_interval == 0:
            new_hess = sophia_hess_fn(obj_fn, params, hess_key=key)
            groups = T.objective_reduce_group()
            if groups:
                # obj_fn is the loss of this rank's part of the batch and the probe is the same on every rank (same key): the
                # estimate for the whole batch is the mean over the ranks
                import torch.distributed as dist

                for k in keys:
                    if k in new_hess:
                        for group in groups:
                            dist.all_reduce(new_hess[k], op=dist.ReduceOp.AVG, group=group)
            for k in keys:
                if k in new_hess:
                    state.h[k].mul_(b2).add_(new_hess[k].to(state.h[k].dtype), alpha=1 - b2)
            hessian_count += 1
            key = (key * 6364136223846793005 + 1442695040888963407) & 0x7FFFFFFFFFFFFFFF
        return out, ScaleBySophiaState(count, hessian_count, state.mu, state.h, key)

    return GradientTransformation(init, update)


@dataclass(frozen=True)
class BaseSophiaConfig(HessianOptConfig):
    weight_decay: float = 0.1
    beta1: float = 0.96
    beta2: float = 0.99
    epsilon: float = 1e-12
    clip_threshold: Optional[float] = 1.0
    rng_seed: int = 0
    gamma: float = GAMMA_SOPHIA_H
    needs_full_tensors = True
    needs_objective = True

    def compute_hessian(self, fn, params, hess_key):
        raise NotImplementedError

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        cache: Dict = {}

        def _optimizer(learning_rate, gamma):
            comps = [_sophia_gradient_transform(self.compute_hessian, self.update_interval, self.beta1, self.beta2, self.epsilon,
                                                gamma, self.clip_threshold, self.rng_seed)]
            if self.weight_decay > 0:
                comps.append(_decay(self.weight_decay, mask_fn, cache))
            comps.append(T.scale(-learning_rate))
            return T.chain(*comps)

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps),
                                                gamma=T.constant_schedule(self.gamma))


@OptimizerConfig.register_subclass("sophia-h")
@dataclass(frozen=True)
class SophiaHConfig(BaseSophiaConfig):
    gamma: float = GAMMA_SOPHIA_H

    def compute_hessian(self, fn, params, hess_key):
        return stochastic_hessian_diagonal(fn, params, hess_key=hess_key)
