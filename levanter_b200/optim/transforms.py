"""Composable gradient transformations over flat ``{path: tensor}`` trees.

The reference builds its optimizers from Optax transformations (``chain(clip_by_global_norm, scale_by_adam,
add_decayed_weights, scale(-lr))`` under ``inject_hyperparams``, src/levanter/optim/config.py:458-494).  This module
supplies the same algebra in PyTorch so every optimizer keeps the reference's composition order *and* its state-tree
shape (``inner_state/<i>/mu/<param path>`` ...), which is what the checkpoint format records.

A "tree" is a ``dict`` from parameter path to tensor (entries may be ``None`` for masked-out leaves).  States are nested
dicts / tuples of tensors and Python scalars.  All arithmetic is done with ``torch._foreach_*`` kernels over the
leaves; in distributed runs each leaf is the local shard and ``global_norm`` all-reduces the squared sum.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, NamedTuple, Optional, Sequence, Tuple, Union

import torch

Tree = Dict[str, Optional[torch.Tensor]]
Schedule = Callable[[int], float]
ScalarOrSchedule = Union[float, Schedule]


class GradientTransformation(NamedTuple):
    init: Callable[[Tree], Any]
    update: Callable[..., Tuple[Tree, Any]]  # (updates, state, params=None, **extra) -> (updates, state)


class EmptyState(NamedTuple):
    pass


# ----------------------------------------------------------------------------------------------- tree helpers
def tree_keys(t: Tree) -> List[str]:
    return [k for k, v in t.items() if v is not None]


def tree_map(fn, tree: Tree, *rest: Tree) -> Tree:
    out = {}
    for k, v in tree.items():
        if v is None:
            out[k] = None
        else:
            out[k] = fn(v, *[r[k] for r in rest])
    return out


def tree_zeros_like(tree: Tree, dtype=None) -> Tree:
    return {k: (None if v is None else torch.zeros_like(v, dtype=dtype or v.dtype)) for k, v in tree.items()}


def _leaves(tree: Tree, keys: Sequence[str]) -> List[torch.Tensor]:
    return [tree[k] for k in keys]


_dist_group = None


def set_norm_reduce_group(group) -> None:
    """Process group over which parameter shards are spread; ``global_norm`` sums squared norms across it."""
    global _dist_group
    _dist_group = group


_objective_group = None


def set_objective_reduce_group(group) -> None:
    """Process groups (a list, one per mesh axis) whose ranks each hold a different part of the step's batch.  A transformation that differentiates the
    batch objective itself (Sophia's Hessian estimate) averages its result over it, so that replicated optimizer state stays
    the same on every rank.  ``None`` clears."""
    global _objective_group
    _objective_group = group


def objective_reduce_group():
    return _objective_group


_model_group = None
_model_sharded: Optional[set] = None


def set_model_parallel_norm(group, sharded_names) -> None:
    """Tensor parallelism: ``sharded_names`` are the leaves of which every rank of ``group`` (the model axis) holds a different
    slice; ``global_norm`` sums their squared norms over the group and counts the replicated leaves once.  ``None`` clears."""
    global _model_group, _model_sharded
    _model_group = group
    _model_sharded = set(sharded_names) if (group is not None and sharded_names is not None) else None


def global_norm(tree: Tree) -> torch.Tensor:
    keys = tree_keys(tree)
    if not keys:
        return torch.zeros(())
    import torch.distributed as dist

    def sumsq(ks):
        if not ks:
            return torch.zeros((), dtype=torch.float32, device=tree[keys[0]].device)
        norms = torch._foreach_norm(_leaves(tree, ks))
        return torch.stack([n.float() ** 2 for n in norms]).sum()

    if _model_group is not None and _model_sharded is not None:
        part = sumsq([k for k in keys if k in _model_sharded])
        rep = sumsq([k for k in keys if k not in _model_sharded])
        if _dist_group is not None:  # slices over the data axis first: both kinds of leaves are cut there
            both = torch.stack([part, rep])
            dist.all_reduce(both, group=_dist_group if _dist_group is not True else None)
            part, rep = both[0], both[1]
        dist.all_reduce(part, group=_model_group)
        return torch.sqrt(part + rep)
    sq = sumsq(keys)
    if _dist_group is not None:
        dist.all_reduce(sq, group=_dist_group if _dist_group is not True else None)
    return torch.sqrt(sq)


def _value(x: ScalarOrSchedule, count: int) -> float:
    return float(x(count)) if callable(x) else float(x)


# ----------------------------------------------------------------------------------------------- basic transforms
def identity() -> GradientTransformation:
    return GradientTransformation(lambda p: EmptyState(), lambda u, s, p=None, **kw: (u, s))


def chain(*transforms: GradientTransformation) -> GradientTransformation:
    def init(params):
        return tuple(t.init(params) for t in transforms)

    def update(updates, state, params=None, **extra):
        new_state = []
        for t, s in zip(transforms, state):
            updates, s2 = t.update(updates, s, params, **extra)
            new_state.append(s2)
        return updates, tuple(new_state)

    return GradientTransformation(init, update)


def scale(factor: float) -> GradientTransformation:
    def update(updates, state, params=None, **extra):
        keys = tree_keys(updates)
        if not keys:
            return updates, state
        torch._foreach_mul_(_leaves(updates, keys), factor)
        return updates, state

    return GradientTransformation(lambda p: EmptyState(), update)


class ScaleByScheduleState(NamedTuple):
    count: int


def scale_by_schedule(fn: Schedule) -> GradientTransformation:
    def update(updates, state, params=None, **extra):
        f = float(fn(state.count))
        keys = tree_keys(updates)
        if not keys:
            return updates, state
        torch._foreach_mul_(_leaves(updates, keys), f)
        return updates, ScaleByScheduleState(state.count + 1)

    return GradientTransformation(lambda p: ScaleByScheduleState(0), update)


def scale_by_learning_rate(lr: ScalarOrSchedule, flip_sign: bool = True) -> GradientTransformation:
    m = -1.0 if flip_sign else 1.0
    if callable(lr):
        return scale_by_schedule(lambda c: m * lr(c))
    return scale(m * lr)


def clip_by_global_norm(max_norm: float) -> GradientTransformation:
    def update(updates, state, params=None, **extra):
        g = global_norm(updates)
        # optax: where(g < max_norm, u, u / g * max_norm)
        coef = torch.where(g < max_norm, torch.ones_like(g), max_norm / g.clamp_min(1e-30))
        keys = tree_keys(updates)
        if not keys:
            return updates, state
        torch._foreach_mul_(_leaves(updates, keys), coef.to(updates[keys[0]].device) if keys else coef)
        return updates, state

    return GradientTransformation(lambda p: EmptyState(), update)


def add_decayed_weights(weight_decay: ScalarOrSchedule, mask: Optional[Dict[str, bool]] = None) -> GradientTransformation:
    """``u += wd * p`` on the leaves selected by ``mask`` (path -> bool)."""

    def update(updates, state, params=None, count: int = 0, **extra):
        if params is None:
            raise ValueError("add_decayed_weights needs params")
        wd = _value(weight_decay, count)
        if wd == 0.0:
            return updates, state
        keys = [k for k in tree_keys(updates) if (mask is None or mask.get(k, True))]
        if keys:
            ps = [params[k].to(updates[k].dtype) if params[k].dtype != updates[k].dtype else params[k] for k in keys]
            torch._foreach_add_(_leaves(updates, keys), ps, alpha=wd)
        return updates, state

    return GradientTransformation(lambda p: EmptyState(), update)


class ScaleByAdamState(NamedTuple):
    count: int
    mu: Tree
    nu: Tree


def _bias_correction(b: float, count: int) -> float:
    return 1.0 - b**count


def scale_by_adam(b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, eps_root: float = 0.0, nesterov: bool = False,
                  mu_dtype=None) -> GradientTransformation:
    def init(params):
        return ScaleByAdamState(0, tree_zeros_like(params, mu_dtype), tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        keys = tree_keys(updates)
        if not keys:
            return updates, state
        g = _leaves(updates, keys)
        mu = _leaves(state.mu, keys)
        nu = _leaves(state.nu, keys)
        torch._foreach_mul_(mu, b1)
        torch._foreach_add_(mu, g, alpha=1 - b1)
        torch._foreach_mul_(nu, b2)
        torch._foreach_addcmul_(nu, g, g, value=1 - b2)
        count = state.count + 1
        bc1, bc2 = _bias_correction(b1, count), _bias_correction(b2, count)
        if nesterov:
            mu_hat = torch._foreach_mul(mu, b1 / _bias_correction(b1, count + 1))
            torch._foreach_add_(mu_hat, g, alpha=(1 - b1) / bc1)
        else:
            mu_hat = torch._foreach_div(mu, bc1)
        denom = torch._foreach_div(nu, bc2)
        if eps_root:
            torch._foreach_add_(denom, eps_root)
        torch._foreach_sqrt_(denom)
        torch._foreach_add_(denom, eps)
        torch._foreach_div_(mu_hat, denom)
        out = dict(updates)
        for k, u in zip(keys, mu_hat):
            out[k] = u
        return out, ScaleByAdamState(count, state.mu, state.nu)

    return GradientTransformation(init, update)


class TraceState(NamedTuple):
    trace: Tree


def trace(decay: float, nesterov: bool = False) -> GradientTransformation:
    """Momentum: ``t = g + decay * t``; nesterov returns ``g + decay * t``."""

    def init(params):
        return TraceState(tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        keys = tree_keys(updates)
        if not keys:
            return updates, state
        g = _leaves(updates, keys)
        t = _leaves(state.trace, keys)
        torch._foreach_mul_(t, decay)
        torch._foreach_add_(t, g)
        if nesterov:
            outl = torch._foreach_mul(t, decay)
            torch._foreach_add_(outl, g)
        else:
            outl = [x.clone() for x in t]
        out = dict(updates)
        for k, u in zip(keys, outl):
            out[k] = u
        return out, state

    return GradientTransformation(init, update)


class EmaState(NamedTuple):
    count: int
    ema: Tree


def ema(decay: float, debias: bool = False) -> GradientTransformation:
    """``e = decay * e + (1 - decay) * g``."""

    def init(params):
        return EmaState(0, tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        keys = tree_keys(updates)
        if not keys:
            return updates, state
        e = _leaves(state.ema, keys)
        torch._foreach_mul_(e, decay)
        torch._foreach_add_(e, _leaves(updates, keys), alpha=1 - decay)
        count = state.count + 1
        outl = torch._foreach_div(e, _bias_correction(decay, count)) if debias else [x.clone() for x in e]
        out = dict(updates)
        for k, u in zip(keys, outl):
            out[k] = u
        return out, EmaState(count, state.ema)

    return GradientTransformation(init, update)


class ScaleByLionState(NamedTuple):
    count: int
    mu: Tree


def scale_by_lion(b1: float = 0.9, b2: float = 0.99) -> GradientTransformation:
    def init(params):
        return ScaleByLionState(0, tree_zeros_like(params))

    def update(updates, state, params=None, **extra):
        keys = tree_keys(updates)
        if not keys:
            return updates, state
        g = _leaves(updates, keys)
        mu = _leaves(state.mu, keys)
        direction = torch._foreach_mul(mu, b1)
        torch._foreach_add_(direction, g, alpha=1 - b1)
        direction = [torch.sign(d) for d in direction]
        torch._foreach_mul_(mu, b2)
        torch._foreach_add_(mu, g, alpha=1 - b2)
        out = dict(updates)
        for k, u in zip(keys, direction):
            out[k] = u
        return out, ScaleByLionState(state.count + 1, state.mu)

    return GradientTransformation(init, update)


class ScaleByRmsState(NamedTuple):
    nu: Tree


def scale_by_rms(decay: float = 0.9, eps: float = 1e-8, initial_scale: float = 0.0) -> GradientTransformation:
    def init(params):
        nu = tree_zeros_like(params)
        if initial_scale:
            for v in nu.values():
                if v is not None:
                    v.fill_(initial_scale)
        return ScaleByRmsState(nu)

    def update(updates, state, params=None, **extra):
        keys = tree_keys(updates)
        if not keys:
            return updates, state
        g = _leaves(updates, keys)
        nu = _leaves(state.nu, keys)
        torch._foreach_mul_(nu, decay)
        torch._foreach_addcmul_(nu, g, g, value=1 - decay)
        denom = torch._foreach_sqrt(nu)
        torch._foreach_add_(denom, eps)
        outl = torch._foreach_div(g, denom)
        out = dict(updates)
        for k, u in zip(keys, outl):
            out[k] = u
        return out, state

    return GradientTransformation(init, update)


def scale_by_sign() -> GradientTransformation:
    def update(updates, state, params=None, **extra):
        return tree_map(torch.sign, updates), state

    return GradientTransformation(lambda p: EmptyState(), update)


# ----------------------------------------------------------------------------------------------- wrappers
class InjectHyperparamsState(NamedTuple):
    count: int
    hyperparams: Dict[str, float]
    hyperparams_states: Dict[str, Any]
    inner_state: Any


def inject_hyperparams(factory: Callable[..., GradientTransformation]):
    """``inject_hyperparams(f)(learning_rate=schedule, **static)``: evaluates scheduled hyperparameters each step, rebuilds
    the inner transformation with their current values and records them in the state (so the learning rate can be
    logged as ``optim/learning_rate``, src/levanter/tracker/helpers.py:20-36)."""

    def make(**kwargs) -> GradientTransformation:
        sched = {k: v for k, v in kwargs.items() if callable(v)}
        static = {k: v for k, v in kwargs.items() if not callable(v)}
        numeric = {k: float(v) for k, v in static.items() if isinstance(v, (int, float)) and not isinstance(v, bool)}

        def current(count):
            hp = dict(numeric)
            hp.update({k: float(f(count)) for k, f in sched.items()})
            return hp

        def init(params):
            hp = current(0)
            inner = factory(**{**static, **{k: hp[k] for k in sched}})
            return InjectHyperparamsState(0, hp, {k: ScaleByScheduleState(0) for k in sched}, inner.init(params))

        def update(updates, state, params=None, **extra):
            hp = current(state.count)
            inner = factory(**{**static, **{k: hp[k] for k in sched}})
            updates, inner_state = inner.update(updates, state.inner_state, params, **extra)
            count = state.count + 1
            return updates, InjectHyperparamsState(count, hp, {k: ScaleByScheduleState(count) for k in sched}, inner_state)

        return GradientTransformation(init, update)

    return make


class MaskedState(NamedTuple):
    inner_state: Any


def masked(inner: GradientTransformation, mask: Union[Dict[str, bool], Callable[[Tree], Dict[str, bool]]]) -> GradientTransformation:
    """Apply ``inner`` only to leaves whose mask is True; other leaves pass through unchanged."""

    def _mask(tree):
        return mask(tree) if callable(mask) else mask

    def init(params):
        m = _mask(params)
        return MaskedState(inner.init({k: (v if m.get(k, False) else None) for k, v in params.items()}))

    def update(updates, state, params=None, **extra):
        m = _mask(updates)
        sub_u = {k: (v if m.get(k, False) else None) for k, v in updates.items()}
        sub_p = None if params is None else {k: (v if m.get(k, False) else None) for k, v in params.items()}
        new_u, s = inner.update(sub_u, state.inner_state, sub_p, **extra)
        out = dict(updates)
        for k, v in new_u.items():
            if v is not None:
                out[k] = v
        return out, MaskedState(s)

    return GradientTransformation(init, update)


class MultiTransformState(NamedTuple):
    inner_states: Dict[str, Any]


def multi_transform(transforms: Dict[str, GradientTransformation], labels: Union[Dict[str, str], Callable[[Tree], Dict[str, str]]]) -> GradientTransformation:
    """Route each leaf to the transformation named by its label (Muon/Scion/Adam-mini use this)."""

    def _labels(tree):
        return labels(tree) if callable(labels) else labels

    def init(params):
        lab = _labels(params)
        return MultiTransformState({name: masked(t, {k: lab.get(k) == name for k in params}).init(params)
                                    for name, t in transforms.items()})

    def update(updates, state, params=None, **extra):
        lab = _labels(updates)
        out = dict(updates)
        new_states = {}
        for name, t in transforms.items():
            m = {k: lab.get(k) == name for k in updates}
            sub_u = {k: (v if m[k] else None) for k, v in updates.items()}
            sub_p = None if params is None else {k: (v if m[k] else None) for k, v in params.items()}
            new_u, s = t.update(sub_u, state.inner_states[name].inner_state, sub_p, **extra)
            new_states[name] = MaskedState(s)
            for k, v in new_u.items():
                if v is not None:
                    out[k] = v
        return out, MultiTransformState(new_states)

    return GradientTransformation(init, update)


def apply_updates(params: Tree, updates: Tree) -> None:
    """``p += u`` in place (updates are cast to the parameter dtype)."""
    keys = [k for k in tree_keys(updates) if params.get(k) is not None]
    ps = _leaves(params, keys)
    us = [updates[k] if updates[k].dtype == params[k].dtype else updates[k].to(params[k].dtype) for k in keys]
    torch._foreach_add_(ps, us)


# ----------------------------------------------------------------------------------------------- schedules
def constant_schedule(value: float) -> Schedule:
    return lambda count: value


def linear_schedule(init_value: float, end_value: float, transition_steps: int, transition_begin: int = 0) -> Schedule:
    def f(count):
        if transition_steps <= 0:
            return end_value
        c = min(max(count - transition_begin, 0), transition_steps)
        return init_value + (end_value - init_value) * (c / transition_steps)

    return f


def cosine_decay_schedule(init_value: float, decay_steps: int, alpha: float = 0.0, exponent: float = 1.0) -> Schedule:
    def f(count):
        if decay_steps <= 0:
            return init_value * alpha if alpha else init_value
        c = min(count, decay_steps)
        cosine = 0.5 * (1 + math.cos(math.pi * c / decay_steps))
        decayed = (1 - alpha) * cosine**exponent + alpha
        return init_value * decayed

    return f


def join_schedules(schedules: Sequence[Schedule], boundaries: Sequence[int]) -> Schedule:
    def f(count):
        out = schedules[0](count)
        for b, s in zip(boundaries, schedules[1:]):
            if count >= b:
                out = s(count - b)
        return out

    return f
