"""Optimizer configs, learning-rate schedules and the weight-decay mask (src/levanter/optim/config.py).

``OptimizerConfig`` is a plugin registry keyed by ``optimizer.type`` (default ``adam``).  ``build(num_train_steps)``
returns a :class:`GradientTransformation`.  The learning-rate schedule is per-cycle ``[linear warmup -> stable ->
decay]`` joined over cycles, exactly as the reference composes it (:239-326), with ``warmup``/``decay``/``rewarmup``
given as fractions or step counts (:386-393).
"""
from __future__ import annotations

import abc
import math
import re
import warnings
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Union

import numpy as np
import torch

from ..config import ChoiceRegistry
from . import transforms as T
from .clip_update_norm import ClipUpdateNormConfig
from .skipstep import SkipStepConfig
from .transforms import GradientTransformation


# ----------------------------------------------------------------------------------------------- schedules
@dataclass
class LrScheduleContext:
    warmup_steps: int
    decay_steps: int
    learning_rate: float
    min_lr_ratio: float
    min_lr: float


@dataclass(frozen=True)
class LrSchedule(ChoiceRegistry):
    def build(self, ctx: LrScheduleContext) -> Callable[[int], float]:
        raise NotImplementedError


@LrSchedule.register_subclass("constant")
@dataclass(frozen=True)
class ConstantLrSchedule(LrSchedule):
    def build(self, ctx):
        return T.constant_schedule(ctx.learning_rate)


@LrSchedule.register_subclass("cosine")
@dataclass(frozen=True)
class CosineLrSchedule(LrSchedule):
    exponent: float = 1.0

    def build(self, ctx):
        return T.cosine_decay_schedule(ctx.learning_rate, ctx.decay_steps, ctx.min_lr_ratio, self.exponent)


@LrSchedule.register_subclass("linear")
@dataclass(frozen=True)
class LinearLrSchedule(LrSchedule):
    def build(self, ctx):
        return T.linear_schedule(ctx.learning_rate, ctx.min_lr, ctx.decay_steps)


@LrSchedule.register_subclass("inv_sqrt")
@dataclass(frozen=True)
class InvSqrtLrSchedule(LrSchedule):
    timescale: float = 10000

    def build(self, ctx):
        return _inv_sqrt_decay_schedule(ctx.learning_rate, ctx.min_lr, ctx.warmup_steps, self.timescale)


@LrSchedule.register_subclass("inv")
@dataclass(frozen=True)
class InvLrSchedule(LrSchedule):
    def build(self, ctx):
        return _inv_decay_schedule(ctx.learning_rate, ctx.min_lr, ctx.decay_steps)


@LrSchedule.register_subclass("power")
@dataclass(frozen=True)
class PowerLrSchedule(LrSchedule):
    """Power scheduler (Shen et al. 2024): ``min(lr, batch_size * a * tokens^b)``."""

    batch_size: int = 1
    seq_length: int = 1
    a: float = 4.6
    b: float = -0.51

    def __post_init__(self):
        if self.a <= 0 or self.b >= 0:
            raise ValueError("Power schedule expects a > 0 and b < 0")

    def build(self, ctx):
        def schedule(step):
            tokens = step * self.batch_size * self.seq_length
            if tokens <= 0:
                return ctx.learning_rate
            return min(ctx.learning_rate, self.batch_size * self.a * tokens**self.b)

        return schedule


def _inv_sqrt_decay_schedule(lr: float, min_lr: float, warmup_steps: int, timescale: float = 10000):
    def schedule(count):
        decay = min(1.0, 1.0 / math.sqrt(max(count + warmup_steps, 1) / timescale))
        return max(lr * decay, min_lr)

    return schedule


def _inv_decay_schedule(lr: float, min_lr: float, decay_steps: int):
    def schedule(count):
        decay = min(1.0, 1.0 / ((lr / min_lr - 1) * max(count, 1) / decay_steps + 1))
        return max(lr * decay, min_lr)

    return schedule


def _convert_frac_or_steps(frac_or_steps, num_train_steps: int) -> int:
    if frac_or_steps < 0.0 or (frac_or_steps > 1.0 and frac_or_steps % 1 != 0):
        raise ValueError(f"Invalid fraction {frac_or_steps}. Must be between 0 and 1. You can also use (whole) steps.")
    if frac_or_steps <= 1.0:
        return int(frac_or_steps * num_train_steps)
    return int(frac_or_steps)


# ----------------------------------------------------------------------------------------------- parameter info
def levanter_path(torch_name: str) -> str:
    """Torch parameter name -> the reference's key path (``layers.<i>.`` becomes ``layers.stacked.``)."""
    return re.sub(r"\.(layers|blocks|h)\.\d+\.", r".\1.stacked.", "." + torch_name)[1:]


class ParamInfo:
    """Per-parameter metadata the optimizers need: owner-class path (for the default weight-decay mask), shape and role."""

    def __init__(self, model: Optional[torch.nn.Module] = None):
        self.class_paths: Dict[str, str] = {}
        self.shapes: Dict[str, tuple] = {}
        self.module_types: Dict[str, str] = {}
        self.lev_shapes: Dict[str, tuple] = {}
        if model is not None:
            for mod_name, mod in model.named_modules():
                for pname, p in mod.named_parameters(recurse=False):
                    full = f"{mod_name}.{pname}" if mod_name else pname
                    self.class_paths[full] = f"{type(mod).__name__}.{pname}"
                    self.shapes[full] = tuple(p.shape)
                    self.module_types[full] = type(mod).__name__
                    if hasattr(p, "lev_shape"):
                        self.lev_shapes[full] = tuple(p.lev_shape)

    def class_path(self, name: str) -> Optional[str]:
        return self.class_paths.get(name)

    def is_linear_weight(self, name: str) -> bool:
        return self.module_types.get(name) in ("Linear", "LoraLinear", "LowRankLinear") and name.endswith("weight")


def _heuristic_class_path(path: str) -> str:
    leaf = path.rsplit(".", 1)[-1]
    low = path.lower()
    if re.search(r"(^|[._])(ln|norm|layernorm|layer_norm)[._0-9a-z]*\.(weight|bias)$", low) or "layernorm" in low or "_norm." in low or ".norm." in low:
        return f"RmsNorm.{leaf}"
    if "embeddings" in low or "wte" in low or "wpe" in low:
        return f"Embedding.{leaf}"
    return f"Linear.{leaf}"


# ----------------------------------------------------------------------------------------------- base config
@dataclass(frozen=True)
class OptimizerConfig(ChoiceRegistry):
    learning_rate: float = 6e-4
    weight_decay: float = 0.1
    min_lr_ratio: float = 0.1
    warmup: Union[int, float] = 0.01
    decay: Union[int, float, None] = None
    rewarmup: Union[int, float] = 0.0
    cooldown: Optional[float] = None
    cycle_length: Union[int, float, None, List[int]] = None
    cycles: Union[int, List[int], None] = None
    lr_schedule: Union[LrSchedule, str] = "cosine"
    haps: Optional[List[int]] = None
    weight_decay_modules: Union[List[str], str, None] = None
    default_weight_decay_mask: Optional[bool] = None

    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return "adam"

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        raise NotImplementedError

    # -- weight decay mask (src/levanter/optim/config.py:148-237) ---------------------------------------------
    def build_weight_decay_mask(self, param_info: Optional[ParamInfo] = None):
        """Returns ``mask_fn(params_tree) -> {path: bool}`` or None (decay everything)."""

        def reasonable_default(path: str):
            if "LayerNorm" in path or "RMSNorm" in path or "RmsNorm" in path or "Embedding" in path:
                return False
            if path.endswith("bias"):
                return False
            return None

        if self.weight_decay_modules is None and self.default_weight_decay_mask is False:
            return None
        use_default = self.default_weight_decay_mask is True or (
            self.default_weight_decay_mask is None and self.weight_decay_modules is None)
        regex = re.compile(self.weight_decay_modules) if isinstance(self.weight_decay_modules, str) else None

        def decide(name: str) -> bool:
            root = levanter_path(name)
            cls_path = (param_info.class_path(name) if param_info is not None else None) or _heuristic_class_path(name)
            should = None
            for kp in (root, cls_path):
                if kp is None:
                    continue
                if regex is not None:
                    should = should or (regex.match(kp) is not None)
                elif isinstance(self.weight_decay_modules, list):
                    should = should or any(t in kp for t in self.weight_decay_modules)
                if use_default and not should:
                    should = reasonable_default(kp)
                if should:
                    break
            if should is None:
                should = bool(use_default)
            return bool(should)

        def mask_fn(params) -> Dict[str, bool]:
            mask = {k: decide(k) for k in params}
            try:
                from .. import tracker

                tracker.log_hyperparameters({"decayed_weights": sorted(levanter_path(k) for k, v in mask.items() if v)})
            except Exception:
                pass
            return mask

        return mask_fn

    # -- learning-rate schedule (src/levanter/optim/config.py:239-326) -----------------------------------------
    def lr_scheduler(self, num_train_steps: int, override_lr: Optional[float] = None) -> Callable[[int], float]:
        if self.cooldown is not None:
            warnings.warn("cooldown is deprecated. Just use the normal schedule.", DeprecationWarning)
            cooldown_steps = _convert_frac_or_steps(self.cooldown, num_train_steps)
        else:
            cooldown_steps = 0
        total_main_steps = num_train_steps - cooldown_steps
        points = self._get_cycle_minima(total_main_steps)
        learning_rate = self.learning_rate if override_lr is None else override_lr
        min_lr = learning_rate * self.min_lr_ratio
        schedules, boundaries = [], []
        previous_end = 0.0
        schedule = None
        lr_decay_steps = 0
        for cycle, (start, end) in enumerate(zip(points[:-1], points[1:])):
            cycle_steps = end - start
            warmup_steps = _convert_frac_or_steps(self.warmup if cycle == 0 else self.rewarmup, cycle_steps)
            if warmup_steps != 0:
                schedules.append(T.linear_schedule(previous_end, learning_rate, warmup_steps))
                boundaries.append(start + warmup_steps)
            lr_decay_steps = (_convert_frac_or_steps(self.decay, cycle_steps) if self.decay is not None
                              else cycle_steps - warmup_steps)
            stable_steps = cycle_steps - warmup_steps - lr_decay_steps
            if stable_steps != 0:
                schedules.append(T.constant_schedule(learning_rate))
                boundaries.append(start + warmup_steps + stable_steps)
            if isinstance(self.lr_schedule, str):
                name = self.lr_schedule
                if name == "constant":
                    schedule = T.constant_schedule(learning_rate)
                elif name == "cosine":
                    schedule = T.cosine_decay_schedule(learning_rate, lr_decay_steps, self.min_lr_ratio)
                elif name == "linear":
                    schedule = T.linear_schedule(learning_rate, min_lr, lr_decay_steps)
                elif name == "inv_sqrt":
                    schedule = _inv_sqrt_decay_schedule(learning_rate, min_lr, warmup_steps, 10000)
                elif name == "inv":
                    schedule = _inv_decay_schedule(learning_rate, min_lr, lr_decay_steps)
                else:
                    raise ValueError(f"Unknown lr_schedule: {self.lr_schedule}")
            elif isinstance(self.lr_schedule, LrSchedule):
                schedule = self.lr_schedule.build(LrScheduleContext(warmup_steps, lr_decay_steps, learning_rate,
                                                                    self.min_lr_ratio, min_lr))
            else:
                raise ValueError(f"lr_schedule must be a string or an LrSchedule, got {self.lr_schedule}")
            previous_end = schedule(lr_decay_steps)
            schedules.append(schedule)
            boundaries.append(end)
        if cooldown_steps != 0:
            final_main_lr = schedule(lr_decay_steps)
            schedules.append(T.linear_schedule(final_main_lr, min_lr, cooldown_steps))
        if len(schedules) > 1:
            return T.join_schedules(schedules, boundaries)
        return schedules[0]

    def _get_cycle_minima(self, total_main_steps: int) -> List[int]:
        if self.cycle_length is not None:
            if self.cycles is not None:
                raise ValueError("Can't use both cycle_length and cycles.")
            if self.haps is not None:
                raise ValueError("Can't use both cycle_length and haps.")
            if isinstance(self.cycle_length, (int, float)):
                cl = _convert_frac_or_steps(self.cycle_length, total_main_steps)
                points = [i * cl for i in range(1, total_main_steps // cl)] if cl > 0 else []
                if cl > 0 and total_main_steps % cl != 0:
                    warnings.warn("Cycle length does not divide total number of steps. The last cycle will be shorter.")
            elif isinstance(self.cycle_length, list):
                steps = np.cumsum(np.array(self.cycle_length))
                if steps[-1] > total_main_steps:
                    raise ValueError(f"Cycle lengths exceed total number of steps: {steps[-1]} > {total_main_steps}")
                points = [int(s) for s in steps.tolist()]
            else:
                raise ValueError("Invalid cycle_length. Must be a fraction, number of steps, or a list of steps.")
        elif self.haps is not None:
            warnings.warn("haps is deprecated. Use cycles instead.", DeprecationWarning)
            points = list(self.haps)
        elif isinstance(self.cycles, int):
            points = [int(total_main_steps / self.cycles * (i + 1)) for i in range(self.cycles - 1)]
        elif isinstance(self.cycles, list):
            points = list(self.cycles)
        else:
            points = []
        points.insert(0, 0)
        if points[-1] != total_main_steps:
            points.append(total_main_steps)
        return points


@dataclass(frozen=True)
class HessianOptConfig(OptimizerConfig):
    update_interval: int = 10
    """How often to update the hessian approximation."""


# ----------------------------------------------------------------------------------------------- Adam / Lion
@OptimizerConfig.register_subclass("adam")
@dataclass(frozen=True)
class AdamConfig(OptimizerConfig):
    """AdamW: ``clip_by_global_norm -> scale_by_adam -> add_decayed_weights -> [update clipping] -> scale(-lr)``
    (src/levanter/optim/config.py:402-494)."""

    beta1: float = 0.9
    beta2: float = 0.95
    epsilon: float = 1e-8
    max_grad_norm: Optional[float] = 1.0
    nesterov: bool = False
    update_rms_clipping: Optional[float] = None
    clip_update_norm: Optional[ClipUpdateNormConfig] = None
    skip_bad_steps: Union[bool, int, SkipStepConfig] = False
    adamc_weight_decay: bool = False

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        from .clip_update_norm import ClipUpdateNormConfig
        from .skipstep import SkipStepConfig
        from .util import scale_by_update_rms_clipping

        mask_fn = self.build_weight_decay_mask(param_info)
        max_lr = self.learning_rate
        mask_cache: Dict[str, Dict[str, bool]] = {}

        def _optimizer(learning_rate):
            comps = []
            if self.max_grad_norm:
                comps.append(T.clip_by_global_norm(self.max_grad_norm))
            comps.append(T.scale_by_adam(self.beta1, self.beta2, self.epsilon, nesterov=self.nesterov))
            if self.weight_decay > 0:
                wd = self.weight_decay * (learning_rate / max_lr) if (self.adamc_weight_decay and max_lr > 0) else self.weight_decay
                comps.append(_decay(wd, mask_fn, mask_cache))
            if self.update_rms_clipping is not None:
                comps.append(scale_by_update_rms_clipping(self.update_rms_clipping))
            if self.clip_update_norm is not None:
                comps.append(self.clip_update_norm.build())
            comps.append(T.scale(-learning_rate))
            opt = T.chain(*comps)
            if self.skip_bad_steps:
                opt = SkipStepConfig.from_bool_int_or_config(self.skip_bad_steps).wrap(opt)
            return opt

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps))

    # hooks for the fused sharded-AdamW kernel path
    def fused_kernel_eligible(self) -> bool:
        return (self.update_rms_clipping is None and self.clip_update_norm is None and not self.skip_bad_steps
                and not self.adamc_weight_decay)


def _decay(weight_decay: float, mask_fn, holder: Optional[Dict[str, Dict[str, bool]]] = None) -> GradientTransformation:
    """``add_decayed_weights`` whose mask is resolved once from the parameter tree (``holder`` caches it across the
    per-step rebuilds done by ``inject_hyperparams``)."""
    holder = {} if holder is None else holder

    def init(params):
        if "mask" not in holder:
            holder["mask"] = mask_fn(params) if mask_fn is not None else {k: True for k in params}
        return T.EmptyState()

    def update(updates, state, params=None, **extra):
        if "mask" not in holder:
            holder["mask"] = mask_fn(updates) if mask_fn is not None else {k: True for k in updates}
        return T.add_decayed_weights(weight_decay, holder["mask"]).update(updates, state, params, **extra)

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("lion")
@dataclass(frozen=True)
class LionConfig(OptimizerConfig):
    """Lion (src/levanter/optim/config.py:497-535): sign of interpolated momentum, decoupled weight decay."""

    beta1: float = 0.9
    beta2: float = 0.99
    max_grad_norm: Optional[float] = 1.0

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        mask_cache: Dict[str, Dict[str, bool]] = {}

        def _optimizer(learning_rate):
            comps = []
            if self.max_grad_norm:
                comps.append(T.clip_by_global_norm(self.max_grad_norm))
            comps.append(T.scale_by_lion(self.beta1, self.beta2))
            if self.weight_decay > 0:
                comps.append(_decay(self.weight_decay, mask_fn, mask_cache))
            comps.append(T.scale(-learning_rate))
            return T.chain(*comps)

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
