"""Training state (src/levanter/trainer_state.py:43-291).

``TrainerState`` bundles the step counter, the model (compute-dtype parameters, views into the engine's flat buffer),
the sharded parameter/optimizer engine, the RNG key and the optional model average.  ``saveable_state`` is the tree the
checkpointer writes: ``step``, ``model`` (trainable parameters in param dtype), ``opt_state``, ``training_key``,
``model_averaging`` (:229-240)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional

import torch
import torch.nn as nn

from .config import Policy
from .parallel.engine import ShardedEngine


@dataclass
class TrainerState:
    step: int
    model: nn.Module
    engine: ShardedEngine
    training_key: torch.Tensor  # uint32[2]-style key material (seed, counter)
    mp: Policy
    model_averaging: Optional[Any] = None
    is_trainable: Optional[Callable[[str], bool]] = None

    @property
    def opt_state(self):
        return self.engine.optimizer_state_tree()

    @property
    def optimizer(self):
        return self.engine.opt

    @property
    def trainable_model(self) -> Dict[str, torch.Tensor]:
        return self.engine.master_tree()

    @property
    def eval_model(self) -> nn.Module:
        """The model to evaluate: the averaged weights when model averaging is on (copied into a shadow module)."""
        if self.model_averaging is None:
            return self.model
        full = self.engine._gather_leaf_tree(self.model_averaging.model_params)
        return _shadow_with(self.model, full, self.mp)

    @property
    def saveable_state(self) -> Dict[str, Any]:
        out = {
            "step": self.step,
            "model": self.engine.deferred_named(self.engine.master),
            "opt_state": self.engine.optimizer_state_tree(deferred=True),
            "training_key": self.training_key,
        }
        if self.model_averaging is not None:
            out["model_averaging"] = {"model": self.engine._deferred_leaf_tree(self.model_averaging.model_params)}
            for k in ("beta", "tot_weight"):
                if hasattr(self.model_averaging, k):
                    out["model_averaging"][k] = getattr(self.model_averaging, k)
        return out

    def next_key(self) -> int:
        """Split the training key: returns a per-step seed and advances the stored key."""
        k = self.training_key
        seed = int(k[0].item()) * 1000003 + int(k[1].item())
        self.training_key = torch.stack([k[0], k[1] + 1])
        return seed & 0x7FFFFFFF


_shadow_cache: Dict[int, nn.Module] = {}


def _shadow_with(model: nn.Module, params: Dict[str, torch.Tensor], mp: Policy) -> nn.Module:
    import copy

    key = id(model)
    shadow = _shadow_cache.get(key)
    if shadow is None:
        shadow = copy.deepcopy(model)
        for p in shadow.parameters():
            p.requires_grad_(False)
        _shadow_cache[key] = shadow
    with torch.no_grad():
        sd = dict(shadow.named_parameters())
        for k, v in params.items():
            if k in sd:
                sd[k].copy_(v.to(sd[k].dtype).view(sd[k].shape))
    return shadow


def make_training_key(seed: int) -> torch.Tensor:
    return torch.tensor([seed & 0xFFFFFFFF, 0], dtype=torch.int64)


def saveable_training_mask(state: TrainerState, is_trainable: Optional[Callable[[str], bool]] = None) -> Dict[str, Any]:
    """Which parts of a trainer state a checkpoint holds (src/levanter/trainer_state.py:229-240): the step, the RNG key, the
    optimizer state and the model average whole, and of the model only the trainable floating-point parameters (frozen
    weights come from wherever the run initialised them, e.g. the base model of a LoRA run).  Returned as a dict with a
    ``model`` entry mapping parameter names to booleans."""
    keep = is_trainable if is_trainable is not None else (state.is_trainable or (lambda name: True))
    model_mask = {name: bool(p.requires_grad and p.is_floating_point() and keep(name)) for name, p in state.model.named_parameters()}
    return {"step": True, "training_key": True, "opt_state": True, "model_averaging": state.model_averaging is not None, "model": model_mask}


def take_train_step(optimizer, params: Dict[str, torch.Tensor], opt_state, grads: Dict[str, torch.Tensor], *,
                    obj_fun: Optional[Callable] = None, loss: Optional[torch.Tensor] = None,
                    is_trainable: Optional[Callable[[str], bool]] = None):
    """One optimizer step on a name -> tensor tree, outside the sharded engine (src/levanter/trainer_state.py:243-275):
    gradients and parameters are restricted to the trainable names, the transformation sees ``obj_fn`` (Sophia's Hessian
    estimate) and ``loss`` (skip-step), and the updates are added in place.  Returns ``(params, new optimizer state, updates)``.
    The engine's own step (``ShardedEngine.step``) is the sharded form of the same call."""
    from .optim import transforms as T

    keep = is_trainable or (lambda name: True)
    train_grads = {k: g for k, g in grads.items() if g is not None and keep(k)}
    train_params = {k: params[k] for k in train_grads}
    updates, opt_state = optimizer.update(train_grads, opt_state, train_params, obj_fn=obj_fun, loss=loss)
    T.apply_updates(train_params, updates)
    return params, opt_state, updates


# ------------------------------------------------------------------------------------------------ trainable subsets
def make_floating_point_trainable_filter(model: torch.nn.Module, is_trainable: Optional[Callable[[str], bool]] = None) -> Callable[[str], bool]:
    """``name -> bool``: ``is_trainable(name)`` and the parameter is a floating-point tensor that asks for gradients
    (src/levanter/trainer_state.py:278-292; integer tables and frozen weights are never trained)."""
    keep = is_trainable or (lambda name: True)
    ok = {name for name, p in model.named_parameters() if p.is_floating_point() and p.requires_grad}
    return lambda name: name in ok and bool(keep(name))


def trainables_only(model: torch.nn.Module, is_trainable: Optional[Callable[[str], bool]] = None) -> Dict[str, torch.Tensor]:
    """The trainable parameters of ``model`` by name (:207-213): what the optimizer state is built for and what a training
    checkpoint holds."""
    f = make_floating_point_trainable_filter(model, is_trainable)
    return {name: p for name, p in model.named_parameters() if f(name)}


def init_optimizer_for_trainables(optimizer, trainable_params: Dict[str, torch.Tensor]):
    """Optimizer state for the trainable parameters only (:180-186)."""
    return optimizer.init(trainable_params)


def cast_params_by_trainability(model: torch.nn.Module, mp, is_trainable: Optional[Callable[[str], bool]] = None) -> torch.nn.Module:
    """Trainable parameters to the policy's parameter dtype, frozen floating-point ones to its compute dtype, in place
    (:216-226): a frozen base model under LoRA costs two bytes per weight, not four."""
    f = make_floating_point_trainable_filter(model, is_trainable)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.is_floating_point():
                p.data = p.data.to(mp.param_dtype if f(name) else mp.compute_dtype)
    return model
