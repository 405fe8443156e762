"""Hook protocol of the trainer (src/levanter/callbacks/_core.py:20-98)."""
from __future__ import annotations

import abc
from dataclasses import dataclass
from typing import Any, Callable, Generic, Optional, TypeVar

import torch

S = TypeVar("S")
M = TypeVar("M")


@dataclass
class StepInfo(Generic[S]):
    """What a hook sees after a step.  ``step`` is the step just *completed* (``state.step - 1``,
    src/levanter/callbacks/_core.py:37): checkpoints are named after it."""

    state: S
    loss: float
    step_duration: float

    @property
    def model(self):
        return self.state.model

    @property
    def opt_state(self):
        return self.state.opt_state

    @property
    def eval_model(self):
        return self.state.eval_model

    @property
    def step(self) -> int:
        return int(self.state.step) - 1

    @property
    def next_step(self) -> int:
        return int(self.state.step)


class Callback(abc.ABC, Generic[S]):
    @abc.abstractmethod
    def on_step(self, info: StepInfo[S], force: bool = False):
        ...


class LambdaCallback(Callback[S]):
    def __init__(self, fn: Callable[[StepInfo[S]], Any]):
        self.fn = fn
        # functions that declare a ``force`` parameter (checkpointing, the eval harness) are told about forced runs
        try:
            import inspect

            self._takes_force = "force" in inspect.signature(fn).parameters
        except (TypeError, ValueError):
            self._takes_force = False

    def on_step(self, info: StepInfo[S], force: bool = False):
        if self._takes_force:
            self.fn(info, force=force)
        else:
            self.fn(info)


class JitCallback(abc.ABC, Generic[S, M]):
    """A hook with a device part and a host part.  ``inside_step`` runs right after the optimizer update with access to
    gradients and updates (the reference runs it inside the compiled step under ``lax.cond``); ``on_step`` receives
    its result on the host."""

    @abc.abstractmethod
    def inside_step(self, state: S, grads: Any) -> M:
        ...

    # True: the engine keeps the step's parameter change (``engine.last_updates``) and ``after_update`` is called with it
    wants_updates = False

    def after_update(self, state: S, engine: Any, cb_info: M) -> M:
        """Called after the optimizer step of a step for which ``inside_step`` ran; returns the (extended) result."""
        return cb_info

    @abc.abstractmethod
    def on_step(self, step_info: StepInfo[S], cb_info: M):
        ...
