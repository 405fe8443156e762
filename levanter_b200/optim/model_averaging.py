"""Exponential moving averages of the model (src/levanter/optim/model_averaging.py): ``ema`` (fixed beta) and
``ema_decay_sqrt`` (EMA followed by a 1-sqrt decay phase)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..config import ChoiceRegistry


@dataclass
class EmaModelAveraging:
    model: Dict[str, torch.Tensor]
    beta: float = 0.999

    def update(self, new_model: Dict[str, torch.Tensor], step: int) -> "EmaModelAveraging":
        keys = [k for k in self.model if k in new_model]
        avg = [self.model[k] for k in keys]
        new = [new_model[k].to(self.model[k].dtype) for k in keys]
        torch._foreach_mul_(avg, self.beta)
        torch._foreach_add_(avg, new, alpha=1 - self.beta)
        return self

    @property
    def model_params(self) -> Dict[str, torch.Tensor]:
        return self.model


@dataclass
class EmaDecaySqrtModelAveraging:
    """EMA until ``switch_step``; afterwards a weighted running average with weights following ``1 - sqrt(t/T)``."""

    model: Dict[str, torch.Tensor]
    beta: float
    switch_step: int
    decay_steps: int
    tot_weight: float = 0.0

    def update(self, new_model: Dict[str, torch.Tensor], step: int) -> "EmaDecaySqrtModelAveraging":
        keys = [k for k in self.model if k in new_model]
        avg = [self.model[k] for k in keys]
        new = [new_model[k].to(self.model[k].dtype) for k in keys]
        if step < self.switch_step:
            torch._foreach_mul_(avg, self.beta)
            torch._foreach_add_(avg, new, alpha=1 - self.beta)
            self.tot_weight = 1.0
        else:
            t = step - self.switch_step
            frac = min(max(t / max(self.decay_steps, 1), 0.0), 1.0)
            w = 1.0 - math.sqrt(frac)
            if w > 0:
                tot = self.tot_weight + w
                torch._foreach_mul_(avg, self.tot_weight / tot)
                torch._foreach_add_(avg, new, alpha=w / tot)
                self.tot_weight = tot
        return self

    @property
    def model_params(self) -> Dict[str, torch.Tensor]:
        return self.model


@dataclass(frozen=True)
class ModelAveragingConfig(ChoiceRegistry):
    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return "ema"

    def create(self, model_params: Dict[str, torch.Tensor]):
        raise NotImplementedError


@ModelAveragingConfig.register_subclass("ema")
@dataclass(frozen=True)
class EmaModelAveragingConfig(ModelAveragingConfig):
    beta: float = 0.999

    def create(self, model_params):
        return EmaModelAveraging({k: v.detach().clone().float() for k, v in model_params.items()}, self.beta)


@ModelAveragingConfig.register_subclass("ema_decay_sqrt")
@dataclass(frozen=True)
class EmaDecaySqrtConfig(ModelAveragingConfig):
    beta: float = 0.999
    switch_step: int = 10000
    decay_steps: int = 10000

    def create(self, model_params):
        return EmaDecaySqrtModelAveraging({k: v.detach().clone().float() for k, v in model_params.items()}, self.beta,
                                          self.switch_step, self.decay_steps)
