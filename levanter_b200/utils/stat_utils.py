"""Streaming statistics (src/levanter/utils/stat_utils.py:16-34)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Union

import torch

Arrayish = Union[float, torch.Tensor]


@dataclass
class RunningMean:
    """Weighted running mean that is safe to merge when the total weight is zero."""

    mean: Arrayish = 0.0
    total: Arrayish = 0.0

    @staticmethod
    def zeros_like(x) -> "RunningMean":
        z = torch.zeros_like(x) if isinstance(x, torch.Tensor) else 0.0
        return RunningMean(z, z if not isinstance(z, torch.Tensor) else z.clone())

    def add(self, x: Arrayish, total: Arrayish) -> "RunningMean":
        new_total = self.total + total
        if isinstance(new_total, torch.Tensor):
            ratio = torch.where(new_total != 0, total / torch.where(new_total != 0, new_total, torch.ones_like(new_total)), torch.zeros_like(new_total))
        else:
            ratio = total / new_total if new_total else 0.0
        new_mean = self.mean + (x - self.mean) * ratio
        return RunningMean(new_mean, new_total)

    def __add__(self, other: "RunningMean") -> "RunningMean":
        return self.add(other.mean, other.total)
