"""Shape specifications for batches and caches (src/levanter/shapes.py)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Sequence, Tuple, Union

import numpy as np
import torch


@dataclass(frozen=True)
class ShapeSpec:
    shape: Optional[Tuple[Optional[int], ...]]
    dtype: Any


@dataclass(frozen=True)
class NamedShapeSpec:
    """A shape whose dimensions carry names, e.g. ``(("batch", 8), ("position", 4096))``."""

    shape: Optional[Tuple[Tuple[str, Optional[int]], ...]]
    dtype: Any

    @property
    def names(self) -> Tuple[str, ...]:
        return tuple(n for n, _ in (self.shape or ()))


def to_raw_shape(spec: Union[ShapeSpec, NamedShapeSpec]) -> Optional[Tuple[Optional[int], ...]]:
    if spec.shape is None:
        return None
    if isinstance(spec, NamedShapeSpec):
        return tuple(s for _, s in spec.shape)
    return tuple(spec.shape)


def shape_spec_of(x) -> ShapeSpec:
    if isinstance(x, torch.Tensor):
        return ShapeSpec(tuple(x.shape), x.dtype)
    a = np.asarray(x)
    return ShapeSpec(tuple(a.shape), a.dtype)


def conforms(spec: Union[ShapeSpec, NamedShapeSpec], x) -> bool:
    raw = to_raw_shape(spec)
    shape = tuple(x.shape) if hasattr(x, "shape") else tuple(np.asarray(x).shape)
    if raw is None:
        return True
    if len(raw) != len(shape):
        return False
    return all(r is None or r == s for r, s in zip(raw, shape))
