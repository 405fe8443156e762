"""Protocol types used in public signatures (src/levanter/utils/types.py:26-57)."""
from __future__ import annotations

from typing import Any, Callable, Protocol, Tuple, TypeVar, Union

import torch

M = TypeVar("M")
X = TypeVar("X")
FilterSpec = Union[bool, Callable[[Any], bool]]


class ValAndGradFn(Protocol[M, X]):
    def __call__(self, model: M, *inputs: X, **kwargs) -> Tuple[torch.Tensor, Any]: ...


class ValFn(Protocol[M, X]):
    def __call__(self, model: M, *inputs: X, **kwargs) -> torch.Tensor: ...


class ComputeLossFunction(Protocol[M, X]):
    """``loss_fn(model, batch, **kw) -> scalar`` (optionally per-position when ``reduction=None``)."""

    def __call__(self, model: M, *inputs: X, **kwargs) -> torch.Tensor: ...
