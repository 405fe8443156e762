"""Batch processors: the unit of work of the cache builder (src/levanter/data/_preprocessor.py:24-69, 160-220)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Callable, Dict, Generic, List, Mapping, Optional, Sequence, TypeVar, Union

import numpy as np

T = TypeVar("T")
U = TypeVar("U")


class BatchProcessor(Generic[T, U], ABC):
    """Maps a batch of raw rows to a batch of processed rows (list of dicts, or a dict of columns).  ``metadata`` goes into
    the cache ledger so a cache built with different settings is detected; ``output_exemplar`` fixes the leaf dtypes."""

    @abstractmethod
    def __call__(self, batch: Sequence[T]) -> Union[Sequence[U], Mapping[str, Sequence]]:
        raise NotImplementedError

    @property
    @abstractmethod
    def output_exemplar(self):
        raise NotImplementedError

    @property
    def resources(self) -> Dict[str, float]:
        return {}

    @property
    @abstractmethod
    def num_cpus(self) -> float:
        raise NotImplementedError

    @property
    def num_gpus(self) -> int:
        return 0

    @property
    @abstractmethod
    def metadata(self) -> Dict[str, Any]:
        raise NotImplementedError

    @property
    def batch_size(self) -> int:
        return 128


def _to_list_of_dicts(batch: Mapping[str, Sequence]) -> List[dict]:
    keys = list(batch.keys())
    if not keys:
        return []
    n = len(batch[keys[0]])
    return [{k: batch[k][i] for k in keys} for i in range(n)]


def _canonicalize_batch(batch) -> List[dict]:
    """Row-major view of a processor result (accepts dict-of-columns, ``BatchEncoding`` or list-of-dicts)."""
    if isinstance(batch, (list, tuple)):
        return list(batch)
    if hasattr(batch, "keys"):
        return _to_list_of_dicts(batch)
    return list(batch)


def dict_from_record_batch(b) -> dict:
    """pyarrow RecordBatch -> dict of python/numpy columns."""
    out = {}
    for name in b.schema.names:
        col = b.column(name)
        try:
            out[name] = col.to_numpy(zero_copy_only=False)
        except Exception:
            out[name] = col.to_pylist()
    return out


class IdentityProcessor(BatchProcessor[T, T]):
    def __init__(self, exemplar):
        self._exemplar = exemplar

    def __call__(self, batch):
        return batch

    @property
    def output_exemplar(self):
        return self._exemplar

    @property
    def num_cpus(self) -> float:
        return 0

    @property
    def metadata(self) -> Dict[str, Any]:
        return {}


class _MapTransform:
    def __init__(self, fn):
        self.fn = fn


class _BatchMapTransform:
    def __init__(self, fn, batch_size, num_cpus=1, num_gpus=0, resources=None, output_exemplar=None):
        self.fn, self.batch_size, self.num_cpus, self.num_gpus = fn, batch_size, num_cpus, num_gpus
        self.resources = resources or {}
        self.output_exemplar = output_exemplar


class _CompositeBatchProcessor(BatchProcessor):
    """Chain of per-row and per-batch transforms collapsed into one processor, so a mapped source can be cached in one pass."""

    def __init__(self, transforms, num_cpus=1, num_gpus=0, resources=None):
        self.transforms = list(transforms)
        self._num_cpus, self._num_gpus, self._resources = num_cpus, num_gpus, resources or {}
        bs = [t.batch_size for t in self.transforms if isinstance(t, _BatchMapTransform)]
        self._batch_size = max(bs) if bs else 1024

    @property
    def batch_size(self):
        return self._batch_size

    @property
    def num_cpus(self):
        return self._num_cpus

    @property
    def num_gpus(self):
        return self._num_gpus

    @property
    def resources(self):
        return self._resources

    @property
    def output_exemplar(self):
        for t in reversed(self.transforms):
            if isinstance(t, _BatchMapTransform) and t.output_exemplar is not None:
                return t.output_exemplar
        raise ValueError("no transform in the chain declares an output exemplar")

    def __call__(self, batch):
        rows = list(batch)
        for t in self.transforms:
            if isinstance(t, _MapTransform):
                rows = [t.fn(r) for r in rows]
            else:
                rows = _canonicalize_batch(t.fn(rows))
        return rows

    @property
    def metadata(self):
        return {}
