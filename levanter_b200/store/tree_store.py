"""A tree (nested dict/list/tuple) of jagged array stores with one row per example (src/levanter/store/tree_store.py:41-180):
every leaf of the example structure is its own :class:`JaggedArrayStore` at ``path/<key path>``."""
from __future__ import annotations

from typing import Any, Callable, Dict, Generic, List, Sequence, Tuple, TypeVar

import numpy as np

from .jagged_array import JaggedArrayStore, PreparedBatch

T = TypeVar("T")


def heuristic_is_leaf(x) -> bool:
    return isinstance(x, (np.ndarray, int, float, np.generic)) or (isinstance(x, list) and (len(x) == 0 or not isinstance(x[0], (dict, list, tuple, np.ndarray))))


def _flatten(tree, prefix=()) -> List[Tuple[Tuple[str, ...], Any]]:
    if isinstance(tree, dict):
        out = []
        for k in sorted(tree.keys()):
            out.extend(_flatten(tree[k], prefix + (str(k),)))
        return out
    if isinstance(tree, tuple) or (isinstance(tree, list) and not heuristic_is_leaf(tree)):
        out = []
        for i, v in enumerate(tree):
            out.extend(_flatten(v, prefix + (str(i),)))
        return out
    return [(prefix, tree)]


def _unflatten(exemplar, leaves: Dict[Tuple[str, ...], Any], prefix=()):
    if isinstance(exemplar, dict):
        return {k: _unflatten(exemplar[k], leaves, prefix + (str(k),)) for k in exemplar}
    if isinstance(exemplar, tuple) or (isinstance(exemplar, list) and not heuristic_is_leaf(exemplar)):
        vals = [_unflatten(v, leaves, prefix + (str(i),)) for i, v in enumerate(exemplar)]
        return type(exemplar)(vals) if not hasattr(exemplar, "_fields") else type(exemplar)(*vals)
    return leaves[prefix]


class TreeBatchPreparer(Generic[T]):
    """Turns a list of examples into one :class:`PreparedBatch` per leaf (done in worker threads, off the writer)."""

    def __init__(self, exemplar: T):
        self.exemplar = exemplar
        self._leaves = [(p, np.asarray(v)) for p, v in _flatten(exemplar)]

    def __call__(self, batch: List[T]) -> Dict[Tuple[str, ...], PreparedBatch]:
        cols: Dict[Tuple[str, ...], list] = {p: [] for p, _ in self._leaves}
        for ex in batch:
            for p, v in _flatten(ex):
                cols[p].append(np.atleast_1d(np.asarray(v)))
        return {p: PreparedBatch.from_batch(cols[p], max(ex.ndim, 1)).astype(ex.dtype) for p, ex in self._leaves}


class TreeStore(Generic[T]):
    def __init__(self, tree: Dict[Tuple[str, ...], JaggedArrayStore], exemplar: T, path: str, mode: str):
        self.path, self.mode, self.tree, self.exemplar = path, mode, tree, exemplar

    @property
    def batch_preparer(self) -> TreeBatchPreparer:
        return TreeBatchPreparer(self.exemplar)

    @staticmethod
    def open(exemplar: T, path: str, *, mode: str = "a", cache_metadata: bool = False) -> "TreeStore":
        tree = {}
        for p, v in _flatten(exemplar):
            v = np.asarray(v)
            sub = "/".join([path.rstrip("/")] + list(p)) if p else path
            tree[p] = JaggedArrayStore.open(sub, mode=mode, item_rank=max(v.ndim, 1), dtype=v.dtype, cache_metadata=cache_metadata)
        return TreeStore(tree, exemplar, path, mode)

    def append(self, ex: T) -> None:
        self.extend([ex])

    def extend(self, batch: Sequence[T]) -> None:
        self.extend_with_batch(self.batch_preparer(list(batch)))

    def extend_with_batch(self, batch) -> None:
        """``batch``: {leaf path: PreparedBatch} from :class:`TreeBatchPreparer`."""
        for p, store in self.tree.items():
            store.extend(batch[p])

    async def extend_with_batch_async(self, batch) -> None:
        self.extend_with_batch(batch)

    def trim_to_size(self, size: int) -> None:
        for store in self.tree.values():
            store.trim_to_size(size)

    async def trim_to_size_async(self, size: int) -> None:
        self.trim_to_size(size)

    def reload(self) -> "TreeStore":
        return TreeStore({p: s.reload() for p, s in self.tree.items()}, self.exemplar, self.path, self.mode)

    def __len__(self) -> int:
        first = next(iter(self.tree.values()), None)
        return 0 if first is None else len(first)

    async def async_len(self) -> int:
        return len(self)

    def get_batch_sync(self, indices) -> List[T]:
        indices = list(indices)
        cols = {p: s.get_batch_sync(indices) for p, s in self.tree.items()}
        return [_unflatten(self.exemplar, {p: c[i] for p, c in cols.items()}) for i in range(len(indices))]

    async def get_batch(self, indices) -> List[T]:
        return self.get_batch_sync(indices)

    def __getitem__(self, item):
        if isinstance(item, slice):
            return self.get_batch_sync(range(*item.indices(len(self))))
        if item < 0:
            item += len(self)
        return self.get_batch_sync([item])[0]

    def __iter__(self):
        n = len(self)
        for s in range(0, n, 256):
            yield from self.get_batch_sync(range(s, min(n, s + 256)))
