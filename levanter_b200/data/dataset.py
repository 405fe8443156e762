"""Dataset abstractions and combinators (src/levanter/data/dataset.py:48-588).

``AsyncDataset`` is the contract the loader consumes: random access by index (``get_batch``), a length that may still be
growing while a cache is being built (``current_len`` / ``wait_until_len_at_least`` / ``final_length_is_known``) and
index-remapping combinators (``map``, ``slice_dataset``, ``take``, ``shuffle``, ``era_shuffle``)."""
from __future__ import annotations

import abc
import asyncio
import logging
from typing import Any, Callable, Generic, List, Optional, Sequence, TypeVar

import numpy as np

from ..utils.thread_utils import blocking_wait

logger = logging.getLogger(__name__)
T = TypeVar("T")
T_co = TypeVar("T_co", covariant=True)
U = TypeVar("U")


class DatasetBase(abc.ABC, Generic[T_co]):
    @abc.abstractmethod
    def as_async_dataset(self) -> "AsyncDataset[T_co]":
        ...

    @abc.abstractmethod
    def as_sync_dataset(self) -> "SyncDataset[T_co]":
        ...


class AsyncDataset(DatasetBase[T_co]):
    def __init__(self):
        self._min_known_len = 0

    @abc.abstractmethod
    async def async_len(self) -> int:
        ...

    @abc.abstractmethod
    async def final_length_is_known(self) -> bool:
        ...

    @abc.abstractmethod
    def is_finite(self) -> bool:
        ...

    @abc.abstractmethod
    async def current_len(self) -> Optional[int]:
        ...

    async def getitem_async(self, index: int) -> T_co:
        return (await self.get_batch([index]))[0]

    @abc.abstractmethod
    async def get_batch(self, indices: Sequence[int]) -> Sequence[T_co]:
        ...

    async def wait_until_len_at_least(self, length: int) -> int:
        if length <= self._min_known_len:
            return self._min_known_len
        res = await naive_busy_wait_until_len_at_least(self, length)
        self._min_known_len = max(self._min_known_len, res)
        return res

    def as_sync_dataset(self) -> "SyncDataset[T_co]":
        return SyncifiedDataset(self)

    def as_async_dataset(self) -> "AsyncDataset[T_co]":
        return self

    def map(self, fn: Callable[..., U], *extra_args, **extra_kwargs) -> "MappedAsyncDataset":
        return MappedAsyncDataset(self, fn, *extra_args, **extra_kwargs)

    def map_batches(self, fn: Callable[..., Sequence[U]], *extra_args, **extra_kwargs) -> "BatchMappedAsyncDataset":
        return BatchMappedAsyncDataset(self, fn, *extra_args, **extra_kwargs)

    def slice_dataset(self, start_index: Optional[int] = None, end_index: Optional[int] = None) -> "SlicedAsyncDataset":
        return SlicedAsyncDataset(self, start_index, end_index)

    def take(self, n: int):
        return self.slice_dataset(end_index=n)

    def shuffle(self, key, *, perm_type: str = "feistel"):
        from . import permutation

        return permutation.PermutationDataset(self, key, perm_type=perm_type)

    def era_shuffle(self, era_length: int, key, *, perm_type: str = "feistel"):
        from . import permutation

        return permutation.EraShufflingDataset(self, era_length, key=key, perm_type=perm_type)


async def naive_busy_wait_until_len_at_least(dataset: AsyncDataset, length: int) -> int:
    while not await dataset.final_length_is_known():
        cur = await dataset.current_len()
        if cur is None:
            raise ValueError("Dataset has unknown length")
        if cur >= length:
            return cur
        await asyncio.sleep(0.1)
    return await dataset.async_len()


class SyncDataset(DatasetBase[T_co]):
    @abc.abstractmethod
    def __len__(self) -> int:
        ...

    @abc.abstractmethod
    def has_len(self) -> bool:
        ...

    @abc.abstractmethod
    def current_len(self) -> Optional[int]:
        ...

    def __getitem__(self, index: int) -> T_co:
        return self.get_batch([index])[0]

    @abc.abstractmethod
    def get_batch(self, indices: Sequence[int]) -> Sequence[T_co]:
        ...

    def as_async_dataset(self) -> AsyncDataset[T_co]:
        return AsyncifiedDataset(self)

    def as_sync_dataset(self) -> "SyncDataset[T_co]":
        return self


class SyncifiedDataset(SyncDataset[T_co]):
    def __init__(self, dataset: AsyncDataset[T_co]):
        self.dataset = dataset

    def _run(self, coro):
        return blocking_wait(coro)

    def __len__(self) -> int:
        return self._run(self.dataset.async_len())

    def has_len(self) -> bool:
        return self.dataset.is_finite()

    def current_len(self) -> Optional[int]:
        return self._run(self.dataset.current_len())

    def get_batch(self, indices: Sequence[int]) -> Sequence[T_co]:
        return self._run(self.dataset.get_batch(indices))

    def __getitem__(self, index: int) -> T_co:
        return self._run(self.dataset.getitem_async(index))


class AsyncifiedDataset(AsyncDataset[T_co]):
    def __init__(self, dataset: SyncDataset[T_co]):
        super().__init__()
        self.dataset = dataset

    async def async_len(self) -> int:
        return len(self.dataset)

    async def final_length_is_known(self) -> bool:
        return self.dataset.has_len()

    def is_finite(self) -> bool:
        return self.dataset.has_len()

    async def current_len(self) -> Optional[int]:
        return self.dataset.current_len()

    async def get_batch(self, indices: Sequence[int]) -> Sequence[T_co]:
        return self.dataset.get_batch(indices)

    async def getitem_async(self, index: int) -> T_co:
        return self.dataset[index]


class ListAsyncDataset(AsyncDataset[T]):
    """In-memory dataset that can be appended to and finalised (mainly for tests and small evaluation sets)."""

    def __init__(self, data: Optional[List[T]] = None, is_complete: bool = False):
        super().__init__()
        self.data = list(data) if data is not None else []
        self.is_complete = is_complete
        self._cond: Optional[asyncio.Condition] = None
        self._finished = asyncio.Event() if False else None

    async def async_len(self) -> int:
        while not self.is_complete:
            await asyncio.sleep(0.01)
        return len(self.data)

    async def final_length_is_known(self) -> bool:
        return self.is_complete

    def is_finite(self) -> bool:
        return True

    async def current_len(self) -> Optional[int]:
        return len(self.data)

    async def get_batch(self, indices: Sequence[int]) -> Sequence[T]:
        if not indices:
            return []
        await self.wait_until_len_at_least(max(indices) + 1)
        return [self.data[i] for i in indices]

    async def wait_until_len_at_least(self, length: int) -> int:
        while len(self.data) < length and not self.is_complete:
            await asyncio.sleep(0.01)
        return len(self.data)

    def append(self, item: T):
        if self.is_complete:
            raise ValueError("Cannot append to a finalized dataset")
        self.data.append(item)

    def finalize(self):
        self.is_complete = True


class MappedAsyncDataset(AsyncDataset[U]):
    """Per-item map.  When ``fn`` accepts ``key`` (or ``rng``) a per-index key derived from the base key is passed so that
    random maps are reproducible per example (src/levanter/data/dataset.py:370-391)."""

    def __init__(self, dataset: AsyncDataset, fn: Callable[..., U], *extra_args, **extra_kwargs):
        super().__init__()
        self.dataset = dataset
        self.fn = fn
        self._extra_args = extra_args
        self._extra_kwargs = dict(extra_kwargs)
        self._key = self._extra_kwargs.pop("key", None)

    async def async_len(self) -> int:
        return await self.dataset.async_len()

    async def final_length_is_known(self) -> bool:
        return await self.dataset.final_length_is_known()

    def is_finite(self) -> bool:
        return self.dataset.is_finite()

    async def current_len(self) -> Optional[int]:
        return await self.dataset.current_len()

    def _call(self, item, index):
        if self._key is not None:
            return self.fn(item, *self._extra_args, key=_fold_in(self._key, index), **self._extra_kwargs)
        return self.fn(item, *self._extra_args, **self._extra_kwargs)

    async def get_batch(self, indices: Sequence[int]) -> Sequence[U]:
        items = await self.dataset.get_batch(indices)
        return [self._call(it, i) for it, i in zip(items, indices)]

    async def getitem_async(self, index: int) -> U:
        return self._call(await self.dataset.getitem_async(index), index)

    async def wait_until_len_at_least(self, length: int) -> int:
        return await self.dataset.wait_until_len_at_least(length)


def _fold_in(key, index: int) -> int:
    """Deterministic 63-bit key derived from ``(key, index)`` (splitmix64 mixing)."""
    k = int(key) if not hasattr(key, "__len__") else int(np.asarray(key).astype(np.uint64).sum())
    z = (k * 0x9E3779B97F4A7C15 + index * 0xBF58476D1CE4E5B9 + 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return (z ^ (z >> 31)) & 0x7FFFFFFFFFFFFFFF


class SlicedAsyncDataset(AsyncDataset[U]):
    def __init__(self, dataset: AsyncDataset[U], start_index: Optional[int] = None, end_index: Optional[int] = None):
        super().__init__()
        if start_index is None:
            start_index = 0
        if end_index is not None and start_index > end_index:
            raise ValueError("End index must come after start index.")
        self.start_index = start_index
        self.end_index = end_index
        self.dataset = dataset
        self._min_known_len = dataset._min_known_len if end_index is None else (end_index - start_index)

    async def get_batch(self, indices: Sequence[int]) -> Sequence[U]:
        shifted = [i + self.start_index for i in indices]
        if self.end_index is not None and any(i >= self.end_index for i in shifted):
            raise IndexError("index out of range of the sliced dataset")
        return await self.dataset.get_batch(shifted)

    async def async_len(self) -> int:
        n = await self.dataset.async_len()
        if self.end_index is None:
            return max(n - self.start_index, 0)
        return max(min(self.end_index, n) - self.start_index, 0)

    async def final_length_is_known(self) -> bool:
        under = await self.dataset.final_length_is_known()
        if under:
            return True
        if self.end_index is not None:
            cur = await self.dataset.current_len()
            return cur is not None and cur >= self.end_index
        return False

    def is_finite(self) -> bool:
        return self.end_index is not None or self.dataset.is_finite()

    async def current_len(self) -> Optional[int]:
        cur = await self.dataset.current_len()
        if cur is None:
            return None
        if self.end_index is None:
            return max(cur - self.start_index, 0)
        return max(min(self.end_index, cur) - self.start_index, 0)

    async def wait_until_len_at_least(self, length: int) -> int:
        n = await self.dataset.wait_until_len_at_least(length + self.start_index)
        if self.end_index is not None:
            n = min(n, self.end_index)
        return max(n - self.start_index, 0)


class BatchMappedAsyncDataset(AsyncDataset[U]):
    """Map applied to whole batches (``fn(list_of_items) -> list_of_items``)."""

    def __init__(self, dataset: AsyncDataset, fn: Callable[..., Sequence[U]], *extra_args, **extra_kwargs):
        super().__init__()
        self.dataset = dataset
        self.fn = fn
        self._extra_args = extra_args
        self._extra_kwargs = dict(extra_kwargs)
        self._key = self._extra_kwargs.pop("key", None)

    async def async_len(self) -> int:
        return await self.dataset.async_len()

    async def final_length_is_known(self) -> bool:
        return await self.dataset.final_length_is_known()

    def is_finite(self) -> bool:
        return self.dataset.is_finite()

    async def current_len(self) -> Optional[int]:
        return await self.dataset.current_len()

    async def get_batch(self, indices: Sequence[int]) -> Sequence[U]:
        items = await self.dataset.get_batch(indices)
        if self._key is not None:
            return self.fn(items, *self._extra_args, key=_fold_in(self._key, indices[0] if indices else 0), **self._extra_kwargs)
        return self.fn(items, *self._extra_args, **self._extra_kwargs)

    async def wait_until_len_at_least(self, length: int) -> int:
        return await self.dataset.wait_until_len_at_least(length)


class EpochDataset(AsyncDataset[T_co]):
    """Infinite view that wraps around the underlying dataset (``index mod len``), optionally for ``max_epochs``
    (src/levanter/data/dataset.py:510-588)."""

    def __init__(self, dataset: AsyncDataset[T_co], max_epochs: Optional[int] = None):
        super().__init__()
        self.dataset = dataset
        self.max_epochs = max_epochs

    async def async_len(self) -> int:
        if self.max_epochs is None:
            raise ValueError("Cannot determine length of an infinite dataset without max_epochs.")
        return self.max_epochs * await self.dataset.async_len()

    async def final_length_is_known(self) -> bool:
        return await self.dataset.final_length_is_known()

    def is_finite(self) -> bool:
        return self.max_epochs is not None and self.dataset.is_finite()

    async def current_len(self) -> Optional[int]:
        if self.max_epochs is None:
            return None
        cur = await self.dataset.current_len()
        return None if cur is None else self.max_epochs * cur

    async def get_batch(self, indices: Sequence[int]) -> Sequence[T_co]:
        if await self.dataset.final_length_is_known():
            n = await self.dataset.async_len()
        else:
            n = await self.dataset.wait_until_len_at_least(max(indices) + 1 if indices else 1)
            if await self.dataset.final_length_is_known():
                n = await self.dataset.async_len()
        if n == 0:
            raise ValueError("Dataset is empty.")
        if self.max_epochs is not None and indices and max(indices) >= self.max_epochs * n:
            raise StopIteration(f"Reached maximum number of epochs: epoch {max(indices) // n}")
        return await self.dataset.get_batch([i % n for i in indices])

    async def wait_until_len_at_least(self, length: int) -> int:
        if await self.dataset.final_length_is_known():
            return length
        return await self.dataset.wait_until_len_at_least(length)
