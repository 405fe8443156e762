"""Resumable, sharded data loader (src/levanter/data/loader.py:68-629).

The order of examples is a pure function of the step: step ``n`` consumes global example indices
``batch_schedule.batch_indices_at_step(n)``; this rank takes the contiguous slice of them that belongs to its
``(replica, data)`` coordinate (every tensor-parallel rank of a group reads the same slice).  Resuming is therefore
``iter_from_step(step)`` with no data seek.  Batches are fetched ``prefetch_size`` at a time by a background thread,
stacked, written into **pinned** host memory and handed to the trainer, which copies them to the GPU on its stream.
A final / non-divisible batch is padded with zeros when ``allow_nondivisible_batch_size`` is set (:340-360)."""
from __future__ import annotations

import asyncio
import logging
import time
from dataclasses import dataclass
from typing import Any, Callable, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..schedule import BatchSchedule, IntSchedule
from ..utils.background_iterable import BackgroundIterator
from ..utils.thread_utils import blocking_wait
from .dataset import AsyncDataset, SyncDataset

logger = logging.getLogger(__name__)


def stack_tree(items: Sequence[Any], pin: bool = False):
    """Stack a list of examples (tensors / numpy arrays / dataclass-like objects with ``stack`` / dicts / tuples)."""
    first = items[0]
    if hasattr(type(first), "stack") and not isinstance(first, torch.Tensor):
        out = type(first).stack(items)
        return _pin(out) if pin else out
    if isinstance(first, torch.Tensor):
        out = torch.stack(list(items))
        return out.pin_memory() if (pin and torch.cuda.is_available()) else out
    if isinstance(first, np.ndarray) or np.isscalar(first):
        out = torch.from_numpy(np.stack([np.asarray(x) for x in items]))
        return out.pin_memory() if (pin and torch.cuda.is_available()) else out
    if isinstance(first, dict):
        return {k: stack_tree([it[k] for it in items], pin) for k in first}
    if isinstance(first, (tuple, list)):
        return type(first)(stack_tree([it[i] for it in items], pin) for i in range(len(first)))
    return list(items)


def _pin(x):
    if not torch.cuda.is_available():
        return x
    if isinstance(x, torch.Tensor):
        return x.pin_memory()
    if hasattr(x, "__dataclass_fields__"):
        import dataclasses

        return dataclasses.replace(x, **{f: _pin(getattr(x, f)) for f in x.__dataclass_fields__})
    if isinstance(x, dict):
        return {k: _pin(v) for k, v in x.items()}
    if isinstance(x, tuple):
        return tuple(_pin(v) for v in x)
    return x


def _zeros_like_example(ex):
    if isinstance(ex, torch.Tensor):
        return torch.zeros_like(ex)
    if isinstance(ex, np.ndarray):
        return np.zeros_like(ex)
    if hasattr(ex, "__dataclass_fields__"):
        import dataclasses

        return dataclasses.replace(ex, **{f: _zeros_like_example(getattr(ex, f)) for f in ex.__dataclass_fields__})
    if isinstance(ex, dict):
        return {k: _zeros_like_example(v) for k, v in ex.items()}
    if isinstance(ex, (tuple, list)):
        return type(ex)(_zeros_like_example(v) for v in ex)
    return ex


class DataLoader(Iterable):
    def __init__(self, data_store: Union[AsyncDataset, SyncDataset], batch_size: Union[int, IntSchedule, BatchSchedule], *,
                 mesh=None, max_buffered_batches: Optional[int] = 64, prefetch_size: int = 32,
                 allow_nondivisible_batch_size: bool = False, pad_final_batch: bool = True, pin_memory: bool = True):
        self.data_store = data_store.as_async_dataset() if hasattr(data_store, "as_async_dataset") else data_store
        self.scheduler = batch_size if isinstance(batch_size, BatchSchedule) else BatchSchedule(batch_size)
        self.mesh = mesh
        self.max_buffered_batches = max_buffered_batches
        self.prefetch_size = prefetch_size
        self.allow_nondivisible_batch_size = allow_nondivisible_batch_size
        self.pad_final_batch = pad_final_batch
        self.pin_memory = pin_memory
        self.num_shards = mesh.batch_size_divisor if mesh is not None else 1
        self.shard_index = mesh.batch_index if mesh is not None else 0
        if not allow_nondivisible_batch_size:
            for bs in self.scheduler.unique_batch_sizes():
                if bs % self.num_shards != 0:
                    raise ValueError(f"batch size {bs} is not divisible by the number of data shards {self.num_shards}; "
                                     "set allow_nondivisible_batch_size")

    def local_indices_at_step(self, step: int) -> Tuple[List[int], int]:
        """Global example indices this rank loads at ``step`` and how many trailing padding rows it adds."""
        idx = self.scheduler.batch_indices_at_step(step)
        bs = len(idx)
        per = -(-bs // self.num_shards)  # ceil
        lo = self.shard_index * per
        hi = min(lo + per, bs)
        mine = [idx[i] for i in range(lo, hi)] if lo < bs else []
        return mine, per - len(mine)

    def __iter__(self) -> "DataLoaderIterator":
        return self.iter_from_step(None)

    def iter_from_step(self, start_from_batch: Optional[int] = None) -> "DataLoaderIterator":
        return DataLoaderIterator(self, start_from_batch=start_from_batch)

    @property
    def batch_size(self) -> int:
        return self.scheduler.batch_size_at_step(0)


class DataLoaderIterator(Iterator):
    def __init__(self, dl: DataLoader, start_from_batch: Optional[int] = None):
        self.dl = dl
        self._start_from_batch = start_from_batch
        self._batch_index = 0 if start_from_batch is None else start_from_batch
        if dl.max_buffered_batches is not None and dl.max_buffered_batches > 0:
            self._batches: Iterator = BackgroundIterator(self._produce_batches, max_capacity=dl.max_buffered_batches)
        else:
            self._batches = _sync_iter(self._produce_batches())

    def __next__(self):
        t0 = time.time()
        item = next(self._batches)
        dt = time.time() - t0
        if dt > 10.0:
            logger.warning(f"Waited {dt:.1f}s for the next batch; the data pipeline is the bottleneck")
        return item

    def __iter__(self):
        return self

    async def _dataset_len_for(self, needed: int) -> Optional[int]:
        ds = self.dl.data_store
        if not ds.is_finite():
            return None
        if await ds.final_length_is_known():
            return await ds.async_len()
        n = await ds.wait_until_len_at_least(needed)
        if await ds.final_length_is_known():
            return await ds.async_len()
        return n if n < needed else None

    async def _produce_batches(self):
        dl = self.dl
        step = self._batch_index
        done = False
        while not done:
            group: List[Tuple[List[int], int]] = []
            for _ in range(dl.prefetch_size):
                idx = dl.scheduler.batch_indices_at_step(step)
                total_len = await self._dataset_len_for(idx[-1] + 1)
                if total_len is not None and idx[0] >= total_len:
                    done = True
                    break
                mine, pad = dl.local_indices_at_step(step)
                if total_len is not None and idx[-1] >= total_len:
                    # ragged final batch
                    if not (dl.pad_final_batch or dl.allow_nondivisible_batch_size):
                        done = True
                        break
                    kept = [i for i in mine if i < total_len]
                    pad += len(mine) - len(kept)
                    mine = kept
                    done = True
                group.append((mine, pad))
                step += 1
                if done:
                    break
            if not group:
                break
            flat = [i for mine, _ in group for i in mine]
            t0 = time.time()
            items = list(await dl.data_store.get_batch(flat)) if flat else []
            dt = time.time() - t0
            if dt > 10.0:
                logger.warning(f"Fetching {len(flat)} examples took {dt:.1f}s")
            pos = 0
            for mine, pad in group:
                rows = items[pos:pos + len(mine)]
                pos += len(mine)
                if pad:
                    if not rows and not items:
                        continue
                    exemplar = rows[0] if rows else items[0]
                    rows = rows + [_zeros_like_example(exemplar)] * pad
                if not rows:
                    continue
                yield stack_tree(rows, pin=dl.pin_memory)


def _sync_iter(agen):
    loop = asyncio.new_event_loop()
    try:
        while True:
            try:
                yield loop.run_until_complete(agen.__anext__())
            except StopAsyncIteration:
                return
    finally:
        loop.close()


def check_sharded_consistency(batch, mesh=None) -> None:
    """Debug check that ranks which must hold identical data (the tensor-parallel group) do
    (src/levanter/data/loader.py:561-620)."""
    import torch.distributed as dist

    if mesh is None or mesh.model_size <= 1 or not dist.is_initialized():
        return
    t = batch.tokens if hasattr(batch, "tokens") else batch
    if not isinstance(t, torch.Tensor):
        return
    dev = torch.device("cuda") if (torch.cuda.is_available() and dist.get_backend() == "nccl") else torch.device("cpu")
    mine = t.to(dev).long().sum().reshape(1)
    parts = [torch.zeros_like(mine) for _ in range(mesh.model_size)]
    dist.all_gather(parts, mine, group=mesh.model_group)
    if any(int(p) != int(mine) for p in parts):
        raise RuntimeError("data differs between tensor-parallel ranks that should hold identical batches")


def stack_batches(example_iterator, Pos, Batch, shard: Optional[Tuple[int, int]] = None):
    """Group an iterator of examples into stacked batches of ``Batch`` rows; a short last batch is padded with all-zero
    examples (zero loss mask).  With ``shard=(index, count)`` each global batch is cut into ``count`` equal slices and only
    slice ``index`` is stacked, so every data-parallel rank can run the same iterator."""
    from .utils import batched

    size = int(getattr(Batch, "size", Batch))
    for rows in batched(example_iterator, size):
        if len(rows) < size:
            rows = rows + [_zeros_like_example(rows[0])] * (size - len(rows))
        if shard is not None:
            idx, cnt = shard
            per = size // cnt
            rows = rows[idx * per:(idx + 1) * per]
        yield stack_tree(rows)
