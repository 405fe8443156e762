"""Deterministic mixtures of datasets (src/levanter/data/mixture.py).

Indices are assigned in blocks of ``block_size``: inside a block each source gets an exact count proportional to its weight
(:157-165), the block's slots are permuted with a key folded with the block number (:304-307), and a source index counts how
many of its items earlier blocks consumed.  Weights may change at *stage* boundaries given as sequence indices that are
multiples of ``block_size`` (:117-136, 219-230).  ``stop_strategy``: ``restart`` wraps exhausted sources, ``first_exhausted``
ends the mixture when any source runs out."""
from __future__ import annotations

import warnings
from typing import Dict, List, Mapping, Optional, Sequence, Tuple, TypeVar, Union

import numpy as np

from ._prp import Permutation
from .dataset import AsyncDataset, _fold_in

T = TypeVar("T")


class StopStrategy:
    FIRST_STOP_STRATEGY = "first_exhausted"
    ALL_STOP_STRATEGY = "all_exhausted"
    RESTART_STRATEGY = "restart"
    VALID = [FIRST_STOP_STRATEGY, ALL_STOP_STRATEGY, RESTART_STRATEGY]


def rescale_mixture_schedule_for_batch_schedule(mixture_schedule: Sequence[Tuple[int, Dict[str, float]]], batch_schedule) -> List[Tuple[int, Dict[str, float]]]:
    """Convert stage starts given in *steps* into sequence indices (src/levanter/data/mixture.py:310-340)."""
    return [(batch_schedule.global_data_offset_by_step(step), w) for step, w in mixture_schedule]


class MixtureDataset(AsyncDataset[T]):
    def __init__(self, datasets: Mapping[str, AsyncDataset[T]], weights: Union[Dict[str, float], List[Tuple[int, Dict[str, float]]]],
                 block_size: int, *, randomize_blocks: bool = True, key, stop_strategy: str = StopStrategy.RESTART_STRATEGY):
        super().__init__()
        if isinstance(weights, dict):
            weight_stages = [(0, weights)]
        else:
            weight_stages = list(weights)
            if not weight_stages:
                raise ValueError("weights must not be empty")
            starts = [s for s, _ in weight_stages]
            if starts[0] != 0:
                raise ValueError("The first stage must start at index 0")
            if any(b <= a for a, b in zip(starts, starts[1:])):
                raise ValueError("Stage start indices must be strictly increasing")
            for s in starts:
                if s % block_size != 0:
                    raise ValueError(f"Stage start index {s} must be a multiple of block_size {block_size}")
        self.weight_stages = [(s, self._normalize(w)) for s, w in weight_stages]
        all_keys = set(datasets.keys())
        for _, w in self.weight_stages:
            if set(w.keys()) != all_keys:
                missing, extra = all_keys - set(w.keys()), set(w.keys()) - all_keys
                if extra:
                    raise ValueError(f"weights name datasets that do not exist: {sorted(extra)}")
                for m in missing:
                    w[m] = 0.0
        self.datasets = {n: d for n, d in datasets.items()}
        self.dataset_index = {n: i for i, n in enumerate(self.datasets)}
        self.block_size = block_size
        self.randomize_blocks = randomize_blocks
        self.key = key
        if stop_strategy not in StopStrategy.VALID:
            raise ValueError(f"Stop strategy {stop_strategy} is not supported.")
        if stop_strategy == StopStrategy.ALL_STOP_STRATEGY:
            raise NotImplementedError("all_exhausted is not supported")
        self.stop_strategy = stop_strategy
        # counts per block for each stage and cumulative counts at stage starts
        self._counts_per_block = [self._compute_expected_counts_per_block(w) for _, w in self.weight_stages]
        self._counts_at_start_of_stage = self._compute_counts_at_start_of_each_stage()

    @staticmethod
    def _normalize(w: Dict[str, float]) -> Dict[str, float]:
        tot = sum(w.values())
        if tot <= 0:
            raise ValueError("Datasets or weights are empty")
        return {k: v / tot for k, v in w.items()}

    def _compute_expected_counts_per_block(self, weights: Dict[str, float]) -> np.ndarray:
        names = list(self.datasets.keys())
        w = np.array([weights.get(n, 0.0) for n in names], dtype=np.float64)
        expected = w * self.block_size
        counts = np.floor(expected).astype(np.int64)
        rem = self.block_size - counts.sum()
        if rem > 0:
            order = np.argsort(-(expected - counts), kind="stable")
            for i in order[:rem]:
                counts[i] += 1
        return counts

    def _compute_counts_at_start_of_each_stage(self) -> List[np.ndarray]:
        out = [np.zeros(len(self.datasets), dtype=np.int64)]
        for i in range(len(self.weight_stages) - 1):
            nblocks = (self.weight_stages[i + 1][0] - self.weight_stages[i][0]) // self.block_size
            out.append(out[-1] + nblocks * self._counts_per_block[i])
        return out

    def _stage_of_block(self, block: int) -> int:
        idx = block * self.block_size
        st = 0
        for i, (s, _) in enumerate(self.weight_stages):
            if idx >= s:
                st = i
        return st

    def _block_assignments(self, block: int) -> np.ndarray:
        """Packed ids ``(dataset << 32) + position-in-block`` for every slot of ``block`` (position counts per source)."""
        stage = self._stage_of_block(block)
        counts = self._counts_per_block[stage]
        ids = np.concatenate([np.full(c, d, dtype=np.int64) for d, c in enumerate(counts)])
        pos = np.concatenate([np.arange(c, dtype=np.int64) for c in counts])
        packed = (ids << 32) + pos
        if self.randomize_blocks:
            perm = Permutation.make("feistel", len(packed), _fold_in(self.key, block))
            packed = packed[perm(np.arange(len(packed)))]
        return packed

    def _index_into_dataset(self, block: int, ds: int, pos: int) -> int:
        stage = self._stage_of_block(block)
        stage_start_block = self.weight_stages[stage][0] // self.block_size
        base = self._counts_at_start_of_stage[stage][ds] + (block - stage_start_block) * self._counts_per_block[stage][ds]
        return int(base + pos)

    async def _remap_indices(self, ds: AsyncDataset, idxs: Sequence[int]) -> Sequence[int]:
        if not idxs:
            return idxs
        mx = max(idxs)
        if self.stop_strategy == StopStrategy.RESTART_STRATEGY:
            if ds.is_finite():
                n = await ds.async_len() if await ds.final_length_is_known() else await ds.wait_until_len_at_least(mx + 1)
                if await ds.final_length_is_known():
                    n = await ds.async_len()
                    if n == 0:
                        raise ValueError("dataset is empty")
                    return [i % n for i in idxs]
            return idxs
        n = await ds.wait_until_len_at_least(mx + 1)
        if mx >= n:
            raise StopIteration
        return idxs

    async def async_len(self) -> int:
        if self.stop_strategy == StopStrategy.RESTART_STRATEGY:
            raise ValueError("Length is infinite for the restart strategy")
        raise NotImplementedError("length of a first_exhausted mixture is not known in advance")

    async def final_length_is_known(self) -> bool:
        return False

    def is_finite(self) -> bool:
        return self.stop_strategy != StopStrategy.RESTART_STRATEGY

    async def current_len(self) -> Optional[int]:
        return None

    async def get_batch(self, indices: Sequence[int]) -> Sequence[T]:
        per_ds: Dict[int, List[Tuple[int, int]]] = {}
        cache: Dict[int, np.ndarray] = {}
        for out_pos, idx in enumerate(indices):
            block, off = divmod(int(idx), self.block_size)
            if block not in cache:
                cache[block] = self._block_assignments(block)
            packed = int(cache[block][off])
            ds, pos = packed >> 32, packed & 0xFFFFFFFF
            per_ds.setdefault(ds, []).append((out_pos, self._index_into_dataset(block, ds, pos)))
        names = list(self.datasets.keys())
        out: List[Optional[T]] = [None] * len(indices)
        for ds, items in per_ds.items():
            d = self.datasets[names[ds]]
            idxs = await self._remap_indices(d, [i for _, i in items])
            got = await d.get_batch(list(idxs))
            for (p, _), g in zip(items, got):
                out[p] = g
        return out  # type: ignore

    async def getitem_async(self, index: int) -> T:
        return (await self.get_batch([index]))[0]
