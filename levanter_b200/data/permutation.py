"""Shuffled views of datasets (src/levanter/data/permutation.py): a full stateless permutation of a finite dataset, and
era shuffling (permute within consecutive windows of ``era_length``) for datasets that are still growing."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from ._prp import Permutation
from .dataset import AsyncDataset, T_co, _fold_in


class PermutationDataset(AsyncDataset[T_co]):
    """Random permutation of a finite dataset; the permutation is built once the length is known."""

    def __init__(self, dataset: AsyncDataset[T_co], key, perm_type: str = "feistel"):
        super().__init__()
        self.dataset = dataset
        self.key = key
        self._permutation: Optional[Permutation] = None
        self._perm_type = perm_type or "feistel"

    async def async_len(self) -> int:
        return await self.dataset.async_len()

    async def final_length_is_known(self) -> bool:
        return await self.dataset.final_length_is_known()

    def is_finite(self) -> bool:
        return self.dataset.is_finite()

    async def current_len(self) -> Optional[int]:
        if await self.final_length_is_known():
            return await self.async_len()
        return None  # cannot index into a permutation of an unknown length

    async def getitem_async(self, index: int) -> T_co:
        perm = await self._get_permutation()
        return await self.dataset.getitem_async(int(perm(index)))

    async def get_batch(self, indices: Sequence[int]) -> Sequence[T_co]:
        perm = await self._get_permutation()
        return await self.dataset.get_batch([int(perm(i)) for i in indices])

    async def _get_permutation(self) -> Permutation:
        if self._permutation is None:
            self._permutation = Permutation.make(self._perm_type, await self.async_len(), self.key)
        return self._permutation

    async def wait_until_len_at_least(self, length: int) -> int:
        return await self.async_len()


class EraShufflingDataset(AsyncDataset[T_co]):
    """Shuffle within eras of ``era_length`` consecutive examples; era ``e`` uses the permutation keyed by ``fold_in(key, e)``.
    Works on datasets whose length is not known yet; an incomplete last era is shuffled over the items that exist."""

    def __init__(self, dataset: AsyncDataset[T_co], era_length: int, *, key, perm_type: str = "feistel"):
        super().__init__()
        self.dataset = dataset
        self.era_length = era_length
        self.key = key
        self._perm_type = perm_type or "feistel"
        self._cache = {}

    def _era_permutation(self, era: int, length: int) -> Permutation:
        k = (era, length)
        if k not in self._cache:
            if len(self._cache) > 16:
                self._cache.pop(next(iter(self._cache)))
            self._cache[k] = Permutation.make(self._perm_type, length, _fold_in(self.key, era))
        return self._cache[k]

    async def _map_index(self, index: int) -> int:
        if index < 0:
            raise ValueError("Negative indices are not supported")
        era = index // self.era_length
        era_start = era * self.era_length
        n = await self.dataset.wait_until_len_at_least((era + 1) * self.era_length)
        era_len = min(self.era_length, n - era_start)
        if era_len <= 0 or index - era_start >= era_len:
            raise IndexError(f"Index {index} is out of bounds for a dataset of length {n}")
        return era_start + int(self._era_permutation(era, era_len)(index - era_start))

    async def async_len(self) -> int:
        return await self.dataset.async_len()

    async def final_length_is_known(self) -> bool:
        return await self.dataset.final_length_is_known()

    def is_finite(self) -> bool:
        return self.dataset.is_finite()

    async def current_len(self) -> Optional[int]:
        return await self.dataset.current_len()

    async def getitem_async(self, index: int) -> T_co:
        return await self.dataset.getitem_async(await self._map_index(index))

    async def get_batch(self, indices: Sequence[int]) -> Sequence[T_co]:
        return await self.dataset.get_batch([await self._map_index(i) for i in indices])

    async def wait_until_len_at_least(self, length: int) -> int:
        return await self.dataset.wait_until_len_at_least(length)
