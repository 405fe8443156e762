"""Synthetic token data: uniform-random token ids that are a pure function of ``(seed, index)``.

Used by the benchmarks and by tests that need a dataset of a given shape without any files."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..models.lm_model import LmExample
from .dataset import AsyncDataset


class SyntheticLmDataset(AsyncDataset[LmExample]):
    def __init__(self, vocab_size: int, seq_len: int, seed: int = 0, length: Optional[int] = None):
        super().__init__()
        self.vocab_size = vocab_size
        self.seq_len = seq_len
        self.seed = seed
        self.length = length

    async def async_len(self) -> int:
        if self.length is None:
            raise ValueError("infinite dataset")
        return self.length

    async def final_length_is_known(self) -> bool:
        return True

    def is_finite(self) -> bool:
        return self.length is not None

    async def current_len(self) -> Optional[int]:
        return self.length

    def tokens_at(self, index: int) -> torch.Tensor:
        # The example index is part of the Philox KEY, not the counter: the counter advances by one per block of draws, so
        # streams that differ only in their starting counter are shifted copies of one another.
        key = np.array([np.uint64(self.seed & 0xFFFFFFFFFFFFFFFF), np.uint64(index & 0xFFFFFFFFFFFFFFFF)], dtype=np.uint64)
        rng = np.random.Generator(np.random.Philox(key=key))
        return torch.from_numpy(rng.integers(0, self.vocab_size, size=self.seq_len, dtype=np.int32))

    async def get_batch(self, indices: Sequence[int]):
        return [LmExample.causal(self.tokens_at(i)) for i in indices]
