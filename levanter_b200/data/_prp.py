"""Stateless pseudo-random permutations of ``[0, n)`` (src/levanter/data/_prp.py): an LCG ``(a x + b) mod n`` and a Feistel
network with cycle walking.  Both map an index to its image without materialising the permutation, so shuffling a
trillion-token dataset costs nothing and is a pure function of (key, index)."""
from __future__ import annotations

import math
from typing import Union

import numpy as np


class Permutation:
    length: int

    def __call__(self, indices):
        raise NotImplementedError

    @staticmethod
    def make(kind: str, length: int, prng_key, **kwargs) -> "Permutation":
        kind = (kind or "feistel").lower()
        if kind == "feistel":
            return FeistelPermutation(length, prng_key, **kwargs)
        if kind == "linear":
            return LcgPermutation(length, prng_key)
        raise ValueError(f"Unknown permutation type: {kind}")


def _rng(prng_key) -> np.random.Generator:
    k = np.asarray(prng_key).astype(np.uint64).reshape(-1) if hasattr(prng_key, "__len__") else np.asarray([int(prng_key)], dtype=np.uint64)
    return np.random.Generator(np.random.PCG64([int(x) for x in k]))


def _check(indices, length):
    if isinstance(indices, (int, np.integer)):
        if indices < 0 or indices >= length:
            raise IndexError(f"index {indices} is out of bounds for length {length}")
        return None
    arr = np.asarray(indices)
    if arr.size and (arr.min() < 0 or arr.max() >= length):
        raise IndexError(f"index out of bounds for length {length}")
    return arr


class LcgPermutation(Permutation):
    """``x -> (a x + b) mod n`` with ``gcd(a, n) = 1`` (a bijection on ``Z_n``)."""

    def __init__(self, length: int, prng_key):
        self.length = int(length)
        rng = _rng(prng_key)
        self.a = self._generate_a(rng)
        self.b = int(rng.integers(0, max(self.length, 1)))

    def _generate_a(self, rng) -> int:
        if self.length <= 1:
            return 1
        while True:
            a = int(rng.integers(1, self.length))
            if math.gcd(a, self.length) == 1:
                return a

    def __call__(self, indices):
        arr = _check(indices, self.length)
        if arr is None:
            return (self.a * int(indices) + self.b) % self.length
        # Python ints avoid overflow for very large lengths
        if self.length > (1 << 31):
            return np.array([(self.a * int(i) + self.b) % self.length for i in arr.reshape(-1)], dtype=np.int64).reshape(arr.shape)
        return ((self.a * arr.astype(np.int64) + self.b) % self.length).astype(np.int64)


class FeistelPermutation(Permutation):
    """Balanced Feistel network over ``2 * ceil(log2(n) / 2)`` bits with cycle walking back into ``[0, n)``."""

    def __init__(self, length: int, prng_key, rounds: int = 5):
        self.length = int(length)
        self.rounds = rounds
        bits = max(2, (max(self.length - 1, 1)).bit_length())
        if bits % 2:
            bits += 1
        self.half_bits = bits // 2
        self.mask = (1 << self.half_bits) - 1
        rng = _rng(prng_key)
        self.keys = [int(rng.integers(0, 1 << 62)) for _ in range(rounds)]

    def _round(self, r: int, key: int) -> int:
        x = (r ^ key) & 0xFFFFFFFFFFFFFFFF
        x = (x * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 29
        x = (x * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 32
        return x & self.mask

    def _encrypt(self, x: int) -> int:
        left, right = x >> self.half_bits, x & self.mask
        for k in self.keys:
            left, right = right, left ^ self._round(right, k)
        return (left << self.half_bits) | right

    def _one(self, i: int) -> int:
        x = self._encrypt(int(i))
        while x >= self.length:
            x = self._encrypt(x)
        return x

    def __call__(self, indices):
        arr = _check(indices, self.length)
        if arr is None:
            return self._one(int(indices))
        return np.array([self._one(int(i)) for i in arr.reshape(-1)], dtype=np.int64).reshape(arr.shape)
