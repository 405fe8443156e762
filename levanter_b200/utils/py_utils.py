"""Host helpers: resource discovery, stopwatch, RNG seeding, cycling iterators
(src/levanter/utils/py_utils.py:11-158)."""
from __future__ import annotations

import contextlib
import os
import random
import sys
import time
from dataclasses import dataclass
from typing import Iterable, Iterator, TypeVar

import numpy as np
import torch

T = TypeVar("T")


def logical_cpu_core_count() -> int:
    """CPU cores this process may use, honouring SLURM's allocation."""
    n = os.getenv("SLURM_CPUS_ON_NODE") or os.getenv("SLURM_CPUS_PER_TASK")
    if n:
        try:
            return int(n)
        except ValueError:
            pass
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def logical_cpu_memory_size() -> float:
    """Memory (GB) available to this job, honouring SLURM."""
    mem = os.getenv("SLURM_MEM_PER_NODE")
    if mem:
        try:
            return float(mem) / 1e3
        except ValueError:
            pass
    try:
        import psutil

        return psutil.virtual_memory().total / 1e9
    except Exception:
        return 16.0


def non_caching_cycle(iterable: Iterable[T]) -> Iterator[T]:
    """Like ``itertools.cycle`` but re-iterates the source instead of caching items."""
    while True:
        empty = True
        for x in iterable:
            empty = False
            yield x
        if empty:
            return


def actual_sizeof(obj) -> int:
    """Recursive ``sys.getsizeof`` over containers."""
    seen = set()

    def go(o):
        if id(o) in seen:
            return 0
        seen.add(id(o))
        size = sys.getsizeof(o)
        if isinstance(o, dict):
            size += sum(go(k) + go(v) for k, v in o.items())
        elif isinstance(o, (list, tuple, set, frozenset)):
            size += sum(go(i) for i in o)
        elif hasattr(o, "__dict__"):
            size += go(vars(o))
        return size

    return go(obj)


class Stopwatch:
    """Resumable stopwatch."""

    def __init__(self):
        self._start = time.perf_counter()
        self._elapsed = 0.0
        self._n = 0

    def start(self):
        self._start = time.perf_counter()
        self._n += 1

    def stop(self):
        self._elapsed += time.perf_counter() - self._start

    def reset(self):
        self._elapsed = 0.0

    def elapsed(self) -> float:
        return self._elapsed

    def average(self) -> float:
        return self._elapsed / max(self._n, 1)

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()


@contextlib.contextmanager
def set_global_rng_seeds(seed: int):
    """Seed python/numpy/torch RNGs and restore their states on exit."""
    py_state = random.getstate()
    np_state = np.random.get_state()
    torch_state = torch.random.get_rng_state()
    try:
        random.seed(seed)
        np.random.seed(seed % (2**32))
        torch.manual_seed(seed)
        yield
    finally:
        random.setstate(py_state)
        np.random.set_state(np_state)
        torch.random.set_rng_state(torch_state)


def dataclass_with_default_init(_cls=None, **kwargs):
    """``@dataclass`` that keeps the generated ``__init__`` as ``__default_init__`` when the class defines its own."""
    import dataclasses

    def wrap(cls):
        user_init = cls.__dict__.get("__init__")
        if user_init is not None:
            delattr(cls, "__init__")
        out = dataclasses.dataclass(cls, **kwargs)
        out.__default_init__ = out.__init__
        if user_init is not None:
            out.__init__ = user_init
        return out

    return wrap if _cls is None else wrap(_cls)
