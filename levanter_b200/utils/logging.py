"""Logging set-up and timing iterators (src/levanter/utils/logging.py:18-89)."""
from __future__ import annotations

import logging as pylogging
import os
import time
from pathlib import Path
from typing import Iterator, Optional, TypeVar, Union

T = TypeVar("T")


def _rank() -> int:
    for k in ("RANK", "SLURM_PROCID"):
        if k in os.environ:
            try:
                return int(os.environ[k])
            except ValueError:
                pass
    return 0


def init_logging(log_dir: Union[str, Path], run_id: str, level: int = pylogging.INFO) -> None:
    """Log to ``<log_dir>/<run_id>.log`` and the console; the format carries the process rank."""
    log_dir = Path(log_dir)
    log_dir.mkdir(parents=True, exist_ok=True)
    path = log_dir / f"{run_id}.log"
    fmt = pylogging.Formatter(f"%(asctime)s - {_rank()} - %(name)s - %(filename)s:%(lineno)d - %(levelname)s :: %(message)s")
    root = pylogging.getLogger()
    for h in list(root.handlers):
        root.removeHandler(h)
    fh = pylogging.FileHandler(path, mode="a")
    fh.setFormatter(fmt)
    sh = pylogging.StreamHandler()
    sh.setFormatter(fmt)
    root.addHandler(fh)
    root.addHandler(sh)
    root.setLevel(level)
    pylogging.getLogger("fsspec").setLevel(pylogging.WARNING)


def silence_transformer_nag():
    os.environ.setdefault("TRANSFORMERS_NO_ADVISORY_WARNINGS", "1")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")


class LoadingTimeTrackerIterator(Iterator[T]):
    """Wrap an iterator and record how long each ``next`` took (feeds ``throughput/loading_time``)."""

    def __init__(self, items: Iterator[T]):
        self.total_time = 0.0
        self.this_load_time = 0.0
        self.items = iter(items)

    def __iter__(self):
        return self

    def __next__(self) -> T:
        t0 = time.perf_counter()
        item = next(self.items)
        self.this_load_time = time.perf_counter() - t0
        self.total_time += self.this_load_time
        return item


def infer_experiment_git_root() -> Optional[str]:
    """Walk up from the caller's file to the enclosing git checkout."""
    import inspect

    for frame in inspect.stack()[1:]:
        fname = frame.filename
        if not os.path.exists(fname):
            continue
        d = os.path.dirname(os.path.abspath(fname))
        while d != os.path.dirname(d):
            if os.path.exists(os.path.join(d, ".git")):
                return d
            d = os.path.dirname(d)
    return None
