"""Tracker helpers (src/levanter/tracker/helpers.py:20-96)."""
from __future__ import annotations

import contextlib
import subprocess
import sys
import time
from typing import Optional


def log_optimizer_hyperparams(opt_state, prefix: Optional[str] = None, *, step=None):
    """Log hyperparameters recorded by ``inject_hyperparams`` (e.g. ``optim/learning_rate``)."""
    from .tracker_fns import jit_log

    params = {}
    hp = getattr(opt_state, "hyperparams", None)
    if hp is None and hasattr(opt_state, "inner_opt_state"):
        hp = getattr(opt_state.inner_opt_state, "hyperparams", None)
    if hp:
        for k, v in hp.items():
            params[f"{prefix}/{k}" if prefix else k] = float(v)
    if params:
        jit_log(params, step=step)
    return params


@contextlib.contextmanager
def capture_time():
    start = time.perf_counter()
    done = False

    def fn():
        return end - start if done else time.perf_counter() - start

    yield fn
    end = time.perf_counter()
    done = True


def generate_pip_freeze() -> str:
    try:
        from importlib.metadata import distributions

        return "\n".join(sorted(f"{d.metadata['Name']}=={d.version}" for d in distributions() if d.metadata["Name"]))
    except Exception:
        try:
            return subprocess.check_output([sys.executable, "-m", "pip", "freeze"], text=True)
        except Exception:
            return ""


def infer_experiment_git_root():
    from ..utils.logging import infer_experiment_git_root as f

    return f()
