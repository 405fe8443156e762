"""Global tracker functions (src/levanter/tracker/tracker_fns.py:36-311): ``log``, ``jit_log``,
``defer_tracker_for_jit``, ``log_summary``, ``log_hyperparameters``, ``log_configuration``, ``current_tracker``,
``get_tracker``.

There is no tracing compiler here, so "jit" metrics are simply values produced inside the training step: ``jit_log``
stores them in the innermost ``defer_tracker_for_jit`` capture (the trainer opens one around every step and logs
the captured dict with the step's other metrics) or logs them directly when no capture is open.  Tensor values are
kept on the device until they are logged, so logging them does not force a synchronisation inside the step."""
from __future__ import annotations

import contextlib
import dataclasses
import logging
import os
import tempfile
import threading
import warnings
from typing import Any, Dict, List, Optional

import torch

from .tracker import CompositeTracker, DictTracker, NoopTracker, Tracker

logger = logging.getLogger(__name__)
_should_use_callback = True
_global_tracker: Optional[Tracker] = None
_has_logged_missing_tracker = False
_tls = threading.local()


def _capture_stack() -> List[Dict[str, Any]]:
    if not hasattr(_tls, "stack"):
        _tls.stack = []
    return _tls.stack


def _to_python(v):
    if isinstance(v, torch.Tensor):
        if v.numel() == 1:
            return v.detach().float().item()
        return v.detach().float().cpu()
    return v


def log(metrics: Dict[str, Any], *, step: Optional[int], commit: Optional[bool] = None):
    """Log metrics to the current global tracker."""
    global _has_logged_missing_tracker
    if _global_tracker is None:
        if not _has_logged_missing_tracker:
            warnings.warn("No global tracker set")
            _has_logged_missing_tracker = True
        return
    _global_tracker.log({k: _to_python(v) for k, v in metrics.items()}, step=step, commit=commit)


log_metrics = log


def jit_log(metrics: Dict[str, Any], *, step=None):
    """Record metrics produced inside a training step."""
    stack = _capture_stack()
    if stack:
        stack[-1].update(metrics)
    else:
        log(metrics, step=step)


@contextlib.contextmanager
def defer_tracker_for_jit():
    """Capture ``jit_log`` calls made in the body into a dict (yielded)."""
    captured: Dict[str, Any] = {}
    stack = _capture_stack()
    stack.append(captured)
    try:
        yield captured
    finally:
        stack.pop()


def log_summary(metrics: Dict[str, Any]):
    global _has_logged_missing_tracker
    if _global_tracker is None:
        if not _has_logged_missing_tracker:
            warnings.warn("No global tracker set")
            _has_logged_missing_tracker = True
        return
    _global_tracker.log_summary({k: _to_python(v) for k, v in metrics.items()})


def log_hyperparameters(hparams: Dict[str, Any]):
    global _has_logged_missing_tracker
    if _global_tracker is None:
        if not _has_logged_missing_tracker:
            warnings.warn("No global tracker set")
            _has_logged_missing_tracker = True
        return
    _global_tracker.log_hyperparameters(hparams)


def log_configuration(hparams: Any, config_name: Optional[str] = None):
    """Log a config dataclass as hyperparameters and as a YAML artifact."""
    global _has_logged_missing_tracker
    if _global_tracker is None:
        if not _has_logged_missing_tracker:
            warnings.warn("No global tracker set")
            _has_logged_missing_tracker = True
        return
    from ..config import encode, to_yaml

    _global_tracker.log_hyperparameters(_flatten(encode(hparams)))
    with tempfile.TemporaryDirectory() as tmpdir:
        path = os.path.join(tmpdir, config_name or "config.yaml")
        with open(path, "w") as f:
            f.write(to_yaml(hparams))
        _global_tracker.log_artifact(path, name=config_name or "config.yaml", type="config")


def _flatten(d, prefix=""):
    out = {}
    if isinstance(d, dict):
        for k, v in d.items():
            out.update(_flatten(v, f"{prefix}{k}." if not prefix else f"{prefix}{k}."))
        return {k.rstrip("."): v for k, v in out.items()}
    out[prefix.rstrip(".")] = d
    return out


def set_global_tracker(tracker: Tracker):
    global _global_tracker
    if _global_tracker is not None:
        warnings.warn("Global tracker is already set. Overwriting it.")
    _global_tracker = tracker


class current_tracker(contextlib.AbstractContextManager):
    """``current_tracker()`` returns the global tracker; ``with current_tracker(t):`` installs ``t`` temporarily."""

    def __new__(cls, tracker: Optional[Tracker] = None):
        if tracker is None:
            global _has_logged_missing_tracker
            if _global_tracker is None:
                raise RuntimeError("No global tracker set")
            return _global_tracker
        return super().__new__(cls)

    def __init__(self, tracker: Optional[Tracker] = None):
        self.tracker = tracker
        self.old = None

    def __enter__(self):
        global _global_tracker
        self.old = _global_tracker
        _global_tracker = self.tracker
        return self.tracker

    def __exit__(self, *exc):
        global _global_tracker
        _global_tracker = self.old


def get_tracker(name: str) -> Tracker:
    """Find a tracker by name in the current (possibly composite) tracker."""
    if _global_tracker is None:
        raise RuntimeError("No global tracker set")
    if isinstance(_global_tracker, CompositeTracker):
        for t in _global_tracker.loggers:
            if t.name == name:
                return t
    elif _global_tracker.name == name:
        return _global_tracker
    raise KeyError(f"Tracker with name {name} not found")
