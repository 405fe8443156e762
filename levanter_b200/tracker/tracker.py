"""Tracker interface and simple implementations (src/levanter/tracker/tracker.py:12-160)."""
from __future__ import annotations

import abc
import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from ..config import ChoiceRegistry


class Tracker(abc.ABC):
    """Receives hyperparameters, per-step metrics, summary values and artifacts.  Usable as a context manager that makes
    it the current global tracker."""

    name: str = "tracker"

    @abc.abstractmethod
    def log_hyperparameters(self, hparams: Dict[str, Any]):
        ...

    @abc.abstractmethod
    def log(self, metrics: Dict[str, Any], *, step: Optional[int], commit: Optional[bool] = None):
        ...

    @abc.abstractmethod
    def log_summary(self, metrics: Dict[str, Any]):
        ...

    @abc.abstractmethod
    def log_artifact(self, artifact_path, *, name: Optional[str] = None, type: Optional[str] = None):
        ...

    def finish(self):
        pass

    def __enter__(self):
        from . import tracker_fns

        self._ctx = tracker_fns.current_tracker(self)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        self._ctx.__exit__(*exc)


class CompositeTracker(Tracker):
    name = "composite"

    def __init__(self, loggers: List[Tracker]):
        self.loggers = list(loggers)

    def log_hyperparameters(self, hparams):
        for t in self.loggers:
            t.log_hyperparameters(hparams)

    def log(self, metrics, *, step, commit=None):
        for t in self.loggers:
            t.log(metrics, step=step, commit=commit)

    def log_summary(self, metrics):
        for t in self.loggers:
            t.log_summary(metrics)

    def log_artifact(self, artifact_path, *, name=None, type=None):
        for t in self.loggers:
            t.log_artifact(artifact_path, name=name, type=type)

    def finish(self):
        excs = []
        for t in self.loggers:
            try:
                t.finish()
            except Exception as e:  # noqa: BLE001
                excs.append(e)
        if excs:
            raise RuntimeError("Errors occurred when finishing trackers", excs)


class NoopTracker(Tracker):
    name = "noop"

    def log_hyperparameters(self, hparams):
        pass

    def log(self, metrics, *, step, commit=None):
        pass

    def log_summary(self, metrics):
        pass

    def log_artifact(self, artifact_path, *, name=None, type=None):
        pass


class DictTracker(Tracker):
    """Collects everything into ``self.metrics`` (used by tests and by in-step metric capture)."""

    name = "dict"

    def __init__(self):
        self.metrics: Dict[str, Any] = {}
        self.history: List[Dict[str, Any]] = []
        self.hparams: Dict[str, Any] = {}
        self.summary: Dict[str, Any] = {}

    def log_hyperparameters(self, hparams):
        self.hparams.update(hparams)
        self.metrics["hparams"] = self.hparams

    def log(self, metrics, *, step, commit=None):
        self.metrics.update(metrics)
        self.history.append({"step": step, **metrics})

    def log_summary(self, metrics):
        self.summary.update(metrics)
        self.metrics.update(metrics)

    def log_artifact(self, artifact_path, *, name=None, type=None):
        self.metrics.setdefault("artifacts", []).append((str(artifact_path), name, type))


@dataclass
class TrackerConfig(ChoiceRegistry):
    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return "wandb"

    def init(self, run_id: Optional[str]) -> Tracker:
        raise NotImplementedError


@TrackerConfig.register_subclass("noop")
@dataclass
class NoopConfig(TrackerConfig):
    def init(self, run_id: Optional[str]) -> Tracker:
        return NoopTracker()
