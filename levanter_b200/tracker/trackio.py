"""trackio tracker (src/levanter/tracker/trackio.py:26-146); only process 0 logs."""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

from .tracker import NoopTracker, Tracker, TrackerConfig

logger = logging.getLogger(__name__)


class TrackioTracker(Tracker):
    name = "trackio"

    def __init__(self, run):
        self.run = run
        self._trackio = None
        try:
            import trackio

            self._trackio = trackio
        except ImportError:
            pass

    def log_hyperparameters(self, hparams: Dict[str, Any]):
        if hasattr(self.run, "config") and isinstance(getattr(self.run, "config"), dict):
            self.run.config.update(hparams)

    def log(self, metrics, *, step, commit=None):
        payload = {}
        for k, v in metrics.items():
            try:
                payload[k] = float(v)
            except (TypeError, ValueError):
                payload[k] = str(v)
        if self._trackio is not None:
            self._trackio.log(payload, step=step)
        elif hasattr(self.run, "log"):
            self.run.log(payload, step=step)

    def log_summary(self, metrics):
        self.log({f"summary/{k}": v for k, v in metrics.items()}, step=None)

    def log_artifact(self, artifact_path, *, name=None, type=None):
        logger.info(f"trackio does not store artifacts; skipping {artifact_path}")

    def finish(self):
        if self._trackio is not None:
            self._trackio.finish()
        elif hasattr(self.run, "finish"):
            self.run.finish()


@TrackerConfig.register_subclass("trackio")
@dataclass
class TrackioConfig(TrackerConfig):
    project: str = "levanter"
    name: Optional[str] = None
    space_id: Optional[str] = None
    dataset_id: Optional[str] = None
    config: Optional[Dict[str, Any]] = None
    mode: Optional[str] = None
    resume: str = "auto"

    def init(self, run_id: Optional[str]) -> Tracker:
        if int(os.environ.get("RANK", "0")) != 0 or self.mode == "disabled":
            return NoopTracker()
        import trackio

        run = trackio.init(project=self.project, name=self.name or run_id, space_id=self.space_id, dataset_id=self.dataset_id,
                           config=self.config, resume=self.resume)
        return TrackioTracker(run)
