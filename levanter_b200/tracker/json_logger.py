"""JSON-lines tracker: one JSON object per event through Python logging (src/levanter/tracker/json_logger.py:52-123)."""
from __future__ import annotations

import json
import logging
from dataclasses import dataclass
from typing import Any, Dict, Optional

from ..utils.json_utils import ConfigJSONEncoder
from .tracker import Tracker, TrackerConfig


class JsonLoggerTracker(Tracker):
    name = "json_logger"

    def __init__(self, logger: logging.Logger):
        self.logger = logger
        self._last_metrics: Dict[str, Any] = {}

    def _emit(self, event: str, **payload):
        self.logger.info(json.dumps({"event": event, **payload}, cls=ConfigJSONEncoder, default=str))

    def log_hyperparameters(self, hparams):
        self._emit("hparams", data=hparams)

    def log(self, metrics, *, step, commit=None):
        self._last_metrics.update(metrics)
        self._emit("log", step=step, metrics={k: (v.tolist() if hasattr(v, "tolist") else v) for k, v in metrics.items()})

    def log_summary(self, metrics):
        self._last_metrics.update(metrics)
        self._emit("summary", metrics=metrics)

    def log_artifact(self, artifact_path, *, name=None, type=None):
        self._emit("artifact", path=str(artifact_path), name=name, artifact_type=type)

    def finish(self):
        self._emit("finish", summary={k: (v.tolist() if hasattr(v, "tolist") else v) for k, v in self._last_metrics.items()})


@TrackerConfig.register_subclass("json_logger")
@dataclass
class JsonLoggerConfig(TrackerConfig):
    logger_name: str = "levanter.json_logger"
    level: int = logging.INFO

    def init(self, run_id: Optional[str]) -> Tracker:
        logger = logging.getLogger(self.logger_name)
        logger.setLevel(self.level)
        return JsonLoggerTracker(logger)
