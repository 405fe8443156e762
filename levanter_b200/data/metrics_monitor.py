"""Progress reporting for cache builds (src/levanter/data/metrics_monitor.py:19-90)."""
from __future__ import annotations

import logging as pylogging
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, Optional, Protocol, Union


@dataclass
class InProgressCacheMetrics:
    rows_finished: int = 0
    shards_finished: int = 0
    field_counts: Dict[str, int] = field(default_factory=dict)
    is_finished: bool = False


class MetricsMonitor(Protocol):
    def __call__(self, metrics: InProgressCacheMetrics): ...


class LoggingMetricsMonitor(MetricsMonitor):
    """Sends build progress to the global tracker under ``<prefix>/...``."""

    def __init__(self, prefix: str = "preproc", commit: bool = False):
        self.prefix = prefix
        self.commit = commit
        self.last_metrics = None
        self.last_time = None

    def __call__(self, metrics: InProgressCacheMetrics):
        from .. import tracker

        to_log = {f"{self.prefix}/shards": metrics.shards_finished, f"{self.prefix}/rows": metrics.rows_finished}
        for f_, c in metrics.field_counts.items():
            to_log[f"{self.prefix}/{f_}"] = c
        if metrics.is_finished:
            to_log[f"{self.prefix}/finished"] = 1
        now = time.time()
        if self.last_metrics is not None and now > self.last_time:
            dt = now - self.last_time
            to_log[f"{self.prefix}/rows_per_sec"] = (metrics.rows_finished - self.last_metrics.rows_finished) / dt
        self.last_metrics, self.last_time = metrics, now
        tracker.log(to_log, step=None, commit=self.commit)


class LoggerMetricsMonitor(MetricsMonitor):
    def __init__(self, logger: Optional[Union[pylogging.Logger, str]] = None, level=pylogging.INFO):
        if isinstance(logger, str):
            logger = pylogging.getLogger(logger)
        self.logger = logger or pylogging.getLogger(__name__)
        self.level = level

    def __call__(self, metrics: InProgressCacheMetrics):
        fields = ", ".join(f"{k}: {v}" for k, v in metrics.field_counts.items())
        self.logger.log(self.level, f"done: shards {metrics.shards_finished}, rows {metrics.rows_finished}, {fields}")
        if metrics.is_finished:
            self.logger.info("Cache creation finished")
