"""TensorBoard tracker (src/levanter/tracker/tensorboard.py:28-128): scalars, histograms, text hyperparameters;
writes to ``<logdir>/<run_id>``."""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional

import numpy as np

from .tracker import Tracker, TrackerConfig

pylogger = logging.getLogger(__name__)


class TensorboardTracker(Tracker):
    name = "tensorboard"

    def __init__(self, writer):
        self.writer = writer

    def log_hyperparameters(self, hparams: Dict[str, Any]):
        for k, v in _flatten(hparams).items():
            try:
                self.writer.add_text(f"config/{k}", str(v))
            except Exception:
                pylogger.exception(f"Error logging {k}")

    def log(self, metrics, *, step, commit=None):
        del commit
        from .histogram import Histogram

        for k, v in _flatten(metrics).items():
            if isinstance(v, Histogram):
                try:
                    counts = np.asarray(v.bucket_counts, dtype=np.float64)
                    limits = np.asarray(v.bucket_limits, dtype=np.float64)
                    self.writer.add_histogram_raw(
                        k, min=float(v.min), max=float(v.max), num=int(v.num), sum=float(v.sum),
                        sum_squares=float(v.sum_squares), bucket_limits=limits[1:].tolist(), bucket_counts=counts.tolist(),
                        global_step=step)
                except Exception:
                    pylogger.exception(f"Error logging histogram {k}")
            elif isinstance(v, str):
                self.writer.add_text(k, v, global_step=step)
            else:
                try:
                    self.writer.add_scalar(k, float(v), global_step=step)
                except (TypeError, ValueError):
                    try:
                        self.writer.add_histogram(k, np.asarray(v), global_step=step)
                    except Exception:
                        pylogger.exception(f"Error logging {k}")

    def log_summary(self, metrics):
        for k, v in _flatten(metrics).items():
            try:
                self.writer.add_scalar(f"summary/{k}", float(v), global_step=None)
            except Exception:
                self.writer.add_text(f"summary/{k}", str(v))

    def log_artifact(self, artifact_path, *, name=None, type=None):
        log_path = self.writer.log_dir
        import shutil

        dest = os.path.join(log_path, "artifacts", name or os.path.basename(str(artifact_path)))
        os.makedirs(os.path.dirname(dest), exist_ok=True)
        try:
            if os.path.isdir(artifact_path):
                shutil.copytree(artifact_path, dest, dirs_exist_ok=True)
            else:
                shutil.copy(artifact_path, dest)
        except Exception:
            pylogger.exception(f"Error logging artifact {artifact_path}")

    def finish(self):
        self.writer.close()


def _flatten(d, prefix=""):
    out = {}
    for k, v in d.items():
        key = f"{prefix}/{k}" if prefix else str(k)
        if isinstance(v, dict):
            out.update(_flatten(v, key))
        else:
            out[key] = v
    return out


@TrackerConfig.register_subclass("tensorboard")
@dataclass
class TensorboardConfig(TrackerConfig):
    logdir: str = "tblogs"
    comment: Optional[str] = ""
    purge_step: Optional[int] = None
    max_queue: Optional[int] = 10
    flush_secs: Optional[int] = 120
    filename_suffix: Optional[str] = ""
    write_to_disk: Optional[bool] = True

    def init(self, run_id: Optional[str]) -> TensorboardTracker:
        from torch.utils.tensorboard import SummaryWriter

        dir_to_write = self.logdir if run_id is None else os.path.join(self.logdir, run_id)
        pylogger.info(f"Writing Tensorboard logs to {dir_to_write}")
        writer = SummaryWriter(dir_to_write, comment=self.comment or "", purge_step=self.purge_step, max_queue=self.max_queue or 10,
                               flush_secs=self.flush_secs or 120, filename_suffix=self.filename_suffix or "")
        return TensorboardTracker(writer)
