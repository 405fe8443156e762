"""Experiment tracking: a global tracker with pluggable backends (noop, JSON lines, TensorBoard, W&B, trackio)."""
from .tracker import CompositeTracker, DictTracker, NoopConfig, NoopTracker, Tracker, TrackerConfig  # noqa: F401
from .tracker_fns import (current_tracker, defer_tracker_for_jit, get_tracker, jit_log, log, log_configuration,  # noqa: F401
                          log_hyperparameters, log_metrics, log_summary, set_global_tracker)
from .helpers import capture_time, log_optimizer_hyperparams  # noqa: F401
from . import json_logger, tensorboard, wandb, trackio  # noqa: F401  (register their config types)
