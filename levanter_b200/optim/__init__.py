"""Optimizers: config registry, composable transformations, and the fused sharded AdamW path."""
from .config import (AdamConfig, HessianOptConfig, LionConfig, LrSchedule, OptimizerConfig, ParamInfo,  # noqa: F401
                     levanter_path)
from .clip_update_norm import ClipUpdateNormConfig  # noqa: F401
from .skipstep import SkipStepConfig  # noqa: F401
from .model_averaging import EmaDecaySqrtConfig, EmaModelAveragingConfig, ModelAveragingConfig  # noqa: F401
