"""Optimizers: config registry, composable transformations, and the fused sharded AdamW path."""
from .config import (AdamConfig, HessianOptConfig, LionConfig, LrSchedule, OptimizerConfig, ParamInfo,  # noqa: F401
                     levanter_path)
from .clip_update_norm import ClipUpdateNormConfig  # noqa: F401
from .skipstep import SkipStepConfig  # noqa: F401
from .model_averaging import EmaDecaySqrtConfig, EmaModelAveragingConfig, ModelAveragingConfig  # noqa: F401
from .adopt import AdoptConfig  # noqa: F401
from .cautious import CautiousConfig  # noqa: F401
from .mars import MarsConfig  # noqa: F401
from .rmsprop import RMSPropMomentumConfig  # noqa: F401
from .muon import MuonConfig  # noqa: F401
from .scion import ScionConfig  # noqa: F401
from .adam_mini import MiniConfig  # noqa: F401
from .sophia import SophiaHConfig  # noqa: F401
from .soap import SoapConfig  # noqa: F401
from .kron import KronConfig  # noqa: F401
