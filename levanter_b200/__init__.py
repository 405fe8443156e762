"""levanter_b200: an LLM training and inference framework for NVIDIA B200 (PyTorch + hand-written sm_100a CUDA kernels +
NCCL / NVLink), with the capabilities and public surface of Levanter (src/levanter/__init__.py)."""
from . import (analysis, callbacks, checkpoint, config, data, distributed, layers, models, optim, parallel, tracker,  # noqa: F401
               trainer, utils)
from .tracker import current_tracker, get_tracker  # noqa: F401
from .trainer import initialize  # noqa: F401

__version__ = "0.1.0"
