"""Low-precision training configuration (the reference's ``haliax.quantization.QuantizationConfig`` reached through
``trainer.quantization``, src/levanter/trainer.py:648, config/gpt2_small_fast_fp8.yaml:17-18).

``fp8: true`` selects fp8 GEMMs for the Linear layers named by ``targets`` (all by default): e4m3 for forward operands,
e5m2 for output gradients.  ``scaling: tensor`` (default) uses one scale per tensor taken from a rolling history of absolute
maxima (delayed scaling, as in the reference); ``scaling: block`` uses one power-of-two scale per 32 values along the
contraction dimension, applied by the tensor core (``tcgen05.mma kind::mxf8f6f4.block_scale``).  ``block_size`` is accepted
for configs that name it; the hardware's block is 32 whatever it says.
``quantize_linear_layers`` swaps matching ``Linear`` modules for ``Fp8Linear``;
master weights, optimizer state and checkpoints are unchanged."""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import List, Optional, Union

import torch
import torch.nn as nn


@dataclass(frozen=True)
class QuantizationConfig:
    targets: Union[None, List[str], str] = None
    amax_history_length: int = 1024
    compute_dtype: Optional[str] = None
    fp8: bool = False
    int8: bool = False
    block_size: int = 128
    scaling: str = "tensor"  # tensor | block

    def __post_init__(self):
        if self.fp8 and self.int8:
            raise ValueError("only one of fp8 / int8 can be enabled")
        if self.scaling not in ("tensor", "block"):
            raise ValueError(f"scaling must be 'tensor' or 'block', got {self.scaling!r}")

    def matches(self, name: str) -> bool:
        if self.targets is None:
            return True
        if isinstance(self.targets, str):
            return re.search(self.targets, name) is not None
        return any(t in name.split(".") or t == name for t in self.targets)


def quantize_linear_layers(model: nn.Module, config: QuantizationConfig) -> nn.Module:
    """Replace targeted ``Linear`` modules by their fp8 counterparts (in place; returns the model)."""
    if not (config.fp8 or config.int8):
        return model
    if config.int8:
        raise NotImplementedError("int8 training is not supported; use fp8")
    from .nn import Linear
    from .ops.fp8 import Fp8Linear

    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if type(child) is Linear and config.matches(full) and "lm_head" not in full:
                setattr(mod, child_name, Fp8Linear.from_linear(child, block=config.block_size, amax_history_length=config.amax_history_length,
                                                                     block_scaled=config.scaling == "block"))
    return model
