"""Activation functions selectable by name in model configs (src/levanter/utils/activation.py:18-40)."""
from __future__ import annotations

import enum
import math

import torch
import torch.nn.functional as F


def _quick_gelu(x):
    return x * torch.sigmoid(1.702 * x)


class ActivationFunctionEnum(str, enum.Enum):
    relu = "relu"
    silu = "silu"
    swish = "swish"
    gelu = "gelu"
    gelu_new = "gelu_new"
    quick_gelu = "quick_gelu"
    tanh = "tanh"

    def to_fn(self):
        return TO_FN[self]


TO_FN = {
    ActivationFunctionEnum.relu: F.relu,
    ActivationFunctionEnum.silu: F.silu,
    ActivationFunctionEnum.swish: F.silu,
    ActivationFunctionEnum.gelu: lambda x: F.gelu(x, approximate="none"),
    ActivationFunctionEnum.gelu_new: lambda x: F.gelu(x, approximate="tanh"),
    ActivationFunctionEnum.quick_gelu: _quick_gelu,
    ActivationFunctionEnum.tanh: torch.tanh,
}

# names used by Hugging Face configs
HF_NAMES = {
    "gelu_pytorch_tanh": ActivationFunctionEnum.gelu_new,
    "gelu_new": ActivationFunctionEnum.gelu_new,
    "gelu": ActivationFunctionEnum.gelu,
    "silu": ActivationFunctionEnum.silu,
    "swish": ActivationFunctionEnum.silu,
    "relu": ActivationFunctionEnum.relu,
    "quick_gelu": ActivationFunctionEnum.quick_gelu,
    "tanh": ActivationFunctionEnum.tanh,
}


def from_hf_name(name: str) -> ActivationFunctionEnum:
    return HF_NAMES[name]
