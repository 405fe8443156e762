"""FLOP accounting and device peak table for MFU.

``lm_flops_per_token`` follows the reference's definition exactly (forward FLOPs with a full S^2 attention
map; src/levanter/utils/flop_utils.py:10-38) so MFU figures stay comparable.  The reference's peak table has
no Blackwell entry (src/levanter/utils/flop_utils.py:43-185); this one adds B200 dense figures.
"""
from __future__ import annotations

from typing import Optional

import torch


def lm_flops_per_token(hidden_dim: int, intermediate_dim: int, num_layers: int, num_kv_heads: int, num_heads: int,
                       seq_len: int, vocab_size: int, glu: bool, num_experts: int = 1, num_shared_experts: int = 0,
                       num_experts_per_tok: int = 1) -> float:
    head_dim = hidden_dim / num_heads
    mlp = 2 * (3 if glu else 2) * hidden_dim * intermediate_dim * (num_experts_per_tok + num_shared_experts)
    if num_experts > 1:
        mlp += 2 * hidden_dim * num_experts
    qkv_proj = 2 * hidden_dim * (num_heads * head_dim + 2 * num_kv_heads * head_dim)
    dense_proj = 2 * hidden_dim * hidden_dim
    key_query_logits = 2 * seq_len**2 * num_heads * head_dim
    mask = 3 * seq_len * seq_len * num_heads
    mask_value = 2 * seq_len * seq_len * head_dim * num_heads
    attn = (key_query_logits + mask + mask_value) / seq_len
    lm_head = 2 * hidden_dim * vocab_size
    return num_layers * (mlp + qkv_proj + dense_proj + attn) + lm_head


# dense (no 2:4 sparsity) peak FLOP/s per device
DEVICE_AVAILABLE_FLOPS = {
    "b200": {"fp8": 4.5e15, "bf16": 2.25e15, "fp16": 2.25e15, "tf32": 1.1e15, "fp32": 8.0e13, "fp4": 9.0e15},
    "gb200": {"fp8": 5.0e15, "bf16": 2.5e15, "fp16": 2.5e15, "tf32": 1.25e15, "fp32": 9.0e13},
    "h200": {"fp8": 1.979e15, "bf16": 9.895e14, "fp16": 9.895e14, "tf32": 4.945e14, "fp32": 6.7e13},
    "h100-sxm": {"fp8": 1.979e15, "bf16": 9.895e14, "fp16": 9.895e14, "tf32": 4.945e14, "fp32": 6.7e13},
    "h100-pcie": {"fp8": 1.513e15, "bf16": 7.565e14, "fp16": 7.565e14, "tf32": 3.78e14, "fp32": 5.1e13},
    "a100": {"bf16": 3.12e14, "fp16": 3.12e14, "tf32": 1.56e14, "fp32": 1.95e13},
    "a10": {"bf16": 1.25e14, "fp16": 1.25e14, "tf32": 6.25e13, "fp32": 3.12e13},
    "v100-sxm": {"fp16": 1.25e14, "fp32": 1.57e13},
    "t4": {"fp16": 6.5e13, "fp32": 8.1e12},
    "l4": {"bf16": 1.21e14, "fp16": 1.21e14, "fp32": 3.03e13},
    "rtx 3090": {"bf16": 7.1e13, "fp16": 7.1e13, "fp32": 3.56e13},
    "rtx 4090": {"bf16": 1.65e14, "fp16": 1.65e14, "fp32": 8.26e13},
    "cpu": {"fp32": 1.0e11, "bf16": 1.0e11},
}


def _dtype_key(dtype) -> str:
    s = str(dtype).replace("torch.", "")
    return {"bfloat16": "bf16", "float16": "fp16", "float32": "fp32", "float8_e4m3fn": "fp8", "float8_e5m2": "fp8"}.get(s, s)


def device_hardware_flops(device: Optional[torch.device] = None, dtype=torch.bfloat16) -> Optional[float]:
    """Peak dense FLOP/s of the device for ``dtype`` (None when unknown)."""
    if device is None:
        device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    kind = device_kind(device)
    key = _dtype_key(dtype)
    for name, table in DEVICE_AVAILABLE_FLOPS.items():
        if name in kind:
            return table.get(key) or (table.get("tf32") if key == "fp32" else None)
    return None


def device_kind(device: Optional[torch.device] = None) -> str:
    if device is None:
        device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda" and torch.cuda.is_available():
        return torch.cuda.get_device_name(device).lower()
    return "cpu"
