"""Rotary position embeddings: default (with linear ``factor``), Llama-3 smoothing, and YaRN.

Frequencies are computed exactly as the reference does (src/levanter/layers/rotary.py:30-46 default,
:97-136 llama3, :186-229 yarn incl. the mscale temperature on cos/sin) with the Hugging Face half-split
``rotate_half`` convention (:17-22).  The cos/sin table is built once per (config, head_dim, length) on
the host side of the model and applied either by the fused CUDA kernel (``ops.rope``) or by PyTorch ops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..config import ChoiceRegistry


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


class RotaryEmbeddings:
    """Callable that rotates ``q`` (``[..., pos, heads..., head_dim]`` with positions given explicitly)."""

    def __init__(self, head_dim: int, inv_freq: torch.Tensor, position_scale: float = 1.0, temperature: float = 1.0):
        self.head_dim = head_dim
        self.inv_freq = inv_freq.float()  # [head_dim // 2]
        self.position_scale = position_scale
        self.temperature = temperature
        self._cache: dict = {}

    def cos_sin(self, position_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos, sin of shape ``position_ids.shape + [head_dim]`` in fp32."""
        inv = self.inv_freq.to(position_ids.device)
        freqs = (position_ids.float() * self.position_scale).unsqueeze(-1) * inv
        emb = torch.cat((freqs, freqs), dim=-1)
        return torch.cos(emb) * self.temperature, torch.sin(emb) * self.temperature

    def table(self, seq_len: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """Cached ``[seq_len, head_dim]`` fp32 cos/sin tables for positions ``0..seq_len-1``."""
        key = (seq_len, str(device))
        if key not in self._cache:
            pos = torch.arange(seq_len, device=device)
            cos, sin = self.cos_sin(pos)
            self._cache[key] = (cos.contiguous(), sin.contiguous())
        return self._cache[key]

    def __call__(self, q: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        """``q``: ``[batch?, pos, heads, head_dim]``; ``position_ids``: ``[pos]`` or ``[batch, pos]``."""
        cos, sin = self.cos_sin(position_ids)
        cos = cos.unsqueeze(-2)
        sin = sin.unsqueeze(-2)
        out = q.float() * cos + rotate_half(q.float()) * sin
        return out.to(q.dtype)


def _base_inv_freq(theta: float, head_dim: int) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


@dataclass(frozen=True)
class RotaryEmbeddingsConfig(ChoiceRegistry):
    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return "default"

    def build(self, head_dim: int) -> RotaryEmbeddings:
        raise NotImplementedError

    @staticmethod
    def from_hf_config(rope_theta: float, config: Optional[dict]) -> "RotaryEmbeddingsConfig":
        if config is None:
            return DefaultRotaryEmbeddingsConfig(theta=rope_theta)
        tpe = config.get("rope_type", config.get("type", "default"))
        if tpe in ("default", "linear"):
            return DefaultRotaryEmbeddingsConfig(theta=rope_theta, factor=float(config.get("factor", 1.0)))
        if tpe == "llama3":
            return Llama3RotaryEmbeddingsConfig.make_from_hf_config(rope_theta, config)
        if tpe == "yarn":
            return YarnRotaryEmbeddingsConfig.make_from_hf_config(rope_theta, config)
        raise ValueError(f"unknown rope scaling type {tpe}")

    def to_hf_config(self) -> Tuple[float, Optional[dict]]:
        raise NotImplementedError


@RotaryEmbeddingsConfig.register_subclass("default")
@dataclass(frozen=True)
class DefaultRotaryEmbeddingsConfig(RotaryEmbeddingsConfig):
    theta: float = 10000
    factor: float = 1.0

    def build(self, head_dim: int) -> RotaryEmbeddings:
        return RotaryEmbeddings(head_dim, _base_inv_freq(self.theta, head_dim) / self.factor)

    def to_hf_config(self):
        if self.factor == 1.0:
            return self.theta, None
        return self.theta, {"rope_type": "linear", "factor": self.factor}


RotaryEmbeddingsConfig.register_subclass("linear")(DefaultRotaryEmbeddingsConfig)
DefaultRotaryEmbeddingsConfig._choice_name = "default"


@RotaryEmbeddingsConfig.register_subclass("llama3")
@dataclass(frozen=True)
class Llama3RotaryEmbeddingsConfig(RotaryEmbeddingsConfig):
    theta: float = 500000
    factor: float = 8.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    def build(self, head_dim: int) -> RotaryEmbeddings:
        inv_freq = _base_inv_freq(self.theta, head_dim)
        old = self.original_max_position_embeddings
        low_wavelen = old / self.low_freq_factor
        high_wavelen = old / self.high_freq_factor
        wavelen = 2 * math.pi / inv_freq
        inv_llama = torch.where(wavelen > low_wavelen, inv_freq / self.factor, inv_freq)
        smooth = (old / wavelen - self.low_freq_factor) / (self.high_freq_factor - self.low_freq_factor)
        smoothed = (1 - smooth) * inv_llama / self.factor + smooth * inv_llama
        medium = (~(wavelen < high_wavelen)) & (~(wavelen > low_wavelen))
        inv_llama = torch.where(medium, smoothed, inv_llama)
        return RotaryEmbeddings(head_dim, inv_llama)

    @classmethod
    def make_from_hf_config(cls, rope_theta: float, config: dict):
        return cls(theta=rope_theta, factor=float(config.get("factor", 8.0)),
                   low_freq_factor=float(config.get("low_freq_factor", 1.0)),
                   high_freq_factor=float(config.get("high_freq_factor", 4.0)),
                   original_max_position_embeddings=int(config.get("original_max_position_embeddings", 8192)))

    def to_hf_config(self):
        return self.theta, {"rope_type": "llama3", "factor": self.factor, "low_freq_factor": self.low_freq_factor,
                            "high_freq_factor": self.high_freq_factor,
                            "original_max_position_embeddings": self.original_max_position_embeddings}


@RotaryEmbeddingsConfig.register_subclass("yarn")
@dataclass(frozen=True)
class YarnRotaryEmbeddingsConfig(RotaryEmbeddingsConfig):
    theta: float = 10000
    factor: float = 1.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    original_max_position_embeddings: int = 2048
    mscale: float = 1.0

    def build(self, head_dim: int) -> RotaryEmbeddings:
        half = head_dim // 2
        inv_freq = _base_inv_freq(self.theta, head_dim)

        def find_dim(n_rot: float) -> float:
            return (half * math.log(self.original_max_position_embeddings / (n_rot * 2 * math.pi))) / (2 * math.log(self.theta))

        low = int(math.floor(find_dim(self.beta_fast)))
        high = int(math.ceil(find_dim(self.beta_slow)))
        low, high = max(low, 0), min(high, half - 1)
        ramp = torch.clamp((torch.arange(half, dtype=torch.float32) - low) / max(high - low, 1), 0.0, 1.0)
        inv = (inv_freq / self.factor) * ramp + inv_freq * (1 - ramp)
        temperature = 1.0 if self.factor < 1.0 else math.sqrt(0.1 * self.mscale * math.log(self.factor) + 1.0)
        return RotaryEmbeddings(head_dim, inv, position_scale=1.0 / self.factor, temperature=temperature)

    @classmethod
    def make_from_hf_config(cls, rope_theta: float, config: dict):
        return cls(theta=rope_theta, factor=float(config.get("factor", 1.0)), beta_fast=float(config.get("beta_fast", 32.0)),
                   beta_slow=float(config.get("beta_slow", 1.0)),
                   original_max_position_embeddings=int(config.get("original_max_position_embeddings", 2048)),
                   mscale=float(config.get("mscale", 1.0)))

    def to_hf_config(self):
        return self.theta, {"type": "yarn", "factor": self.factor, "beta_fast": self.beta_fast, "beta_slow": self.beta_slow,
                            "original_max_position_embeddings": self.original_max_position_embeddings, "mscale": self.mscale}


def rope_config_from_hf(get, default_theta: float = 10000.0) -> RotaryEmbeddingsConfig:
    """RoPE config from an HF config accessor ``get(key, default)``: understands both the legacy ``rope_theta`` +
    ``rope_scaling`` keys and the merged ``rope_parameters`` dict of newer ``transformers`` releases."""
    params = get("rope_parameters", None)
    theta = get("rope_theta", None)
    scaling = get("rope_scaling", None)
    if isinstance(params, dict):
        if "rope_theta" not in params and any(isinstance(v, dict) for v in params.values()):
            # per-layer-type parameters (e.g. full_attention / sliding_attention): take the global one
            params = params.get("full_attention") or next(v for v in params.values() if isinstance(v, dict))
        theta = params.get("rope_theta", theta)
        if params.get("rope_type", params.get("type", "default")) != "default":
            scaling = {k: v for k, v in params.items() if k != "rope_theta"}
    if theta is None:
        theta = default_theta
    return RotaryEmbeddingsConfig.from_hf_config(float(theta), scaling)


def rope_to_hf_dict(rope: RotaryEmbeddingsConfig) -> dict:
    """Keys to merge into an HF config for ``rope``: legacy (``rope_theta``, ``rope_scaling``) and ``rope_parameters``."""
    theta, scaling = rope.to_hf_config()
    params = {"rope_theta": theta, "rope_type": "default"}
    if scaling:
        params.update(scaling)
        params["rope_type"] = scaling.get("rope_type", scaling.get("type", "default"))
        params.pop("type", None)
    return {"rope_theta": theta, "rope_scaling": scaling, "rope_parameters": params}
