"""Qwen2 and Qwen3 (src/levanter/models/qwen.py).

``qwen``: Llama with biases on q/k/v only (o_proj and MLP unbiased, :125-138).  A sliding window that would actually
take effect raises ``NotImplementedError`` like the reference (:173-176).
``qwen3``: Llama plus per-head RMSNorm on q and k before RoPE (:374-376) and an explicit ``head_dim``."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, Optional, Type

from ..layers.attention import Attention, AttentionConfig
from ..layers.rotary import rope_config_from_hf, rope_to_hf_dict, RotaryEmbeddingsConfig
from ..utils.activation import ActivationFunctionEnum
from .llama import LlamaConfig, LlamaDecoderLayer, LlamaLMHeadModel, _getter
from .lm_model import LmConfig


@LmConfig.register_subclass("qwen")
@dataclass(frozen=True)
class QwenConfig(LlamaConfig):
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    reference_checkpoint: str = "Qwen/Qwen2.5-0.5B"

    hf_model_type = "qwen2"
    hf_architecture = "Qwen2ForCausalLM"

    @property
    def model_type(self) -> Type["QwenLMHeadModel"]:
        return QwenLMHeadModel

    @classmethod
    def from_hf_config(cls, hf_config) -> "QwenConfig":
        g = _getter(hf_config)
        return cls(seq_len=g("max_position_embeddings"), hidden_dim=g("hidden_size"), intermediate_dim=g("intermediate_size"),
                   num_layers=g("num_hidden_layers"), num_heads=g("num_attention_heads"), num_kv_heads=g("num_key_value_heads"),
                   use_sliding_window=bool(g("use_sliding_window", False)), sliding_window=g("sliding_window", None),
                   max_window_layers=g("max_window_layers", 0) or 0,
                   activation_function=ActivationFunctionEnum(g("hidden_act", "silu")),
                   initializer_range=g("initializer_range", 0.02), layer_norm_epsilon=g("rms_norm_eps", 1e-6),
                   tie_word_embeddings=bool(g("tie_word_embeddings", False)),
                   rope=rope_config_from_hf(g, 10000.0))

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        theta, scaling = self.rope.to_hf_config()
        cfg = dict(model_type="qwen2", architectures=["Qwen2ForCausalLM"], max_position_embeddings=self.seq_len,
                   hidden_size=self.hidden_dim, intermediate_size=self.intermediate_dim, num_hidden_layers=self.num_layers,
                   num_attention_heads=self.num_heads, num_key_value_heads=self.num_kv_heads,
                   use_sliding_window=self.use_sliding_window, sliding_window=self.sliding_window,
                   max_window_layers=self.max_window_layers, hidden_act=self.activation_function.name,
                   initializer_range=self.initializer_range, rms_norm_eps=self.layer_norm_epsilon,
                   tie_word_embeddings=self.tie_word_embeddings, vocab_size=vocab_size, rope_theta=theta, rope_scaling=scaling)
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    def attention_config(self) -> AttentionConfig:
        cfg = super().attention_config()
        return dataclasses.replace(cfg, use_bias=True, use_output_bias=False)

    def total_trainable_params(self, vocab_size):
        hs = self.actual_head_size
        qkv_biases = hs * (self.num_heads + 2 * self.num_kv_heads)
        return super().total_trainable_params(vocab_size) + self.num_layers * qkv_biases


class QwenDecoderLayer(LlamaDecoderLayer):
    def __init__(self, config: QwenConfig, *, tp=None, layer_idx: int = 0):
        super().__init__(config, tp=tp)
        self.layer_idx = layer_idx

    def forward(self, x, mask=None, pos_ids=None):
        c = self.config
        if c.use_sliding_window and c.sliding_window is not None and self.layer_idx >= c.max_window_layers \
                and x.shape[-2] > c.sliding_window:
            raise NotImplementedError("Sliding window attention is not supported for Qwen2 layers")
        return super().forward(x, mask, pos_ids)


class QwenLMHeadModel(LlamaLMHeadModel):
    def __init__(self, vocab_size: int, config: QwenConfig, *, tp=None, **kw):
        counter = iter(range(10**9))
        super().__init__(vocab_size, config, tp=tp, layer_cls=lambda cfg, tp=None: QwenDecoderLayer(cfg, tp=tp, layer_idx=next(counter)))


@LmConfig.register_subclass("qwen3")
@dataclass(frozen=True)
class Qwen3Config(LlamaConfig):
    use_sliding_window: bool = False
    sliding_window: int = 4096
    reference_checkpoint: str = "Qwen/Qwen3-0.6B"

    hf_model_type = "qwen3"
    hf_architecture = "Qwen3ForCausalLM"

    @property
    def model_type(self) -> Type["Qwen3LMHeadModel"]:
        return Qwen3LMHeadModel

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        theta, scaling = self.rope.to_hf_config()
        cfg = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], max_position_embeddings=self.seq_len,
                   hidden_size=self.hidden_dim, intermediate_size=self.intermediate_dim, num_hidden_layers=self.num_layers,
                   num_attention_heads=self.num_heads, num_key_value_heads=self.num_kv_heads, sliding_window=self.sliding_window,
                   use_sliding_window=self.use_sliding_window, hidden_act=self.activation_function.name,
                   initializer_range=self.initializer_range, rms_norm_eps=self.layer_norm_epsilon,
                   tie_word_embeddings=self.tie_word_embeddings, vocab_size=vocab_size, rope_theta=theta, rope_scaling=scaling,
                   attention_bias=self.use_bias, head_dim=self.head_dim or self.hidden_dim // self.num_heads)
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    @classmethod
    def from_hf_config(cls, hf_config) -> "Qwen3Config":
        g = _getter(hf_config)
        return cls(seq_len=g("max_position_embeddings"), hidden_dim=g("hidden_size"), intermediate_dim=g("intermediate_size"),
                   num_layers=g("num_hidden_layers"), num_heads=g("num_attention_heads"), num_kv_heads=g("num_key_value_heads"),
                   sliding_window=g("sliding_window", 4096) or 4096, use_sliding_window=bool(g("use_sliding_window", True)),
                   activation_function=ActivationFunctionEnum(g("hidden_act", "silu")),
                   initializer_range=g("initializer_range", 0.02), layer_norm_epsilon=g("rms_norm_eps", 1e-6),
                   tie_word_embeddings=bool(g("tie_word_embeddings", False)),
                   rope=rope_config_from_hf(g, 10000.0),
                   use_bias=bool(g("attention_bias", False)), head_dim=g("head_dim", None))

    def attention_config(self) -> AttentionConfig:
        cfg = super().attention_config()
        return dataclasses.replace(cfg, qk_norm=self.norm_config)

    def total_trainable_params(self, vocab_size):
        hs = self.actual_head_size
        biases = hs * (2 * self.num_heads + 2 * self.num_kv_heads) if self.use_bias else 0
        return super().total_trainable_params(vocab_size) + self.num_layers * (2 * hs + biases)  # q and k norms per layer


class Qwen3LMHeadModel(LlamaLMHeadModel):
    pass
