"""Mistral (src/levanter/models/mistral.py): the Llama transformer with GQA defaults (8 KV heads, intermediate 14336,
seq 8192) and an always-untied LM head.

``sliding_window`` is a config field that the reference records but does not pass to its attention module
(:161-172), so reference training is fully causal; ``apply_sliding_window: true`` here opts in to windowed attention
(the flash kernel skips key blocks left of the window)."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, Optional, Type

from ..compat.hf_checkpoints import HFCheckpointConverter
from ..layers.attention import AttentionBackend, AttentionConfig
from ..layers.rotary import rope_config_from_hf, rope_to_hf_dict, DefaultRotaryEmbeddingsConfig, RotaryEmbeddingsConfig
from ..utils.activation import ActivationFunctionEnum
from ..utils.flop_utils import lm_flops_per_token
from .llama import LlamaConfig, LlamaLMHeadModel, _getter
from .lm_model import LmConfig


@LmConfig.register_subclass("mistral")
@dataclass(frozen=True)
class MistralConfig(LlamaConfig):
    seq_len: int = 8192
    hidden_dim: int = 4096
    intermediate_dim: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    layer_norm_epsilon: float = 1e-6
    sliding_window: int = 4096
    apply_sliding_window: bool = False
    use_flash_attention: Optional[bool] = True
    reference_checkpoint: str = "mistralai/Mistral-7B-v0.1"

    hf_model_type = "mistral"
    hf_architecture = "MistralForCausalLM"

    @property
    def model_type(self) -> Type["MistralLMHeadModel"]:
        return MistralLMHeadModel

    @classmethod
    def from_hf_config(cls, hf_config) -> "MistralConfig":
        g = _getter(hf_config)
        return cls(seq_len=g("max_position_embeddings"), hidden_dim=g("hidden_size"), intermediate_dim=g("intermediate_size"),
                   num_layers=g("num_hidden_layers"), num_heads=g("num_attention_heads"),
                   num_kv_heads=g("num_key_value_heads", g("num_attention_heads")),
                   activation_function=ActivationFunctionEnum(g("hidden_act", "silu")),
                   initializer_range=g("initializer_range", 0.02), layer_norm_epsilon=g("rms_norm_eps", 1e-6),
                   sliding_window=g("sliding_window", 4096) or 4096,
                   rope=rope_config_from_hf(g, 10000.0))

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        theta, _ = self.rope.to_hf_config()
        cfg = dict(model_type="mistral", architectures=["MistralForCausalLM"], max_position_embeddings=self.seq_len,
                   hidden_size=self.hidden_dim, intermediate_size=self.intermediate_dim, num_hidden_layers=self.num_layers,
                   num_attention_heads=self.num_heads, num_key_value_heads=self.num_kv_heads,
                   hidden_act=self.activation_function.name, initializer_range=self.initializer_range,
                   rms_norm_eps=self.layer_norm_epsilon, sliding_window=self.sliding_window, vocab_size=vocab_size,
                   rope_theta=theta, tie_word_embeddings=False)
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    def attention_config(self) -> AttentionConfig:
        cfg = super().attention_config()
        if self.apply_sliding_window:
            cfg = dataclasses.replace(cfg, sliding_window=self.sliding_window)
        return cfg

    def flops_per_token(self, vocab_size: int):
        # the reference counts Mistral with glu=False and num_kv_heads=num_heads (src/levanter/models/mistral.py:149-159)
        return lm_flops_per_token(hidden_dim=self.hidden_dim, intermediate_dim=self.intermediate_dim, num_layers=self.num_layers,
                                  num_kv_heads=self.num_heads, num_heads=self.num_heads, seq_len=self.seq_len,
                                  vocab_size=vocab_size, glu=False)


class MistralLMHeadModel(LlamaLMHeadModel):
    def __init__(self, vocab_size: int, config: MistralConfig, **kw):
        if config.tie_word_embeddings:
            config = dataclasses.replace(config, tie_word_embeddings=False)
        super().__init__(vocab_size, config, **kw)
