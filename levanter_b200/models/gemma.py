"""Gemma 1 / 2 / 3 (src/levanter/models/gemma.py).

``gemma``  : Llama-like decoder with ``gelu_new`` gating, tied embeddings, ``head_dim=256``, embeddings scaled by
             ``sqrt(hidden_dim)`` (:425-426) and ``GemmaRMSNorm`` (fp32, ``(1 + w)`` scaling, zero-initialised weight, :259-291).
``gemma2`` : four norms per layer (pre/post attention, pre/post feed-forward, :599-670) and attention logit soft-capping;
             ``query_pre_attn_scalar`` and ``final_logit_softcapping`` are recorded in the config (and exported to HF) but,
             as in the reference, not applied in the forward/loss path.
``gemma3`` : gemma2 + per-head qk-norm, soft-caps off, ``rope_local_base_freq`` / ``sliding_window_pattern`` recorded but every
             layer is global (:783-799, 859-860)."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, Optional, Type

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..compat.hf_checkpoints import HFCheckpointConverter, HFCompatConfig
from ..layers.attention import Attention, AttentionBackend, AttentionConfig
from ..layers.normalization import LayerNormConfigBase
from ..layers.rotary import rope_config_from_hf, rope_to_hf_dict, DefaultRotaryEmbeddingsConfig, RotaryEmbeddingsConfig
from ..nn import Linear
from ..ops.norm import fused_norm
from ..utils.activation import ActivationFunctionEnum, from_hf_name
from ..utils.flop_utils import lm_flops_per_token
from ..utils.remat import should_recompute
from .llama import LlamaEmbedding, LlamaMlp, _getter
from .lm_model import LmConfig, LmHeadModel


class GemmaRMSNorm(nn.Module):
    """RMSNorm computed in fp32 with ``(1 + weight)`` scaling; the weight starts at zero."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.dim = dim
        self.eps = eps
        self.weight = nn.Parameter(torch.zeros(dim))
        self.weight.lev_shape = (dim,)

    def forward(self, x):
        return fused_norm(x, self.weight, None, self.eps, w_offset=1.0)[0]


@LayerNormConfigBase.register_subclass("gemma")
@dataclass(frozen=True)
class GemmaNormConfig(LayerNormConfigBase):
    def build(self, dim: int):
        assert self.use_weight and not self.use_bias
        return GemmaRMSNorm(dim, eps=self.eps)


@LmConfig.register_subclass("gemma")
@dataclass(frozen=True)
class GemmaConfig(HFCompatConfig):
    activation_function: ActivationFunctionEnum = ActivationFunctionEnum.gelu_new
    initializer_range: float = 0.02
    layer_norm_epsilon: float = 1e-5
    tie_word_embeddings: bool = True
    seq_len: int = 8192
    hidden_dim: int = 2048
    intermediate_dim: int = 16384
    vocab_size: int = 256_000
    num_layers: int = 18
    num_heads: int = 8
    head_dim: int = 256
    num_kv_heads: int = 1
    use_bias: bool = False
    input_embedding_norm: bool = False
    upcast_attn: bool = False
    use_flash_attention: Optional[bool] = None
    attn_backend: Optional[AttentionBackend] = None
    flash_attention_block_size: Optional[int] = None
    rope: RotaryEmbeddingsConfig = dataclasses.field(default_factory=DefaultRotaryEmbeddingsConfig)
    query_pre_attn_scalar: Optional[float] = None
    gradient_checkpointing: bool = True
    scan_layers: bool = True
    cross_entropy_block_size: Optional[int] = None
    reference_checkpoint: str = "google/gemma-2b"

    hf_model_type = "gemma"
    hf_architecture = "GemmaForCausalLM"

    def __post_init__(self):
        assert self.num_heads % self.num_kv_heads == 0

    @property
    def model_type(self) -> Type["GemmaLMHeadModel"]:
        return GemmaLMHeadModel

    def hf_checkpoint_converter(self, ref_checkpoint: Optional[str] = None) -> HFCheckpointConverter:
        return HFCheckpointConverter(self.__class__, reference_checkpoint=ref_checkpoint or self.reference_checkpoint)

    @classmethod
    def _common_from_hf(cls, hf_config) -> dict:
        g = _getter(hf_config)
        act = g("hidden_activation", None) or g("hidden_act", "gelu_pytorch_tanh")
        return dict(seq_len=g("max_position_embeddings"), hidden_dim=g("hidden_size"), intermediate_dim=g("intermediate_size"),
                    num_layers=g("num_hidden_layers"), num_heads=g("num_attention_heads"), num_kv_heads=g("num_key_value_heads"),
                    head_dim=g("head_dim", 256), activation_function=from_hf_name(act) if act in ("gelu_pytorch_tanh",) else ActivationFunctionEnum(act),
                    initializer_range=g("initializer_range", 0.02), layer_norm_epsilon=g("rms_norm_eps", 1e-6),
                    tie_word_embeddings=bool(g("tie_word_embeddings", True)),
                    rope=rope_config_from_hf(g, 10000.0))

    @classmethod
    def from_hf_config(cls, hf_config):
        return cls(**cls._common_from_hf(hf_config))

    def _common_to_hf(self, vocab_size: int) -> dict:
        theta, scaling = self.rope.to_hf_config()
        act = "gelu_pytorch_tanh" if self.activation_function == ActivationFunctionEnum.gelu_new else self.activation_function.value
        return dict(max_position_embeddings=self.seq_len, hidden_size=self.hidden_dim, intermediate_size=self.intermediate_dim,
                    num_hidden_layers=self.num_layers, num_attention_heads=self.num_heads, num_key_value_heads=self.num_kv_heads,
                    head_dim=self.head_dim, hidden_activation=act, hidden_act=act, initializer_range=self.initializer_range,
                    rms_norm_eps=self.layer_norm_epsilon, tie_word_embeddings=self.tie_word_embeddings, vocab_size=vocab_size,
                    rope_theta=theta, rope_scaling=scaling, attention_bias=self.use_bias)

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        cfg = dict(model_type=self.hf_model_type, architectures=[self.hf_architecture], **self._common_to_hf(vocab_size))
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    @property
    def norm_config(self) -> LayerNormConfigBase:
        return GemmaNormConfig(eps=self.layer_norm_epsilon, use_weight=True, use_bias=False)

    def mk_LayerNorm(self, dim: int):
        return self.norm_config.build(dim)

    def attention_config(self) -> AttentionConfig:
        return AttentionConfig(hidden_dim=self.hidden_dim, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                               head_dim=self.head_dim, use_bias=self.use_bias, upcast_attn=self.upcast_attn,
                               attn_backend=self.attn_backend, flash_attention_block_size=self.flash_attention_block_size,
                               rope=self.rope, qk_norm=self.norm_config if getattr(self, "use_qk_norm", False) else None)

    def flops_per_token(self, vocab_size: int):
        return lm_flops_per_token(hidden_dim=self.hidden_dim, intermediate_dim=self.intermediate_dim, num_layers=self.num_layers,
                                  num_kv_heads=self.num_kv_heads, num_heads=self.num_heads, seq_len=self.seq_len,
                                  vocab_size=vocab_size, glu=True)

    def total_trainable_params(self, vocab_size: int) -> int:
        e, hd = self.hidden_dim, self.head_dim
        attn = e * hd * self.num_heads + 2 * e * hd * self.num_kv_heads + hd * self.num_heads * e
        norms = 2 * e
        layer = attn + 3 * e * self.intermediate_dim + norms
        return self.num_layers * layer + e + vocab_size * e * (1 if self.tie_word_embeddings else 2)


class GemmaDecoderLayer(nn.Module):
    """``x + attn(norm(x))`` then ``x + mlp(norm(x))`` (Gemma 1)."""

    def __init__(self, config: GemmaConfig, *, tp=None):
        super().__init__()
        self.config = config
        self.self_attn = Attention(config.attention_config(), init_std=config.initializer_range, tp=tp)
        self.mlp = LlamaMlp(config.hidden_dim, config.intermediate_dim, config.activation_function, use_bias=config.use_bias,
                            init_std=config.initializer_range, tp=tp)
        self.input_layernorm = config.mk_LayerNorm(config.hidden_dim)
        self.post_attention_layernorm = config.mk_LayerNorm(config.hidden_dim)

    def forward(self, x, mask=None, pos_ids=None):
        x = self.self_attn(self.input_layernorm(x), mask, pos_ids, residual=x)
        return self.mlp(self.post_attention_layernorm(x), residual=x)


class Gemma2DecoderLayer(nn.Module):
    """``x + post_attn_norm(attn(pre_attn_norm(x)))`` then ``x + post_ff_norm(mlp(pre_ff_norm(x)))``."""

    def __init__(self, config: "Gemma2Config", *, tp=None):
        super().__init__()
        self.config = config
        self.self_attn = Attention(config.attention_config(), init_std=config.initializer_range, tp=tp)
        self.mlp = LlamaMlp(config.hidden_dim, config.intermediate_dim, config.activation_function, use_bias=config.use_bias,
                            init_std=config.initializer_range, tp=tp)
        self.input_layernorm = config.mk_LayerNorm(config.hidden_dim)
        self.post_attention_layernorm = config.mk_LayerNorm(config.hidden_dim)
        self.pre_feedforward_layernorm = config.mk_LayerNorm(config.hidden_dim)
        self.post_feedforward_layernorm = config.mk_LayerNorm(config.hidden_dim)

    def forward(self, x, mask=None, pos_ids=None):
        x = x + self.post_attention_layernorm(self.self_attn(self.input_layernorm(x), mask, pos_ids))
        return x + self.post_feedforward_layernorm(self.mlp(self.pre_feedforward_layernorm(x)))


class GemmaTransformer(nn.Module):
    def __init__(self, config: GemmaConfig, layer_cls, *, tp=None):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([layer_cls(config, tp=tp) for _ in range(config.num_layers)])
        self.norm = config.mk_LayerNorm(config.hidden_dim)

    def forward(self, x, mask=None, pos_ids=None):
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        for layer in self.layers:
            x = checkpoint(layer, x, mask, pos_ids, use_reentrant=False) if remat else layer(x, mask, pos_ids)
        return self.norm(x)


class GemmaLMHeadModel(LmHeadModel):
    layer_cls = GemmaDecoderLayer

    def __init__(self, vocab_size: int, config: GemmaConfig, *, tp=None):
        super().__init__()
        self.config = config
        self._vocab_size = vocab_size
        self.transformer = GemmaTransformer(config, type(self).layer_cls, tp=tp)
        self.embeddings = LlamaEmbedding(vocab_size, config, norm=config.input_embedding_norm)
        self.lm_head = None if config.tie_word_embeddings else Linear(config.hidden_dim, vocab_size, bias=False,
                                                                      init_std=config.initializer_range)

    @classmethod
    def init(cls, vocab_size: int, config, *, tp=None):
        return cls(vocab_size, config, tp=tp)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def activations(self, input_ids, attn_mask=None, *, pos_ids=None):
        x = self.embeddings.embed(input_ids)
        x = x * torch.tensor(self.config.hidden_dim ** 0.5, dtype=x.dtype, device=x.device)
        return self.transformer(x, attn_mask, pos_ids)

    def get_lm_head(self) -> torch.Tensor:
        return self.embeddings.token_embeddings.weight if self.lm_head is None else self.lm_head.weight

    def resize_vocab(self, new_size: int):
        self.embeddings.token_embeddings = self.embeddings.token_embeddings.resize_embeddings(new_size, self.config.initializer_range)
        if self.lm_head is not None:
            old = self.lm_head
            new = Linear(self.config.hidden_dim, new_size, bias=False, init_std=self.config.initializer_range,
                         device=old.weight.device, dtype=old.weight.dtype)
            n = min(new_size, old.out_features)
            with torch.no_grad():
                new.weight[:n].copy_(old.weight[:n])
            self.lm_head = new
        self._vocab_size = new_size
        return self

    @staticmethod
    def hf_key_map() -> Dict[str, Optional[str]]:
        return {"transformer": "model", "embeddings": None, "token_embeddings": "model.embed_tokens"}


@LmConfig.register_subclass("gemma2")
@dataclass(frozen=True)
class Gemma2Config(GemmaConfig):
    query_pre_attn_scalar: Optional[float] = 256.0
    final_logit_softcapping: Optional[float] = 30.0
    attn_logit_softcapping: Optional[float] = 50.0
    use_qk_norm: bool = False
    sliding_window: Optional[int] = None
    reference_checkpoint: str = "google/gemma-2-2b"

    hf_model_type = "gemma2"
    hf_architecture = "Gemma2ForCausalLM"

    @property
    def model_type(self):
        return Gemma2LMHeadModel

    @classmethod
    def from_hf_config(cls, hf_config):
        g = _getter(hf_config)
        return cls(**cls._common_from_hf(hf_config), query_pre_attn_scalar=g("query_pre_attn_scalar", 256.0),
                   final_logit_softcapping=g("final_logit_softcapping", None), attn_logit_softcapping=g("attn_logit_softcapping", None),
                   sliding_window=g("sliding_window", None))

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        cfg = dict(model_type=self.hf_model_type, architectures=[self.hf_architecture], **self._common_to_hf(vocab_size),
                   query_pre_attn_scalar=_int_if_whole(self.query_pre_attn_scalar or self.head_dim),
                   final_logit_softcapping=self.final_logit_softcapping, attn_logit_softcapping=self.attn_logit_softcapping,
                   sliding_window=self.sliding_window if self.sliding_window is not None else self.seq_len)
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    def attention_config(self) -> AttentionConfig:
        return dataclasses.replace(super().attention_config(), logits_soft_cap=self.attn_logit_softcapping)

    def total_trainable_params(self, vocab_size: int) -> int:
        return super().total_trainable_params(vocab_size) + self.num_layers * 2 * self.hidden_dim


class Gemma2LMHeadModel(GemmaLMHeadModel):
    layer_cls = Gemma2DecoderLayer


def _int_if_whole(x):
    """transformers types this field as an integer and refuses ``256.0``."""
    return int(x) if float(x).is_integer() else x


@LmConfig.register_subclass("gemma3")
@dataclass(frozen=True)
class Gemma3Config(Gemma2Config):
    use_qk_norm: bool = True
    final_logit_softcapping: Optional[float] = None
    attn_logit_softcapping: Optional[float] = None
    sliding_window_pattern: Optional[int] = None
    rope_local_base_freq: float = 10_000.0
    reference_checkpoint: str = "google/gemma-3-1b-pt"

    hf_model_type = "gemma3_text"
    hf_architecture = "Gemma3ForCausalLM"

    @property
    def local_rope(self) -> RotaryEmbeddingsConfig:
        return dataclasses.replace(self.rope, theta=self.rope_local_base_freq)

    @property
    def model_type(self):
        return Gemma3LMHeadModel

    @classmethod
    def from_hf_config(cls, hf_config):
        g = _getter(hf_config)
        return cls(**cls._common_from_hf(hf_config), query_pre_attn_scalar=g("query_pre_attn_scalar", None),
                   final_logit_softcapping=g("final_logit_softcapping", None), attn_logit_softcapping=g("attn_logit_softcapping", None),
                   sliding_window=g("sliding_window", None), sliding_window_pattern=g("sliding_window_pattern", None),
                   rope_local_base_freq=g("rope_local_base_freq", 10000.0), use_qk_norm=True)

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        cfg = super().to_hf_config(vocab_size, None)
        cfg.update(use_qk_norm=self.use_qk_norm, rope_local_base_freq=self.rope_local_base_freq,
                   sliding_window_pattern=self.sliding_window_pattern if self.sliding_window_pattern is not None else 1,
                   attention_dropout=0.0, use_cache=True)
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    def attention_config(self) -> AttentionConfig:
        return dataclasses.replace(super().attention_config(), qk_norm=self.norm_config, logits_soft_cap=self.attn_logit_softcapping)

    def total_trainable_params(self, vocab_size: int) -> int:
        return super().total_trainable_params(vocab_size) + self.num_layers * 2 * self.head_dim


class Gemma3LMHeadModel(GemmaLMHeadModel):
    layer_cls = Gemma2DecoderLayer
