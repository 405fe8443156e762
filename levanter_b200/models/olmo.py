"""OLMo-2 (src/levanter/models/olmo.py): post-norm residual blocks ``x + norm(attn(x))`` / ``h + norm(mlp(h))`` (:406-422),
RMSNorm on the *whole* projected q and k (all heads together, before the head split, :312-314,327-333), SwiGLU MLP,
untied head by default."""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass
from typing import Dict, Optional, Type

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..compat.hf_checkpoints import HFCheckpointConverter, HFCompatConfig
from ..layers.attention import AttentionBackend, AttentionMask, dot_product_attention
from ..layers.normalization import LayerNormConfigBase, RmsNormConfig
from ..layers.rotary import rope_config_from_hf, rope_to_hf_dict, DefaultRotaryEmbeddingsConfig, RotaryEmbeddingsConfig
from ..nn import Dropout, Linear
from ..ops import rope as rope_op
from ..utils.activation import ActivationFunctionEnum
from ..utils.flop_utils import lm_flops_per_token
from ..utils.remat import should_recompute
from .llama import LlamaEmbedding, LlamaMlp, _getter
from .lm_model import LmConfig, LmHeadModel


@LmConfig.register_subclass("olmo2")
@dataclass(frozen=True)
class Olmo2Config(HFCompatConfig):
    seq_len: int = 4096
    hidden_dim: int = 4096
    intermediate_dim: int = 11008
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    activation_function: ActivationFunctionEnum = ActivationFunctionEnum.silu
    initializer_range: float = 0.02
    layer_norm_epsilon: float = 1e-6
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    attention_dropout: float = 0.0
    upcast_attn: bool = False
    use_flash_attention: Optional[bool] = True
    attn_backend: Optional[AttentionBackend] = None
    flash_attention_block_size: Optional[int] = None
    gradient_checkpointing: bool = True
    scan_layers: bool = True
    use_bias: bool = False
    use_layer_norm_weight: bool = True
    rope: RotaryEmbeddingsConfig = dataclasses.field(default_factory=DefaultRotaryEmbeddingsConfig)
    reference_checkpoint: str = "allenai/OLMo-2-1124-7B"
    tokenizer: Optional[str] = None
    cross_entropy_block_size: Optional[int] = None
    input_embedding_norm: bool = False

    hf_model_type = "olmo2"
    hf_architecture = "Olmo2ForCausalLM"

    def __post_init__(self):
        assert self.num_heads % self.num_kv_heads == 0

    @property
    def model_type(self) -> Type["Olmo2LMHeadModel"]:
        return Olmo2LMHeadModel

    @property
    def head_size(self) -> int:
        return self.hidden_dim // self.num_heads

    def hf_checkpoint_converter(self, ref_checkpoint: Optional[str] = None) -> HFCheckpointConverter:
        return HFCheckpointConverter(self.__class__, reference_checkpoint=ref_checkpoint or self.reference_checkpoint,
                                     tokenizer=ref_checkpoint if self.tokenizer is None else self.tokenizer)

    @classmethod
    def from_hf_config(cls, hf_config) -> "Olmo2Config":
        g = _getter(hf_config)
        return cls(seq_len=g("max_position_embeddings"), hidden_dim=g("hidden_size"), intermediate_dim=g("intermediate_size"),
                   num_layers=g("num_hidden_layers"), num_heads=g("num_attention_heads"),
                   num_kv_heads=g("num_key_value_heads", g("num_attention_heads")),
                   activation_function=ActivationFunctionEnum(g("hidden_act", "silu")),
                   initializer_range=g("initializer_range", 0.02), layer_norm_epsilon=g("rms_norm_eps", 1e-6),
                   tie_word_embeddings=bool(g("tie_word_embeddings", False)), attention_bias=bool(g("attention_bias", False)),
                   attention_dropout=g("attention_dropout", 0.0),
                   rope=rope_config_from_hf(g, 500000.0))

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        theta, scaling = self.rope.to_hf_config()
        cfg = dict(model_type="olmo2", architectures=["Olmo2ForCausalLM"], max_position_embeddings=self.seq_len,
                   hidden_size=self.hidden_dim, intermediate_size=self.intermediate_dim, num_hidden_layers=self.num_layers,
                   num_attention_heads=self.num_heads, num_key_value_heads=self.num_kv_heads,
                   hidden_act=self.activation_function.name, initializer_range=self.initializer_range,
                   rms_norm_eps=self.layer_norm_epsilon, tie_word_embeddings=self.tie_word_embeddings,
                   attention_bias=self.attention_bias, attention_dropout=self.attention_dropout, rope_theta=theta,
                   rope_scaling=scaling, vocab_size=vocab_size, pad_token_id=None)
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    @property
    def norm_config(self) -> LayerNormConfigBase:
        return RmsNormConfig(use_weight=self.use_layer_norm_weight, use_bias=self.use_bias, eps=self.layer_norm_epsilon)

    def mk_LayerNorm(self, dim: int):
        return self.norm_config.build(dim)

    def flops_per_token(self, vocab_size: int):
        return lm_flops_per_token(hidden_dim=self.hidden_dim, intermediate_dim=self.intermediate_dim, num_layers=self.num_layers,
                                  num_kv_heads=self.num_kv_heads, num_heads=self.num_heads, seq_len=self.seq_len,
                                  vocab_size=vocab_size, glu=True)

    def total_trainable_params(self, vocab_size: int) -> int:
        e, hs = self.hidden_dim, self.head_size
        attn = e * hs * self.num_heads + 2 * e * hs * self.num_kv_heads + hs * self.num_heads * e
        qk_norm = hs * self.num_heads + hs * self.num_kv_heads
        layer = attn + qk_norm + 3 * e * self.intermediate_dim + 2 * e
        return self.num_layers * layer + e + vocab_size * e * (1 if self.tie_word_embeddings else 2)


class Olmo2Attention(nn.Module):
    def __init__(self, config: Olmo2Config):
        super().__init__()
        c = config
        self.config = c
        hs, H, KV = c.head_size, c.num_heads, c.num_kv_heads
        G = H // KV
        b = c.attention_bias
        self.q_proj = Linear(c.hidden_dim, H * hs, bias=b, init_std=c.initializer_range, lev_out=(KV, G, hs), lev_in=(c.hidden_dim,))
        self.k_proj = Linear(c.hidden_dim, KV * hs, bias=b, init_std=c.initializer_range, lev_out=(KV, hs), lev_in=(c.hidden_dim,))
        self.v_proj = Linear(c.hidden_dim, KV * hs, bias=b, init_std=c.initializer_range, lev_out=(KV, hs), lev_in=(c.hidden_dim,))
        self.o_proj = Linear(H * hs, c.hidden_dim, bias=b, init_std=c.initializer_range, lev_out=(c.hidden_dim,), lev_in=(H, hs))
        # normalisation runs over the entire projected dimension (all heads), not per head
        self.q_norm = c.mk_LayerNorm(H * hs)
        self.k_norm = c.mk_LayerNorm(KV * hs)
        if self.q_norm.weight is not None:
            self.q_norm.weight.lev_shape = (KV, G, hs)
            self.k_norm.weight.lev_shape = (KV, hs)
        self.rot = c.rope.build(hs) if c.rope is not None else None
        self.dropout = c.attention_dropout

    def forward(self, x, mask=None, pos_ids=None):
        c = self.config
        B, S, _ = x.shape
        q = self.q_norm(self.q_proj(x)).view(B, S, c.num_heads, c.head_size)
        k = self.k_norm(self.k_proj(x)).view(B, S, c.num_kv_heads, c.head_size)
        v = self.v_proj(x).view(B, S, c.num_kv_heads, c.head_size)
        if self.rot is not None:
            q, k = rope_op.apply_rope(q, k, self.rot, pos_ids)
        out = dot_product_attention(q, k, v, mask, attention_dtype=torch.float32 if c.upcast_attn else None,
                                    attn_backend=c.attn_backend, flash_block_size=c.flash_attention_block_size,
                                    use_flash=c.use_flash_attention, dropout=self.dropout, inference=not self.training)
        return self.o_proj(out.reshape(B, S, -1).to(x.dtype))


class Olmo2DecoderLayer(nn.Module):
    def __init__(self, config: Olmo2Config, *, tp=None):
        super().__init__()
        self.self_attn = Olmo2Attention(config)
        self.mlp = LlamaMlp(config.hidden_dim, config.intermediate_dim, config.activation_function, use_bias=config.use_bias,
                            init_std=config.initializer_range)
        self.post_attention_layernorm = config.mk_LayerNorm(config.hidden_dim)
        self.post_feedforward_layernorm = config.mk_LayerNorm(config.hidden_dim)

    def forward(self, x, mask=None, pos_ids=None):
        h = x + self.post_attention_layernorm(self.self_attn(x, mask, pos_ids))
        return h + self.post_feedforward_layernorm(self.mlp(h))


class Olmo2Transformer(nn.Module):
    def __init__(self, config: Olmo2Config):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([Olmo2DecoderLayer(config) for _ in range(config.num_layers)])
        self.norm = config.mk_LayerNorm(config.hidden_dim)

    def forward(self, x, mask=None, pos_ids=None):
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        for layer in self.layers:
            x = checkpoint(layer, x, mask, pos_ids, use_reentrant=False) if remat else layer(x, mask, pos_ids)
        return self.norm(x)


class Olmo2LMHeadModel(LmHeadModel):
    def __init__(self, vocab_size: int, config: Olmo2Config, *, tp=None):
        super().__init__()
        self.config = config
        self._vocab_size = vocab_size
        self.transformer = Olmo2Transformer(config)
        self.embeddings = LlamaEmbedding(vocab_size, config)
        self.lm_head = None if config.tie_word_embeddings else Linear(config.hidden_dim, vocab_size, bias=False,
                                                                      init_std=config.initializer_range)

    @classmethod
    def init(cls, vocab_size: int, config, *, tp=None):
        return cls(vocab_size, config)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def activations(self, input_ids, attn_mask=None, *, pos_ids=None):
        return self.transformer(self.embeddings.embed(input_ids), attn_mask, pos_ids)

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
