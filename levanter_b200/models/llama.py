"""Llama 1/2/3 family (src/levanter/models/llama.py).

Defaults are Llama-2-7B (:54-63).  Supports ``hybrid_norm`` (extra norms after attention and MLP, :289-332),
``input_embedding_norm`` (:442-465), tied embeddings, biases, a ``head_dim`` override, any RoPE config, per-layer
activation checkpointing, and the paged-KV ``decode`` path used by the inference engine (:336-370, 581-634).

Torch parameter names mirror the reference's tree (``transformer.layers.<i>.self_attn.q_proj.weight`` ...); the
checkpoint writer stacks ``layers.<i>`` into the reference's ``layers/stacked`` leading axis.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, Optional, Tuple, Type, Union

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..compat.hf_checkpoints import HFCheckpointConverter, HFCompatConfig
from ..layers.attention import Attention, AttentionBackend, AttentionConfig, AttentionMask, KvPageCache
from ..layers.normalization import LayerNormConfigBase, RmsNormConfig
from ..layers.rotary import rope_config_from_hf, rope_to_hf_dict, DefaultRotaryEmbeddingsConfig, RotaryEmbeddingsConfig
from ..nn import Embedding, Linear
from ..ops.gemm import linear_residual
from ..ops.glu import gated_activation
from ..utils.activation import ActivationFunctionEnum
from ..utils.flop_utils import lm_flops_per_token
from ..utils.remat import ScanCheckpointPolicy, checkpoint_layer, keeps_attention, should_recompute
from .lm_model import LmConfig, LmHeadModel


@LmConfig.register_subclass("llama")
@dataclass(frozen=True)
class LlamaConfig(HFCompatConfig):
    seq_len: int = 2048
    hidden_dim: int = 4096
    intermediate_dim: int = 11008
    num_layers: int = 32
    num_heads: int = 32
    head_dim: Optional[int] = None
    num_kv_heads: int = 32
    activation_function: ActivationFunctionEnum = ActivationFunctionEnum.silu
    initializer_range: float = 0.02
    layer_norm_epsilon: float = 1e-5
    tie_word_embeddings: bool = False
    hybrid_norm: bool = False
    input_embedding_norm: bool = False

    upcast_attn: bool = False
    attn_backend: Optional[AttentionBackend] = None
    flash_attention_block_size: Optional[int] = None

    gradient_checkpointing: Union[bool, ScanCheckpointPolicy, str] = True
    scan_layers: bool = True

    use_bias: bool = False
    use_layer_norm_weight: bool = True
    rope: RotaryEmbeddingsConfig = dataclasses.field(default_factory=DefaultRotaryEmbeddingsConfig)

    reference_checkpoint: str = "NousResearch/Llama-2-7b-hf"
    tokenizer: Optional[str] = None
    cross_entropy_block_size: Optional[int] = None

    def __post_init__(self):
        assert self.num_heads % self.num_kv_heads == 0, \
            f"num_heads={self.num_heads} not divisible by num_kv_heads={self.num_kv_heads}."

    hf_model_type = "llama"
    hf_architecture = "LlamaForCausalLM"

    def hf_checkpoint_converter(self, ref_checkpoint: Optional[str] = None) -> HFCheckpointConverter:
        return HFCheckpointConverter(self.__class__, reference_checkpoint=ref_checkpoint or self.reference_checkpoint,
                                     tokenizer=ref_checkpoint if self.tokenizer is None else self.tokenizer)

    @classmethod
    def from_hf_config(cls, hf_config) -> "LlamaConfig":
        g = _getter(hf_config)
        rope = rope_config_from_hf(g, 10000.0)
        return cls(
            seq_len=g("max_position_embeddings"), hidden_dim=g("hidden_size"), intermediate_dim=g("intermediate_size"),
            num_layers=g("num_hidden_layers"), num_heads=g("num_attention_heads"),
            num_kv_heads=g("num_key_value_heads", g("num_attention_heads")),
            activation_function=ActivationFunctionEnum(g("hidden_act", "silu")),
            initializer_range=g("initializer_range", 0.02), layer_norm_epsilon=g("rms_norm_eps", 1e-5),
            tie_word_embeddings=bool(g("tie_word_embeddings", False)), rope=rope,
            use_bias=bool(g("attention_bias", False)),
        )

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        if self.hybrid_norm or self.input_embedding_norm:
            raise ValueError("Cannot export to HuggingFace format with hybrid_norm or input_embedding_norm enabled.")
        theta, scaling = self.rope.to_hf_config()
        cfg = dict(
            model_type=self.hf_model_type, architectures=[self.hf_architecture],
            max_position_embeddings=self.seq_len, hidden_size=self.hidden_dim, intermediate_size=self.intermediate_dim,
            num_hidden_layers=self.num_layers, num_attention_heads=self.num_heads, num_key_value_heads=self.num_kv_heads,
            hidden_act=self.activation_function.name, initializer_range=self.initializer_range,
            rms_norm_eps=self.layer_norm_epsilon, tie_word_embeddings=self.tie_word_embeddings, vocab_size=vocab_size,
            rope_theta=theta, rope_scaling=scaling, attention_bias=self.use_bias, mlp_bias=self.use_bias,
        )
        if self.head_dim is not None:
            cfg["head_dim"] = self.head_dim
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    @property
    def model_type(self) -> Type["LlamaLMHeadModel"]:
        return LlamaLMHeadModel

    @property
    def norm_config(self) -> LayerNormConfigBase:
        return RmsNormConfig(use_weight=self.use_layer_norm_weight, use_bias=self.use_bias, eps=self.layer_norm_epsilon)

    def mk_LayerNorm(self, dim: int):
        return self.norm_config.build(dim)

    def flops_per_token(self, vocab_size: int):
        return lm_flops_per_token(hidden_dim=self.hidden_dim, intermediate_dim=self.intermediate_dim,
                                  num_layers=self.num_layers, num_kv_heads=self.num_kv_heads, num_heads=self.num_heads,
                                  seq_len=self.seq_len, vocab_size=vocab_size, glu=True)

    def total_trainable_params(self, vocab_size):
        token_embedding = vocab_size * self.hidden_dim
        hs = self.actual_head_size
        attn = self.hidden_dim * hs * self.num_heads + 2 * self.hidden_dim * hs * self.num_kv_heads + hs * self.num_heads * self.hidden_dim
        mlp = 3 * self.hidden_dim * self.intermediate_dim
        layer = attn + mlp + 2 * self.hidden_dim + (2 * self.hidden_dim if self.hybrid_norm else 0)
        transformer = self.num_layers * layer + self.hidden_dim + (self.hidden_dim if self.input_embedding_norm else 0)
        return transformer + token_embedding + (0 if self.tie_word_embeddings else token_embedding)

    def attention_config(self) -> AttentionConfig:
        return AttentionConfig(hidden_dim=self.hidden_dim, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                               head_dim=self.head_dim, use_bias=self.use_bias, upcast_attn=self.upcast_attn,
                               attn_backend=self.attn_backend, flash_attention_block_size=self.flash_attention_block_size,
                               rope=self.rope)

    @property
    def actual_head_size(self) -> int:
        return self.head_dim if self.head_dim is not None else self.hidden_dim // self.num_heads


def _getter(hf_config):
    if isinstance(hf_config, dict):
        return lambda k, d=None: hf_config.get(k, d) if hf_config.get(k, d) is not None else d
    return lambda k, d=None: getattr(hf_config, k, d) if getattr(hf_config, k, d) is not None else d


class LlamaMlp(nn.Module):
    """SwiGLU MLP: ``down(act(gate(x)) * up(x))`` (src/levanter/models/llama.py:243-280)."""

    def __init__(self, hidden: int, intermediate: int, activation: ActivationFunctionEnum, *, use_bias: bool = False,
                 init_std: float = 0.02, tp=None):
        super().__init__()
        tp_size = tp.size if tp is not None else 1
        assert intermediate % tp_size == 0
        local = intermediate // tp_size
        self.tp = tp
        self.gate_proj = Linear(hidden, local, bias=use_bias, init_std=init_std, parallel=("column", tp))
        self.up_proj = Linear(hidden, local, bias=use_bias, init_std=init_std, parallel=("column", tp))
        self.down_proj = Linear(local, hidden, bias=use_bias, init_std=init_std, parallel=("row", tp))
        self.act = activation if isinstance(activation, ActivationFunctionEnum) else ActivationFunctionEnum(activation)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.tp is not None and self.tp.size > 1:
            x = self.tp.copy_to_region(x)
        h = gated_activation(self.gate_proj(x), self.up_proj(x), self.act)
        if self.tp is not None and self.tp.size > 1:
            out = self.tp.row_linear(h, self.down_proj)
            if self.down_proj.bias is not None:
                out = out + self.down_proj.bias
            return out if residual is None else out + residual
        if type(self.down_proj) is Linear:
            return linear_residual(h, self.down_proj.weight, self.down_proj.bias, residual)
        out = self.down_proj(h)
        return out if residual is None else out + residual


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config: LlamaConfig, *, tp=None, attn_config: Optional[AttentionConfig] = None):
        super().__init__()
        self.config = config
        self.tp = tp
        self.self_attn = Attention(attn_config or config.attention_config(), init_std=config.initializer_range, tp=tp)
        self.mlp = LlamaMlp(config.hidden_dim, config.intermediate_dim, config.activation_function,
                            use_bias=config.use_bias, init_std=config.initializer_range, tp=tp)
        self.input_layernorm = config.mk_LayerNorm(config.hidden_dim)
        self.post_attention_layernorm = config.mk_LayerNorm(config.hidden_dim)
        if config.hybrid_norm:
            self.post_attn_layernorm = config.mk_LayerNorm(config.hidden_dim)
            self.post_mlp_layernorm = config.mk_LayerNorm(config.hidden_dim)
        else:
            self.post_attn_layernorm = None
            self.post_mlp_layernorm = None

    def _attn_block(self, x, mask, pos_ids):
        """``x + attn(norm(x))`` with the residual add folded into the output-projection GEMM epilogue."""
        a = self.self_attn
        h = self.input_layernorm(x)
        tp_on = self.tp is not None and self.tp.size > 1
        if self.post_attn_layernorm is not None or tp_on:
            if tp_on:
                h = self.tp.copy_to_region(h)
            out = a(h, mask, pos_ids) if not tp_on else self._tp_attn(h, mask, pos_ids)
            if self.post_attn_layernorm is not None:
                out = self.post_attn_layernorm(out)
            return x + out
        return a.forward_with_residual(h, mask, pos_ids, x)

    def _tp_attn(self, h, mask, pos_ids):
        a = self.self_attn
        out = a.forward(h, mask, pos_ids, skip_out_bias=True, row_parallel=self.tp)
        if a.o_proj.bias is not None:
            out = out + a.o_proj.bias
        return out

    def forward(self, x: torch.Tensor, mask=None, pos_ids=None) -> torch.Tensor:
        x = self._attn_block(x, mask, pos_ids)
        h = self.post_attention_layernorm(x)
        if self.post_mlp_layernorm is not None:
            return x + self.post_mlp_layernorm(self.mlp(h))
        return self.mlp(h, residual=x)

    def decode(self, x, kv_cache: KvPageCache, batch_info, pos_ids):
        h = self.input_layernorm(x)
        tp_on = self.tp is not None and self.tp.size > 1
        if not tp_on and self.post_attn_layernorm is None:
            # both residual adds ride in the epilogues of the output and down projections
            x, kv_cache = self.self_attn.paged_decode(h, kv_cache, batch_info, pos_ids, residual=x)
        else:
            attn_out, kv_cache = self.self_attn.paged_decode(h, kv_cache, batch_info, pos_ids)
            if tp_on:
                attn_out = self.tp.all_reduce(attn_out)
            if self.post_attn_layernorm is not None:
                attn_out = self.post_attn_layernorm(attn_out)
            x = x + attn_out
        h = self.post_attention_layernorm(x)
        if self.post_mlp_layernorm is None:
            return self.mlp(h, residual=x), kv_cache
        return x + self.post_mlp_layernorm(self.mlp(h)), kv_cache


class LlamaTransformer(nn.Module):
    def __init__(self, config: LlamaConfig, *, tp=None, layer_cls=LlamaDecoderLayer):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([layer_cls(config, tp=tp) for _ in range(config.num_layers)])
        self.norm = config.mk_LayerNorm(config.hidden_dim)

    def forward(self, x, mask=None, pos_ids=None):
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        keep = keeps_attention(self.config.gradient_checkpointing)
        for layer in self.layers:
            if remat:
                x = checkpoint_layer(layer, x, mask, pos_ids, keep_attention=keep)
            else:
                x = layer(x, mask, pos_ids)
        return self.norm(x)

    def decode(self, x, caches, batch_info, pos_ids):
        new = []
        for layer, c in zip(self.layers, caches):
            x, c = layer.decode(x, c, batch_info, pos_ids)
            new.append(c)
        return self.norm(x), new

    def initial_cache(self, max_pages: int, page_size: int, *, dtype=torch.bfloat16, device=None):
        return [l.self_attn.empty_page_cache(max_pages, page_size, dtype=dtype, device=device) for l in self.layers]


class LlamaEmbedding(nn.Module):
    def __init__(self, vocab_size: int, config, *, norm: bool = False):
        super().__init__()
        self.token_embeddings = Embedding(vocab_size, config.hidden_dim, init_std=config.initializer_range)
        self.norm = config.mk_LayerNorm(config.hidden_dim) if norm else None

    def embed(self, input_ids):
        x = self.token_embeddings(input_ids)
        return self.norm(x) if self.norm is not None else x

    forward = embed

    def unembed(self, x):
        return self.token_embeddings.unembed(x)


class LlamaLMHeadModel(LmHeadModel):
    def __init__(self, vocab_size: int, config: LlamaConfig, *, tp=None, layer_cls=LlamaDecoderLayer):
        super().__init__()
        self.config = config
        self._vocab_size = vocab_size
        self.transformer = LlamaTransformer(config, tp=tp, layer_cls=layer_cls)
        self.embeddings = LlamaEmbedding(vocab_size, config, norm=getattr(config, "input_embedding_norm", False))
        if config.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = Linear(config.hidden_dim, vocab_size, bias=False, init_std=config.initializer_range)

    @classmethod
    def init(cls, vocab_size: int, config: LlamaConfig, *, tp=None) -> "LlamaLMHeadModel":
        return cls(vocab_size, config, tp=tp)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def activations(self, input_ids, attn_mask=None, *, pos_ids=None):
        x = self.embeddings.embed(input_ids)
        return self.transformer(x, attn_mask, pos_ids)

    def get_lm_head(self) -> torch.Tensor:
        return self.embeddings.token_embeddings.weight if self.lm_head is None else self.lm_head.weight

    def resize_vocab(self, new_size: int) -> "LlamaLMHeadModel":
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

    # -- paged-KV inference ------------------------------------------------------------------------------------
    def initial_cache(self, max_pages, page_size: Optional[int] = None, *, dtype=torch.bfloat16, device=None):
        """One ``KvPageCache`` per layer.  ``max_pages`` may be a page table (then its sizes are used), as in the reference
        (src/levanter/models/llama.py:581-586)."""
        if page_size is None and hasattr(max_pages, "num_pages"):
            max_pages, page_size = max_pages.num_pages, max_pages.page_size
        if device is None:
            device = next(self.parameters()).device
        return self.transformer.initial_cache(max_pages, page_size, dtype=dtype, device=device)

    def decode(self, input_ids: torch.Tensor, kv_cache, batch_info, pos_ids: torch.Tensor, logit_rows: Optional[torch.Tensor] = None):
        """Logits for packed tokens ``[T]`` given the paged KV cache (src/levanter/models/llama.py:589-634); with
        ``logit_rows`` only for those token rows (a prefill needs the last token of every prompt, not ``T x vocab`` logits)."""
        x = self.embeddings.embed(input_ids)
        x, kv_cache = self.transformer.decode(x, kv_cache, batch_info, pos_ids)
        if logit_rows is not None:
            x = x.index_select(0, logit_rows)
        head = self.get_lm_head()
        logits = torch.nn.functional.linear(x, head.to(x.dtype))
        return logits, kv_cache

    # -- HF key mapping (src/levanter/models/llama.py:470-471,578-579) -------------------------------------------
    @staticmethod
    def hf_key_map() -> Dict[str, Optional[str]]:
        return {"transformer": "model", "embeddings": None, "token_embeddings": "model.embed_tokens"}
