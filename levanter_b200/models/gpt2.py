"""GPT-2 (src/levanter/models/gpt2.py): learned token + position embeddings, pre-LayerNorm blocks, a fused ``c_attn``
projection to ``(qkv, heads, head_size)``, ``gelu_new`` MLP, biases, tied LM head, optional
``scale_attn_by_inverse_layer_idx`` and dropout (all 0 by default).  Linear weights are stored by the reference with
inputs first (``out_first=False``: ``c_attn.weight [embed, qkv, heads, head_size]``, :172-177), which is also Hugging
Face's Conv1D layout; here they are ``[out, in]`` in memory and marked ``lev_transposed`` for checkpoint I/O."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Type

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..compat.hf_checkpoints import HFCheckpointConverter, HFCompatConfig
from ..layers.attention import AttentionBackend, AttentionMask, dot_product_attention
from ..nn import Dropout, Embedding, LayerNorm, Linear, trunc_normal_
from ..utils.activation import ActivationFunctionEnum
from ..utils.flop_utils import lm_flops_per_token
from ..utils.remat import should_recompute
from .lm_model import LmConfig, LmHeadModel


@LmConfig.register_subclass("gpt2")
@dataclass(frozen=True)
class Gpt2Config(HFCompatConfig):
    seq_len: int = 1024
    hidden_dim: int = 768
    num_layers: int = 12
    num_heads: int = 12
    mlp_scale: int = 4
    initializer_range: float = 0.02
    embed_pdrop: float = 0.0
    resid_pdrop: float = 0.0
    attn_pdrop: float = 0.0
    layer_norm_epsilon: float = 1e-5
    activation_function: ActivationFunctionEnum = ActivationFunctionEnum.gelu_new
    scale_attn_by_inverse_layer_idx: bool = False
    upcast_attn: bool = False
    gradient_checkpointing: bool = True
    use_bias: bool = True
    use_flash_attention: Optional[bool] = None
    attn_backend: Optional[AttentionBackend] = None
    flash_attention_block_size: Optional[int] = None
    cross_entropy_block_size: Optional[int] = None

    hf_model_type = "gpt2"
    hf_architecture = "GPT2LMHeadModel"

    @property
    def model_type(self) -> Type["Gpt2LMHeadModel"]:
        return Gpt2LMHeadModel

    @property
    def head_size(self) -> int:
        return self.hidden_dim // self.num_heads

    def hf_checkpoint_converter(self, ref_checkpoint: Optional[str] = None) -> HFCheckpointConverter:
        return HFCheckpointConverter(self.__class__, reference_checkpoint=ref_checkpoint or "gpt2", ignore_prefix="transformer")

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[dict] = None) -> dict:
        cfg = dict(model_type="gpt2", architectures=["GPT2LMHeadModel"], vocab_size=vocab_size, n_positions=self.seq_len,
                   n_layer=self.num_layers, n_head=self.num_heads, n_embd=self.hidden_dim,
                   initializer_range=self.initializer_range, attn_pdrop=self.attn_pdrop, embd_pdrop=self.embed_pdrop,
                   resid_pdrop=self.resid_pdrop, layer_norm_epsilon=self.layer_norm_epsilon,
                   activation_function=self.activation_function.value,
                   scale_attn_by_inverse_layer_idx=self.scale_attn_by_inverse_layer_idx,
                   reorder_and_upcast_attn=self.upcast_attn)
        cfg.update(config_overrides or {})
        return cfg

    @classmethod
    def from_hf_config(cls, hf_config) -> "Gpt2Config":
        g = (lambda k, d=None: hf_config.get(k, d)) if isinstance(hf_config, dict) else (lambda k, d=None: getattr(hf_config, k, d))
        return cls(seq_len=g("n_positions"), num_layers=g("n_layer"), num_heads=g("n_head"), hidden_dim=g("n_embd"),
                   initializer_range=g("initializer_range", 0.02), attn_pdrop=g("attn_pdrop", 0.0),
                   embed_pdrop=g("embd_pdrop", 0.0), resid_pdrop=g("resid_pdrop", 0.0),
                   layer_norm_epsilon=g("layer_norm_epsilon", 1e-5),
                   activation_function=ActivationFunctionEnum(g("activation_function", "gelu_new")),
                   scale_attn_by_inverse_layer_idx=bool(g("scale_attn_by_inverse_layer_idx", False)),
                   upcast_attn=bool(g("reorder_and_upcast_attn", False)))

    def flops_per_token(self, vocab_size: int) -> Optional[float]:
        return lm_flops_per_token(hidden_dim=self.hidden_dim, intermediate_dim=self.hidden_dim * self.mlp_scale,
                                  num_layers=self.num_layers, num_kv_heads=self.num_heads, num_heads=self.num_heads,
                                  seq_len=self.seq_len, vocab_size=vocab_size, glu=False)

    def total_trainable_params(self, vocab_size: int) -> int:
        e = self.hidden_dim
        b = 1 if self.use_bias else 0
        attn = e * 3 * e + b * 3 * e + e * e + b * e
        mlp = 2 * e * e * self.mlp_scale + b * (e * self.mlp_scale + e)
        ln = 2 * (e + b * e)
        return self.num_layers * (attn + mlp + ln) + (e + b * e) + vocab_size * e + self.seq_len * e


class Gpt2Mlp(nn.Module):
    def __init__(self, config: Gpt2Config):
        super().__init__()
        e, m = config.hidden_dim, config.hidden_dim * config.mlp_scale
        self.c_fc = Linear(e, m, bias=config.use_bias, init_std=config.initializer_range, out_first=False)
        self.c_proj = Linear(m, e, bias=config.use_bias, init_std=config.initializer_range, out_first=False)
        self.act = config.activation_function.to_fn()

    def forward(self, x):
        return self.c_proj(self.act(self.c_fc(x)))


class Gpt2Attention(nn.Module):
    def __init__(self, config: Gpt2Config):
        super().__init__()
        self.config = config
        e, h, d = config.hidden_dim, config.num_heads, config.head_size
        self.c_attn = Linear(e, 3 * e, bias=config.use_bias, init_std=config.initializer_range, out_first=False,
                             lev_out=(3, h, d), lev_in=(e,))
        self.c_proj = Linear(e, e, bias=config.use_bias, init_std=config.initializer_range, out_first=False,
                             lev_out=(e,), lev_in=(h, d))

    def forward(self, x, mask, layer_idx: int):
        c = self.config
        B, S, E = x.shape
        qkv = self.c_attn(x).view(B, S, 3, c.num_heads, c.head_size)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if c.scale_attn_by_inverse_layer_idx:
            q = q / (layer_idx + 1.0)
        out = dot_product_attention(q, k, v, mask, inference=not self.training, dropout=c.attn_pdrop,
                                    use_flash=c.use_flash_attention, attn_backend=c.attn_backend,
                                    flash_block_size=c.flash_attention_block_size,
                                    attention_dtype=torch.float32 if c.upcast_attn else None)
        return self.c_proj(out.reshape(B, S, E).to(x.dtype))


class Gpt2Block(nn.Module):
    def __init__(self, config: Gpt2Config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.ln_1 = LayerNorm(config.hidden_dim, eps=config.layer_norm_epsilon, use_bias=config.use_bias)
        self.attn = Gpt2Attention(config)
        self.ln_2 = LayerNorm(config.hidden_dim, eps=config.layer_norm_epsilon, use_bias=config.use_bias)
        self.mlp = Gpt2Mlp(config)
        self.resid_dropout = Dropout(config.resid_pdrop)

    def forward(self, x, mask):
        x = x + self.resid_dropout(self.attn(self.ln_1(x), mask, self.layer_idx))
        x = x + self.resid_dropout(self.mlp(self.ln_2(x)))
        return x


class Gpt2Transformer(nn.Module):
    def __init__(self, config: Gpt2Config):
        super().__init__()
        self.config = config
        self.blocks = nn.ModuleList([Gpt2Block(config, i) for i in range(config.num_layers)])
        self.ln_f = LayerNorm(config.hidden_dim, eps=config.layer_norm_epsilon, use_bias=config.use_bias)

    def forward(self, x, mask):
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        for blk in self.blocks:
            x = checkpoint(blk, x, mask, use_reentrant=False) if remat else blk(x, mask)
        return self.ln_f(x)


class Gpt2Embeddings(nn.Module):
    def __init__(self, vocab_size: int, config: Gpt2Config):
        super().__init__()
        self.token_embeddings = Embedding(vocab_size, config.hidden_dim, init_std=config.initializer_range)
        # position embeddings start at half the scale of token embeddings (src/levanter/models/gpt2.py:291-296)
        self.position_embeddings = Embedding(config.seq_len, config.hidden_dim, init_std=config.initializer_range / 2)
        self.dropout = Dropout(config.embed_pdrop)

    def embed(self, input_ids, pos_ids=None):
        S = input_ids.shape[-1]
        if pos_ids is None:
            pos_ids = torch.arange(S, device=input_ids.device)
        return self.dropout(self.token_embeddings(input_ids) + self.position_embeddings(pos_ids))

    def unembed(self, x):
        return self.token_embeddings.unembed(x)


class Gpt2LMHeadModel(LmHeadModel):
    def __init__(self, vocab_size: int, config: Gpt2Config):
        super().__init__()
        self.config = config
        self._vocab_size = vocab_size
        self.transformer = Gpt2Transformer(config)
        self.embeddings = Gpt2Embeddings(vocab_size, config)

    @classmethod
    def init(cls, vocab_size: int, config: Gpt2Config, *, tp=None) -> "Gpt2LMHeadModel":
        return cls(vocab_size, config)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def activations(self, input_ids, attn_mask=None, *, pos_ids=None):
        x = self.embeddings.embed(input_ids, pos_ids)
        return self.transformer(x, attn_mask)

    def get_lm_head(self) -> torch.Tensor:
        return self.embeddings.token_embeddings.weight

    def resize_vocab(self, new_size: int) -> "Gpt2LMHeadModel":
        self.embeddings.token_embeddings = self.embeddings.token_embeddings.resize_embeddings(new_size, self.config.initializer_range)
        self._vocab_size = new_size
        return self

    @staticmethod
    def hf_key_map() -> Dict[str, Optional[str]]:
        # transformer/embeddings are flattened away; blocks -> h, token_embeddings -> wte, position_embeddings -> wpe
        return {"transformer": None, "embeddings": None, "blocks": "h", "token_embeddings": "wte", "position_embeddings": "wpe"}
