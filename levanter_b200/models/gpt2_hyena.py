"""GPT-2 with the attention of every block replaced by a Hyena operator (src/levanter/models/gpt2_hyena.py:29-190)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Type

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..nn import Dropout, Embedding, LayerNorm, Linear
from ..utils.remat import should_recompute
from .hyena import HyenaConfig, HyenaOperator
from .lm_model import LmConfig, LmHeadModel


@LmConfig.register_subclass("gpt2_hyena")
@dataclass(frozen=True)
class Gpt2HyenaConfig(LmConfig):
    num_layers: int = 12
    mlp_scale: int = 4
    initializer_range: float = 0.02
    embed_pdrop: float = 0.0
    layer_norm_epsilon: float = 1e-5
    gradient_checkpointing: bool = True
    gradient_checkpointing_block_size: int = 5
    hyena: HyenaConfig = field(default_factory=HyenaConfig)
    cross_entropy_block_size: Optional[int] = None

    @property
    def seq_len(self) -> int:
        return self.hyena.seq_len

    @property
    def hidden_dim(self) -> int:
        return self.hyena.hidden_dim

    @property
    def model_type(self) -> Type["Gpt2HyenaModel"]:
        return Gpt2HyenaModel

    def flops_per_token(self, vocab_size: int) -> Optional[float]:
        return None


class _Mlp(nn.Module):
    def __init__(self, config: Gpt2HyenaConfig):
        super().__init__()
        e, m = config.hidden_dim, config.hidden_dim * config.mlp_scale
        self.c_fc = Linear(e, m, bias=config.hyena.use_bias, init_std=config.initializer_range, out_first=False)
        self.c_proj = Linear(m, e, bias=config.hyena.use_bias, init_std=config.initializer_range, out_first=False)
        self.act = config.hyena.activation.to_fn()

    def forward(self, x):
        return self.c_proj(self.act(self.c_fc(x)))


class Gpt2HyenaBlock(nn.Module):
    def __init__(self, config: Gpt2HyenaConfig):
        super().__init__()
        b = config.hyena.use_bias
        self.ln_1 = LayerNorm(config.hidden_dim, eps=config.layer_norm_epsilon, use_bias=b)
        self.hyena_operator = HyenaOperator(config.hyena)
        self.ln_2 = LayerNorm(config.hidden_dim, eps=config.layer_norm_epsilon, use_bias=b)
        self.mlp = _Mlp(config)
        self.resid_dropout = Dropout(config.hyena.resid_pdrop)

    def forward(self, x):
        x = x + self.resid_dropout(self.hyena_operator(self.ln_1(x)))
        return x + self.resid_dropout(self.mlp(self.ln_2(x)))


class Gpt2HyenaBackbone(nn.Module):
    def __init__(self, config: Gpt2HyenaConfig):
        super().__init__()
        self.config = config
        self.blocks = nn.ModuleList([Gpt2HyenaBlock(config) for _ in range(config.num_layers)])
        self.ln_f = LayerNorm(config.hidden_dim, eps=config.layer_norm_epsilon, use_bias=config.hyena.use_bias)

    def forward(self, x):
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        for blk in self.blocks:
            x = checkpoint(blk, x, use_reentrant=False) if remat else blk(x)
        return self.ln_f(x)


class _Embeddings(nn.Module):
    def __init__(self, vocab_size: int, config: Gpt2HyenaConfig):
        super().__init__()
        self.token_embeddings = Embedding(vocab_size, config.hidden_dim, init_std=config.initializer_range)
        self.position_embeddings = Embedding(config.seq_len, config.hidden_dim, init_std=config.initializer_range / 2)
        self.dropout = Dropout(config.embed_pdrop)

    def embed(self, input_ids, pos_ids=None):
        if pos_ids is None:
            pos_ids = torch.arange(input_ids.shape[-1], device=input_ids.device)
        return self.dropout(self.token_embeddings(input_ids) + self.position_embeddings(pos_ids))


class Gpt2HyenaModel(LmHeadModel):
    def __init__(self, vocab_size: int, config: Gpt2HyenaConfig):
        super().__init__()
        self.config = config
        self._vocab_size = vocab_size
        self.backbone = Gpt2HyenaBackbone(config)
        self.embeddings = _Embeddings(vocab_size, config)

    @classmethod
    def init(cls, vocab_size: int, config: Gpt2HyenaConfig, *, tp=None) -> "Gpt2HyenaModel":
        return cls(vocab_size, config)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def activations(self, input_ids, attn_mask=None, *, pos_ids=None):
        # the mask is unused: the operator is causal by construction and has no notion of segments
        x = self.embeddings.embed(input_ids, pos_ids)
        if x.dim() == 2:
            return self.backbone(x.unsqueeze(0)).squeeze(0)
        return self.backbone(x)

    def get_lm_head(self) -> torch.Tensor:
        return self.embeddings.token_embeddings.weight

    def resize_vocab(self, new_size: int) -> "Gpt2HyenaModel":
        self.embeddings.token_embeddings = self.embeddings.token_embeddings.resize_embeddings(new_size, self.config.initializer_range)
        self._vocab_size = new_size
        return self

    @staticmethod
    def hf_key_map() -> Dict[str, Optional[str]]:
        return {"backbone": None, "embeddings": None, "blocks": "h", "token_embeddings": "wte", "position_embeddings": "wpe"}
