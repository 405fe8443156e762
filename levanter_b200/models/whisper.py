"""Whisper encoder-decoder speech recognition model (src/levanter/models/whisper.py:34-509).

Encoder: conv1d(n_mels -> d, k3, p1) -> GELU -> conv1d(d -> d, k3, s2, p1) -> GELU -> + fixed sinusoids -> pre-LN
layers with unmasked self-attention -> LayerNorm.  Decoder: token embedding + learned positions (zero-initialised) ->
layers of causal self-attention, cross-attention over the encoder output and an MLP -> LayerNorm -> unembedding tied
to the token embedding.  ``k_proj`` has no bias; q/v/out do (:168-171).  Module names follow the Hugging Face
checkpoint (``self_attn``, ``encoder_attn``, ``fc1``, ...), so the state-dict key map is the identity below ``model.``."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Type

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..compat.hf_checkpoints import HFCheckpointConverter, HFCompatConfig
from ..layers.attention import AttentionBackend, AttentionMask, dot_product_attention
from ..nn import Embedding, LayerNorm, Linear
from ..ops import conv1d as conv_ops
from ..utils.activation import ActivationFunctionEnum
from ..utils.remat import should_recompute
from .asr_model import ASRConfig, ASRMixin


def whisper_sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """``[length, channels]`` table: sin of the scaled positions in the first half of the channels, cos in the second
    (src/levanter/models/whisper.py:499-509)."""
    assert channels % 2 == 0
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([torch.sin(t), torch.cos(t)], dim=1)


@ASRConfig.register_subclass("whisper")
@dataclass(frozen=True)
class WhisperConfig(HFCompatConfig, ASRConfig):
    """Defaults are whisper-tiny."""

    d_model: int = 384
    encoder_layers: int = 4
    encoder_attention_heads: int = 6
    encoder_ffn_dim: int = 1536
    decoder_layers: int = 4
    decoder_attention_heads: int = 6
    decoder_ffn_dim: int = 1536
    num_mel_bins: int = 80
    max_source_positions: int = 1500
    max_length: int = 448
    vocab_size: int = 51865
    activation_function: ActivationFunctionEnum = ActivationFunctionEnum.gelu
    initializer_range: float = 0.02
    layer_norm_epsilon: float = 1e-5
    gradient_checkpointing: bool = True
    upcast_attn: bool = True
    use_flash_attention: Optional[bool] = False
    attn_backend: Optional[AttentionBackend] = None
    flash_attention_block_size: Optional[int] = None

    hf_model_type = "whisper"
    hf_architecture = "WhisperForConditionalGeneration"

    @property
    def model_type(self) -> Type["WhisperModel"]:
        return WhisperModel

    @property
    def asr_model_type(self) -> Type["WhisperASRModel"]:
        return WhisperASRModel

    @property
    def max_seq_len(self) -> int:
        return self.max_length

    @property
    def embed_dim(self) -> int:
        return self.d_model

    def hf_checkpoint_converter(self, ref_checkpoint: Optional[str] = None) -> HFCheckpointConverter:
        return HFCheckpointConverter(self.__class__, reference_checkpoint=ref_checkpoint or "openai/whisper-base", ignore_prefix="model")

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[dict] = None) -> dict:
        cfg = dict(model_type="whisper", architectures=["WhisperForConditionalGeneration"], vocab_size=vocab_size,
                   d_model=self.d_model, encoder_layers=self.encoder_layers, encoder_attention_heads=self.encoder_attention_heads,
                   encoder_ffn_dim=self.encoder_ffn_dim, decoder_layers=self.decoder_layers,
                   decoder_attention_heads=self.decoder_attention_heads, decoder_ffn_dim=self.decoder_ffn_dim,
                   num_mel_bins=self.num_mel_bins, max_source_positions=self.max_source_positions,
                   max_target_positions=self.max_length, max_length=self.max_length,
                   activation_function=self.activation_function.value, init_std=self.initializer_range)
        cfg.update(config_overrides or {})
        return cfg

    @classmethod
    def from_hf_config(cls, hf_config) -> "WhisperConfig":
        g = (lambda k, d=None: hf_config.get(k, d)) if isinstance(hf_config, dict) else (lambda k, d=None: getattr(hf_config, k, d))
        return cls(d_model=g("d_model"), encoder_layers=g("encoder_layers"), encoder_attention_heads=g("encoder_attention_heads"),
                   encoder_ffn_dim=g("encoder_ffn_dim"), decoder_layers=g("decoder_layers"),
                   decoder_attention_heads=g("decoder_attention_heads"), decoder_ffn_dim=g("decoder_ffn_dim"),
                   num_mel_bins=g("num_mel_bins", 80), max_source_positions=g("max_source_positions", 1500),
                   max_length=g("max_target_positions", g("max_length", 448)), vocab_size=g("vocab_size", 51865),
                   activation_function=ActivationFunctionEnum(g("activation_function", "gelu")),
                   initializer_range=g("init_std", 0.02))

    def build(self, vocab_size: Optional[int] = None, *, seed: Optional[int] = None, device=None, dtype=None, tp=None):
        return self.build_asr(vocab_size or self.vocab_size, seed=seed, device=device, dtype=dtype)


class WhisperMlp(nn.Module):
    def __init__(self, d: int, ffn: int, act: ActivationFunctionEnum, std: float):
        super().__init__()
        self.fc1 = Linear(d, ffn, bias=True, init_std=std)
        self.fc2 = Linear(ffn, d, bias=True, init_std=std)
        self.act = act.to_fn()

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class WhisperAttention(nn.Module):
    """Self-attention (``xa=None``) or cross-attention with keys/values from the encoder output ``xa``."""

    def __init__(self, config: WhisperConfig, heads: int):
        super().__init__()
        self.config = config
        self.heads = heads
        d, std = config.d_model, config.initializer_range
        self.head_size = d // heads
        self.q_proj = Linear(d, d, bias=True, init_std=std)
        self.k_proj = Linear(d, d, bias=False, init_std=std)
        self.v_proj = Linear(d, d, bias=True, init_std=std)
        self.out_proj = Linear(d, d, bias=True, init_std=std)

    def forward(self, x, xa=None, mask=None):
        c = self.config
        B, S, E = x.shape
        src = x if xa is None else xa
        q = self.q_proj(x).view(B, S, self.heads, self.head_size)
        k = self.k_proj(src).view(B, src.shape[1], self.heads, self.head_size)
        v = self.v_proj(src).view(B, src.shape[1], self.heads, self.head_size)
        out = dot_product_attention(q, k, v, mask, inference=not self.training, use_flash=c.use_flash_attention,
                                    attn_backend=c.attn_backend, flash_block_size=c.flash_attention_block_size,
                                    attention_dtype=torch.float32 if c.upcast_attn else None)
        return self.out_proj(out.reshape(B, S, E).to(x.dtype))


class WhisperEncoderLayer(nn.Module):
    def __init__(self, config: WhisperConfig):
        super().__init__()
        d, eps = config.d_model, config.layer_norm_epsilon
        self.self_attn_layer_norm = LayerNorm(d, eps=eps)
        self.self_attn = WhisperAttention(config, config.encoder_attention_heads)
        self.final_layer_norm = LayerNorm(d, eps=eps)
        self.mlp = WhisperMlp(d, config.encoder_ffn_dim, config.activation_function, config.initializer_range)

    def forward(self, x):
        x = x + self.self_attn(self.self_attn_layer_norm(x))
        return x + self.mlp(self.final_layer_norm(x))


class WhisperDecoderLayer(nn.Module):
    def __init__(self, config: WhisperConfig):
        super().__init__()
        d, eps = config.d_model, config.layer_norm_epsilon
        self.self_attn_layer_norm = LayerNorm(d, eps=eps)
        self.self_attn = WhisperAttention(config, config.decoder_attention_heads)
        self.encoder_attn_layer_norm = LayerNorm(d, eps=eps)
        self.encoder_attn = WhisperAttention(config, config.decoder_attention_heads)
        self.final_layer_norm = LayerNorm(d, eps=eps)
        self.mlp = WhisperMlp(d, config.decoder_ffn_dim, config.activation_function, config.initializer_range)

    def forward(self, x, xa, mask):
        x = x + self.self_attn(self.self_attn_layer_norm(x), mask=mask)
        x = x + self.encoder_attn(self.encoder_attn_layer_norm(x), xa=xa)
        return x + self.mlp(self.final_layer_norm(x))


class _FixedPositions(nn.Module):
    """The encoder's sinusoid table, kept under the checkpoint's name (``embed_positions.weight``) as a buffer."""

    def __init__(self, length: int, channels: int):
        super().__init__()
        self.register_buffer("weight", whisper_sinusoids(length, channels))


class WhisperEncoder(nn.Module):
    def __init__(self, config: WhisperConfig):
        super().__init__()
        self.config = config
        d = config.d_model
        self.conv1 = nn.Conv1d(config.num_mel_bins, d, kernel_size=3, padding=1)
        self.conv2 = nn.Conv1d(d, d, kernel_size=3, stride=2, padding=1)
        self.embed_positions = _FixedPositions(config.max_source_positions, d)
        self.layers = nn.ModuleList([WhisperEncoderLayer(config) for _ in range(config.encoder_layers)])
        self.layer_norm = LayerNorm(d, eps=config.layer_norm_epsilon)

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        """``mel[B, n_mels, frames]`` -> ``[B, frames / 2, d_model]``."""
        w = self.conv1.weight
        mel = mel.to(w.dtype)
        if mel.is_cuda and w.dtype == torch.bfloat16 and mel.shape[-1] % 2 == 0 and conv_ops.lib.available():
            # both stem convolutions as tensor-core GEMMs over channels-last, zero-padded activations (ops/conv1d.py)
            h = F.gelu(conv_ops.conv1d_k3(conv_ops.pad_channels_last(mel), w, self.conv1.bias, 1))
            hp = F.pad(h, (0, 0, 1, 1))
            x = F.gelu(conv_ops.conv1d_k3(hp, self.conv2.weight, self.conv2.bias, 2))
        else:
            x = F.gelu(self.conv1(mel))
            x = F.gelu(self.conv2(x)).transpose(1, 2)
        if x.shape[1] > self.embed_positions.weight.shape[0]:
            raise ValueError(f"audio of {x.shape[1]} positions exceeds max_source_positions={self.embed_positions.weight.shape[0]}")
        x = x + self.embed_positions.weight[: x.shape[1]].to(x.dtype)
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        for layer in self.layers:
            x = checkpoint(layer, x, use_reentrant=False) if remat else layer(x)
        return self.layer_norm(x)


class WhisperDecoder(nn.Module):
    def __init__(self, vocab_size: int, config: WhisperConfig):
        super().__init__()
        self.config = config
        d = config.d_model
        self.embed_tokens = Embedding(vocab_size, d, init_std=config.initializer_range)
        self.embed_positions = Embedding(config.max_length, d, init_std=config.initializer_range)
        with torch.no_grad():
            self.embed_positions.weight.zero_()  # learned positions start at zero (src/levanter/models/whisper.py:367-368)
        self.layers = nn.ModuleList([WhisperDecoderLayer(config) for _ in range(config.decoder_layers)])
        self.layer_norm = LayerNorm(d, eps=config.layer_norm_epsilon)

    def forward(self, input_ids: torch.Tensor, xa: torch.Tensor, mask=None) -> torch.Tensor:
        S = input_ids.shape[-1]
        pos = torch.arange(S, device=input_ids.device)
        x = self.embed_tokens(input_ids) + self.embed_positions(pos)
        if mask is None:
            mask = AttentionMask.causal()
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        for layer in self.layers:
            x = checkpoint(layer, x, xa, mask, use_reentrant=False) if remat else layer(x, xa, mask)
        x = self.layer_norm(x)
        return self.embed_tokens.unembed(x)


class WhisperModel(ASRMixin):
    def __init__(self, vocab_size: int, config: WhisperConfig):
        super().__init__()
        self.config = config
        self._vocab_size = vocab_size
        self.encoder = WhisperEncoder(config)
        self.decoder = WhisperDecoder(vocab_size, config)

    @classmethod
    def init(cls, vocab_size: int, config: WhisperConfig, *, tp=None) -> "WhisperModel":
        return cls(vocab_size, config)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def forward(self, mel: torch.Tensor, input_ids: torch.Tensor, attn_mask=None) -> torch.Tensor:
        return self.decoder(input_ids, self.encoder(mel), attn_mask)

    def resize_vocab(self, new_size: int) -> "WhisperModel":
        self.decoder.embed_tokens = self.decoder.embed_tokens.resize_embeddings(new_size, self.config.initializer_range)
        self._vocab_size = new_size
        return self

    @staticmethod
    def hf_key_map() -> Dict[str, Optional[str]]:
        # module names already match the checkpoint except for the MLP wrapper, which the checkpoint flattens away
        return {"mlp": None}


WhisperASRModel = WhisperModel
