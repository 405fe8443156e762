"""Speech-recognition model interfaces (src/levanter/models/asr_model.py:19-123): the audio+text training example, the
config registry for encoder-decoder ASR models and the loss mix-in."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Type, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ChoiceRegistry
from ..layers.attention import AttentionMask


@dataclass
class AudioTextExample:
    """``audio[..., n_mels, frames]`` log-mel features, ``tokens[..., S]`` transcript ids, ``loss_mask[..., S]``."""

    audio: torch.Tensor
    tokens: torch.Tensor
    loss_mask: torch.Tensor
    attn_mask: Union[AttentionMask, torch.Tensor] = field(default_factory=AttentionMask.causal)

    @staticmethod
    def init(audio: torch.Tensor, tokens: torch.Tensor, *, attn_mask=None, loss_mask: Optional[torch.Tensor] = None,
             ignore_id: Optional[int] = None) -> "AudioTextExample":
        """Default loss mask: every position but the last, and not where the *next* token is ``ignore_id`` (padding)
        (src/levanter/models/asr_model.py:29-51)."""
        if tokens.dtype not in (torch.int32, torch.int64, torch.int16, torch.uint8):
            raise ValueError("tokens must be an integer array")
        S = tokens.shape[-1]
        if loss_mask is None:
            loss_mask = torch.ones(tokens.shape, dtype=torch.float32, device=tokens.device)
            loss_mask[..., S - 1] = 0.0
        if ignore_id is not None:
            loss_mask = loss_mask * (torch.roll(tokens, -1, dims=-1) != ignore_id).to(loss_mask.dtype)
        return AudioTextExample(audio, tokens, loss_mask, attn_mask if attn_mask is not None else AttentionMask.causal())

    @staticmethod
    def stack(examples) -> "AudioTextExample":
        return AudioTextExample(torch.stack([e.audio for e in examples]), torch.stack([e.tokens for e in examples]),
                                torch.stack([e.loss_mask for e in examples]), examples[0].attn_mask)

    def to(self, device, non_blocking: bool = False) -> "AudioTextExample":
        mv = lambda t: t.to(device, non_blocking=non_blocking) if isinstance(t, torch.Tensor) else t  # noqa: E731
        return AudioTextExample(mv(self.audio), mv(self.tokens), mv(self.loss_mask), mv(self.attn_mask))

    def slice(self, start: int, stop: int) -> "AudioTextExample":
        return AudioTextExample(self.audio[start:stop], self.tokens[start:stop], self.loss_mask[start:stop], self.attn_mask)

    @property
    def batch_size(self) -> int:
        return self.tokens.shape[0] if self.tokens.dim() > 1 else 1


@dataclass(frozen=True)
class ASRConfig(ChoiceRegistry):
    """Base of ASR model configs, selected in YAML by ``model.type`` (src/levanter/models/asr_model.py:55-73)."""

    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return "whisper"

    @property
    def model_type(self) -> Type["ASRMixin"]:
        raise NotImplementedError

    def build_asr(self, vocab_size: int, *, seed: Optional[int] = None, device=None, dtype=None):
        import contextlib

        dev_ctx = torch.device(device) if device is not None else contextlib.nullcontext()
        with dev_ctx:
            if seed is not None:
                devs = [torch.device(device)] if device is not None and torch.device(device).type == "cuda" else []
                with torch.random.fork_rng(devices=devs):
                    torch.manual_seed(seed)
                    m = self.model_type.init(vocab_size, self)
            else:
                m = self.model_type.init(vocab_size, self)
        return m.to(dtype=dtype) if dtype is not None else m


class ASRMixin(nn.Module):
    """An encoder-decoder speech model: ``forward(mel, input_ids, attn_mask) -> logits[..., S, vocab]``.

    ``compute_loss`` is the plain (not vocabulary-blocked) cross-entropy in fp32 against the tokens shifted by one,
    averaged over ``loss_mask`` (src/levanter/models/asr_model.py:98-119)."""

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    @property
    def Vocab(self) -> int:
        return self.vocab_size

    def compute_loss(self, example: AudioTextExample, *, reduction: Optional[str] = "mean", reduction_dim=None) -> torch.Tensor:
        logits = self(example.audio, example.tokens, example.attn_mask).float()
        targets = torch.roll(example.tokens, -1, dims=-1).long()
        per_tok = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), reduction="none").view(targets.shape)
        mask = example.loss_mask.to(per_tok.dtype)
        per_tok = per_tok * mask
        if reduction is None:
            return per_tok
        if reduction == "sum":
            return per_tok.sum() if reduction_dim is None else per_tok.sum(dim=reduction_dim)
        if reduction_dim is None:
            return per_tok.sum() / mask.sum().clamp_min(1.0)
        return per_tok.sum(dim=reduction_dim) / mask.sum(dim=reduction_dim).clamp_min(1.0)


def compute_asr_loss(model: ASRMixin, example: AudioTextExample, *, reduction="mean", reduction_dim=None, **_):
    """Loss function with the trainer's ``(model, batch)`` signature."""
    return model.compute_loss(example, reduction=reduction, reduction_dim=reduction_dim)
