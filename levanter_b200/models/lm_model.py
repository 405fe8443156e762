"""Language-model interfaces: ``LmExample``, the ``LmConfig`` plugin registry, ``LmHeadModel`` and the loss entry point
(src/levanter/models/lm_model.py:24-294)."""
from __future__ import annotations

import abc
from dataclasses import dataclass, field
from typing import Generic, List, Optional, Sequence, Tuple, Type, TypeVar, Union

import torch
import torch.nn as nn

from ..config import ChoiceRegistry
from ..layers.attention import AttentionMask
from .loss import maybe_fused_next_token_loss

LmT = TypeVar("LmT", bound="LmHeadModel")


@dataclass
class LmExample:
    """One example or a batch: ``tokens[..., S]`` int, ``loss_mask[..., S]``, and the attention mask."""

    tokens: torch.Tensor
    loss_mask: torch.Tensor
    attn_mask: Union[AttentionMask, torch.Tensor] = field(default_factory=AttentionMask.causal)

    @staticmethod
    def causal_loss_mask(seq_len: int, prompt_length=None, device=None) -> torch.Tensor:
        mask = torch.ones(seq_len, dtype=torch.float32, device=device)
        mask[-1] = 0.0
        if prompt_length is not None:
            pos = torch.arange(seq_len, device=device)
            if isinstance(prompt_length, torch.Tensor) and prompt_length.dim() > 0:
                mask = mask * (pos[None, :] >= (prompt_length[:, None] - 1)).float()
            else:
                mask = mask * (pos >= (int(prompt_length) - 1)).float()
        return mask

    @staticmethod
    def causal(tokens: torch.Tensor, *, loss_mask: Optional[torch.Tensor] = None, ignore_id: Optional[int] = None,
               eos_id: Optional[int] = None, segment_ids: Optional[torch.Tensor] = None,
               sliding_window: Optional[int] = None) -> "LmExample":
        """Causal LM example: loss on every position but the last (and not where the *next* token is ``ignore_id``);
        when ``eos_id`` is given, the token after each EOS starts a new attention segment
        (src/levanter/models/lm_model.py:30-74)."""
        if tokens.dtype not in (torch.int32, torch.int64, torch.int16, torch.uint8):
            raise ValueError("tokens must be an integer array")
        S = tokens.shape[-1]
        causal_lm = LmExample.causal_loss_mask(S, device=tokens.device)
        if loss_mask is not None:
            lm = loss_mask.to(torch.float32) * causal_lm
        else:
            lm = causal_lm.expand(tokens.shape).clone()
        if ignore_id is not None:
            lm = lm * (torch.roll(tokens, -1, dims=-1) != ignore_id).float()
        lm = lm.to(torch.int32)
        attn = AttentionMask.causal(sliding_window=sliding_window)
        if eos_id is not None and segment_ids is None:
            eos_mask = torch.roll(tokens, 1, dims=-1) == eos_id
            eos_mask[..., 0] = False
            segment_ids = torch.cumsum(eos_mask.to(torch.int32), dim=-1).to(torch.int32)
            attn = attn.with_segment_ids(segment_ids)
        elif segment_ids is not None:
            attn = attn.with_segment_ids(segment_ids)
        return LmExample(tokens=tokens, loss_mask=lm, attn_mask=attn)

    @staticmethod
    def from_prompt_and_completion(tokens: torch.Tensor, prompt_length, *, ignore_id: Optional[int] = None,
                                   all_causal: bool = True, sliding_window: Optional[int] = None) -> "LmExample":
        if not all_causal:
            raise NotImplementedError("only fully causal attention is supported for prompt/completion examples")
        S = tokens.shape[-1]
        lm = LmExample.causal_loss_mask(S, prompt_length=prompt_length, device=tokens.device)
        if lm.dim() < tokens.dim():
            lm = lm.expand(tokens.shape).clone()
        if ignore_id is not None:
            lm = lm * (torch.roll(tokens, -1, dims=-1) != ignore_id).float()
        return LmExample(tokens=tokens, loss_mask=lm, attn_mask=AttentionMask.causal(sliding_window=sliding_window))

    # -- batching helpers -------------------------------------------------------------------------------------
    @staticmethod
    def stack(examples: Sequence["LmExample"]) -> "LmExample":
        tokens = torch.stack([e.tokens for e in examples])
        lm = torch.stack([e.loss_mask for e in examples])
        m0 = examples[0].attn_mask
        if isinstance(m0, AttentionMask):
            seg = None
            if m0.segment_ids is not None:
                seg = (torch.stack([e.attn_mask.segment_ids[0] for e in examples]),
                       torch.stack([e.attn_mask.segment_ids[1] for e in examples]))
            em = None
            if m0.explicit_mask is not None:
                em = torch.stack([e.attn_mask.explicit_mask for e in examples])
            mask = AttentionMask(m0.is_causal, m0.causal_offset, em, seg, m0.sliding_window)
        else:
            mask = torch.stack([e.attn_mask for e in examples])
        return LmExample(tokens, lm, mask)

    def to(self, device, non_blocking: bool = False) -> "LmExample":
        def mv(t):
            return t.to(device, non_blocking=non_blocking) if isinstance(t, torch.Tensor) else t

        m = self.attn_mask
        if isinstance(m, AttentionMask):
            seg = None if m.segment_ids is None else (mv(m.segment_ids[0]), mv(m.segment_ids[1]))
            m = AttentionMask(m.is_causal, mv(m.causal_offset), mv(m.explicit_mask), seg, m.sliding_window)
        else:
            m = mv(m)
        return LmExample(mv(self.tokens), mv(self.loss_mask), m)

    def slice(self, start: int, stop: int) -> "LmExample":
        """Rows ``start:stop`` of a batched example (microbatching)."""
        m = self.attn_mask
        if isinstance(m, AttentionMask):
            seg = None if m.segment_ids is None else (m.segment_ids[0][start:stop], m.segment_ids[1][start:stop])
            em = None if m.explicit_mask is None else (m.explicit_mask[start:stop] if m.explicit_mask.dim() > 2 else m.explicit_mask)
            off = m.causal_offset
            if isinstance(off, torch.Tensor) and off.dim() > 0:
                off = off[start:stop]
            m = AttentionMask(m.is_causal, off, em, seg, m.sliding_window)
        else:
            m = m[start:stop] if m.dim() > 2 else m
        return LmExample(self.tokens[start:stop], self.loss_mask[start:stop], m)

    @property
    def batch_size(self) -> int:
        return self.tokens.shape[0] if self.tokens.dim() > 1 else 1


@dataclass(frozen=True)
class LmConfig(ChoiceRegistry):
    """Base of every model config; selected in YAML by ``model.type`` (llama is the default, as in
    src/levanter/main/train_lm.py:42)."""

    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return "llama"

    @property
    def model_type(self) -> Type["LmHeadModel"]:
        raise NotImplementedError

    @property
    def max_seq_len(self) -> int:
        return getattr(self, "seq_len")

    @property
    def embed_dim(self) -> int:
        return getattr(self, "hidden_dim")

    def flops_per_token(self, vocab_size: int) -> Optional[float]:
        return None

    def total_trainable_params(self, vocab_size: int) -> Optional[float]:
        return None

    def build(self, vocab_size: int, *, seed: Optional[int] = None, device=None, dtype=None, tp=None) -> "LmHeadModel":
        """Random-init model.  ``seed`` makes initialisation reproducible; ``tp`` is the tensor-parallel group."""
        import contextlib

        dev_ctx = torch.device(device) if device is not None else contextlib.nullcontext()
        with dev_ctx:  # parameters are created (and initialised) directly on the target device
            if seed is not None:
                devs = [torch.device(device)] if device is not None and torch.device(device).type == "cuda" else []
                with torch.random.fork_rng(devices=devs):
                    torch.manual_seed(seed)
                    m = self.model_type.init(vocab_size, self, tp=tp)
            else:
                m = self.model_type.init(vocab_size, self, tp=tp)
        if dtype is not None:
            m = m.to(dtype=dtype)
        return m


class LmHeadModel(nn.Module, Generic[LmT]):
    """Transformer body + LM head.  ``activations`` returns final hidden states (or ``(hidden, aux_loss)`` for MoE);
    ``get_lm_head`` returns the ``[vocab, embed]`` head matrix (src/levanter/models/lm_model.py:153-253)."""

    config: LmConfig

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    @property
    def Vocab(self) -> int:
        return self.vocab_size

    @classmethod
    def init(cls, vocab_size: int, config, *, tp=None) -> "LmHeadModel":
        raise NotImplementedError

    def activations(self, input_ids: torch.Tensor, attn_mask=None, *, pos_ids=None):
        raise NotImplementedError

    def get_lm_head(self) -> torch.Tensor:
        raise NotImplementedError

    def resize_vocab(self, new_size: int) -> "LmHeadModel":
        raise NotImplementedError

    def forward(self, input_ids: torch.Tensor, attn_mask=None, *, pos_ids=None) -> torch.Tensor:
        """Logits ``[..., S, V]``."""
        x = self.activations(input_ids, attn_mask, pos_ids=pos_ids)
        if isinstance(x, tuple):
            x = x[0]
        head = self.get_lm_head()
        return torch.nn.functional.linear(x, head.to(x.dtype))

    def compute_loss(self, example: LmExample, *, reduction="mean", reduction_dim=None, **kw):
        return compute_next_token_loss(self, example, reduction=reduction, reduction_dim=reduction_dim, **kw)


def compute_next_token_loss(model: LmHeadModel, example: LmExample, *, reduction="mean", reduction_dim=None,
                            logsumexp_weight: Optional[float] = None, loss_dtype: Optional[torch.dtype] = torch.float32,
                            logit_soft_cap: Optional[float] = None):
    """Cross-entropy of the model on ``example``; MoE auxiliary losses returned by ``activations`` are added
    (src/levanter/models/lm_model.py:256-294)."""
    acts = model.activations(example.tokens, example.attn_mask)
    aux = 0.0
    if isinstance(acts, tuple):
        acts, aux = acts
    head = model.get_lm_head()
    if head.dtype != acts.dtype:
        head = head.to(acts.dtype)
    loss = maybe_fused_next_token_loss(
        acts, head, example.tokens, loss_mask=example.loss_mask, reduction=reduction, reduction_dim=reduction_dim,
        logsumexp_weight=logsumexp_weight, dtype=loss_dtype,
        block_size=getattr(model.config, "cross_entropy_block_size", None), logit_soft_cap=logit_soft_cap)
    return loss + aux
