"""Helpers shared by the entry points: building a model from a framework or Hugging Face checkpoint."""
from __future__ import annotations

import logging
from typing import Optional

import torch

from ..checkpoint import load_checkpoint
from ..models.lm_model import LmConfig, LmHeadModel

logger = logging.getLogger(__name__)


def compute_logits(model: LmHeadModel, example) -> torch.Tensor:
    acts = model.activations(example.tokens, example.attn_mask)
    acts = acts[0] if isinstance(acts, tuple) else acts
    return acts @ model.get_lm_head().to(acts.dtype).t()


def load_model(model_config: LmConfig, tokenizer, *, checkpoint_path: Optional[str] = None, hf_checkpoint=None,
               dtype: Optional[torch.dtype] = None, device=None, vocab_size: Optional[int] = None) -> LmHeadModel:
    """Exactly one of ``checkpoint_path`` (a checkpoint written by this framework) and ``hf_checkpoint`` must be given."""
    if checkpoint_path is None and hf_checkpoint is None:
        raise ValueError("Must specify either checkpoint_path or hf_checkpoint")
    if checkpoint_path is not None and hf_checkpoint is not None:
        raise ValueError("Must specify either checkpoint_path or hf_checkpoint, not both")
    if checkpoint_path is not None:
        model = model_config.build(vocab_size or len(tokenizer), seed=0, device=device)
        model = load_checkpoint(model, checkpoint_path, subpath="model")
        return model.to(dtype) if dtype is not None else model
    if not hasattr(model_config, "hf_checkpoint_converter"):
        raise ValueError("Model config does not have an HF checkpoint converter. Can't load HF checkpoint.")
    converter = model_config.hf_checkpoint_converter().replaced(reference_checkpoint=str(hf_checkpoint), tokenizer=tokenizer)
    return converter.load_pretrained(ref=str(hf_checkpoint), dtype=dtype, device=device)
