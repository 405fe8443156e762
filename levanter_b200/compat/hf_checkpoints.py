"""Hugging Face checkpoint import/export (placeholder header; the full converter is defined below)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..models.lm_model import LmConfig


@dataclass(frozen=True)
class HFCompatConfig(LmConfig):
    def hf_checkpoint_converter(self, ref_checkpoint: Optional[str] = None) -> "HFCheckpointConverter":
        raise NotImplementedError

    @classmethod
    def from_hf_config(cls, hf_config):
        raise NotImplementedError

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[dict] = None) -> dict:
        raise NotImplementedError


class HFCheckpointConverter:
    def __init__(self, config_class, reference_checkpoint=None, tokenizer=None, **kw):
        self.config_class = config_class
        self.reference_checkpoint = reference_checkpoint
        self.tokenizer_name = tokenizer
