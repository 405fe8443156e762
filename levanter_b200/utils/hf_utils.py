"""Tokenizer helpers (src/levanter/utils/hf_utils.py:26-60)."""
from __future__ import annotations

import os
import re

from .py_utils import logical_cpu_core_count

_HF_BYTE = re.compile(r"^<0x([0-9A-Fa-f]{2})>$")


def num_cpus_used_by_tokenizer(tokenizer) -> int:
    if getattr(tokenizer, "is_fast", False):
        if os.getenv("TOKENIZERS_PARALLELISM", "true").lower() in {"f", "false", "0", "off", "n", "no"}:
            return 1
        return min(max(1, logical_cpu_core_count() - 4), 12)
    return 1


def byte_length_of_token(tokenizer, idx: int) -> int:
    """UTF-8 bytes a token contributes (special tokens 0, ``<0xNN>`` byte tokens 1); feeds bits-per-byte."""
    if idx in getattr(tokenizer, "all_special_ids", []):
        return 0
    repr_ = tokenizer.convert_ids_to_tokens(idx)
    if repr_ is not None and _HF_BYTE.match(str(repr_)):
        return 1
    # decoding with a prefix token keeps a leading space that a bare decode would strip
    prefix = "."
    pid = tokenizer.convert_tokens_to_ids(prefix)
    if pid is None or pid == getattr(tokenizer, "unk_token_id", None):
        return len(tokenizer.decode([idx]).encode("utf-8"))
    with_prefix = tokenizer.decode([pid, idx])
    only_prefix = tokenizer.decode([pid])
    return len(with_prefix.encode("utf-8")) - len(only_prefix.encode("utf-8"))
