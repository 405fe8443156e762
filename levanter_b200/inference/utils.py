"""Small helpers of the inference engine (src/levanter/inference/utils.py:12-159).  ``INVALID`` marks unused entries of
every index array; negative values are invalid too."""
from __future__ import annotations

from typing import List, Tuple

import numpy as np
import torch

INVALID = 2_000_000


def is_invalid(x, invalid=INVALID):
    return (x < 0) | (x == invalid)


def is_valid(x, invalid=INVALID):
    return (x >= 0) & (x != invalid)


def masked_set(dest, axis: int, start: int, src, num_to_copy: int):
    """``dest[..., start:start + num_to_copy, ...] = src[..., :num_to_copy, ...]`` along ``axis`` (clipped to ``dest``)."""
    n = int(min(num_to_copy, src.shape[axis], max(dest.shape[axis] - start, 0)))
    if n <= 0:
        return dest
    idx_d = [slice(None)] * dest.ndim
    idx_s = [slice(None)] * src.ndim
    idx_d[axis] = slice(start, start + n)
    idx_s[axis] = slice(0, n)
    dest[tuple(idx_d)] = src[tuple(idx_s)]
    return dest


def is_stop_signal(tail_tokens, stop_sequences, invalid=INVALID) -> bool:
    """Does ``tail_tokens[L]`` end with any row of ``stop_sequences[n, L]``?  Rows are *left padded* with ``invalid``; a row
    of only padding never matches."""
    tail = np.asarray(tail_tokens)
    stops = np.asarray(stop_sequences)
    if stops.size == 0:
        return False
    ok = is_valid(stops, invalid)
    has_tokens = ok.any(axis=-1)
    total = ok.sum(axis=-1)
    match = ((tail[None, :] == stops) & (tail[None, :] != invalid)).sum(axis=-1) == total
    return bool((has_tokens & match).any())


def purge_raw(array, mask, max_nnz=None, invalid=INVALID):
    """Drop the entries where ``mask`` is True, slide the rest to the front, pad with ``invalid``."""
    array = np.asarray(array)
    if array.ndim != 1:
        raise ValueError("purge function only supports 1D arrays")
    keep = array[~np.asarray(mask, dtype=bool)]
    n = array.size if max_nnz is None else max_nnz
    out = np.full(n, invalid, dtype=array.dtype)
    out[:min(len(keep), n)] = keep[:n]
    return out


def purge(array, mask, invalid=INVALID):
    return purge_raw(array, mask, invalid=invalid)


def pad_to_standard_length(tokens: np.ndarray, allowed_lengths: List[int], pad_token_id: int) -> np.ndarray:
    cur = tokens.shape[0]
    target = min((n for n in allowed_lengths if n >= cur), default=None)
    if target is None:
        raise ValueError(f"Current length {cur} exceeds all allowed lengths {allowed_lengths}")
    if target > cur:
        tokens = np.concatenate([tokens, np.full((target - cur,), pad_token_id, dtype=tokens.dtype)])
    return tokens


def get_unique_in_order(array, size=None, fill_value=INVALID) -> Tuple[np.ndarray, np.ndarray]:
    """(unique values in order of first appearance padded to ``size``, for each element its index among them)."""
    array = np.asarray(array)
    uniq, first, inverse = np.unique(array, return_index=True, return_inverse=True)
    order = np.argsort(first, kind="stable")
    rank = np.empty_like(order)
    rank[order] = np.arange(len(order))
    uniq_in_order = uniq[order]
    if size is not None:
        out = np.full(size, fill_value, dtype=array.dtype)
        out[:min(size, len(uniq_in_order))] = uniq_in_order[:size]
        uniq_in_order = out
    return uniq_in_order, rank[inverse]
