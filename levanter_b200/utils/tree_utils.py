"""Helpers over nested containers of tensors and modules (src/levanter/utils/tree_utils.py:17-202).

A "tree" here is any nesting of dicts, lists, tuples, dataclasses and ``nn.Module`` objects whose leaves are tensors or
plain Python values."""
from __future__ import annotations

import dataclasses
from enum import Enum
from typing import Any, Dict, Iterator, List, Sequence, Tuple

import torch
import torch.nn as nn


class NonePolicy(str, Enum):
    PRESERVE = "preserve"
    REPLACE = "replace"
    ERROR = "error"


def inference_mode(tree, value: bool, none_policy: str = NonePolicy.REPLACE):
    """Put every module in ``tree`` into inference (``value=True``) or training mode and return the tree.  Objects with an
    ``inference`` attribute that is ``None`` follow ``none_policy`` (src/levanter/utils/tree_utils.py:26-60)."""
    for _, node in _walk(tree, ()):
        if isinstance(node, nn.Module):
            node.train(not value)
        elif hasattr(node, "inference") and not isinstance(node, torch.Tensor):
            if node.inference is None:
                if none_policy == NonePolicy.PRESERVE:
                    continue
                if none_policy == NonePolicy.ERROR:
                    raise ValueError(f"None found in {type(node).__name__}.inference with none_policy={none_policy}")
            try:
                object.__setattr__(node, "inference", value)
            except Exception:  # noqa: BLE001
                pass
    return tree


def _children(node) -> List[Tuple[Any, Any]]:
    if isinstance(node, nn.Module):
        return [(k, v) for k, v in list(node.named_children()) + [(k, p) for k, p in node.named_parameters(recurse=False)]
                + [(k, b) for k, b in node.named_buffers(recurse=False)]]
    if isinstance(node, dict):
        return list(node.items())
    if isinstance(node, (list, tuple)):
        return list(enumerate(node))
    if dataclasses.is_dataclass(node) and not isinstance(node, type):
        return [(f.name, getattr(node, f.name)) for f in dataclasses.fields(node)]
    return []


def _walk(node, path) -> Iterator[Tuple[tuple, Any]]:
    yield path, node
    if isinstance(node, torch.Tensor):
        return
    for k, v in _children(node):
        yield from _walk(v, path + (k,))


def tree_flatten_one_level_with_keys(tree) -> Tuple[List[Tuple[Any, Any]], Any]:
    """The direct children of ``tree`` with their keys, and the node's type as a stand-in for the tree definition."""
    return _children(tree), type(tree)


def key_path_to_str(path: Sequence) -> str:
    """``("layers", 3, "weight") -> "layers.3.weight"`` (src/levanter/utils/tree_utils.py:123-146)."""
    return ".".join(str(p) for p in path)


def leaf_key_paths(tree, prefix: str = "") -> Dict[str, Any]:
    """``{dotted path: leaf}`` for every tensor (or scalar) leaf of ``tree`` (the reference's ``jax_utils.leaf_key_paths``)."""
    out = {}
    for path, node in _walk(tree, ()):
        if isinstance(node, torch.Tensor) or not _children(node) and not isinstance(node, (nn.Module, dict, list, tuple)):
            name = key_path_to_str(path)
            out[f"{prefix}.{name}" if prefix and name else (prefix or name)] = node
    return out


@dataclasses.dataclass(frozen=True)
class PackedLeaf:
    offset: int
    shape: tuple
    dtype: torch.dtype


def pack_pytree(tree, dtype=torch.float32):
    """Concatenate every tensor leaf into one flat ``dtype`` vector; returns ``(tree of PackedLeaf, flat)`` — the form the
    checkpoint of the skip-step optimizer state and the flat-buffer engine use (src/levanter/utils/tree_utils.py:156-187)."""
    flats, offset = [], 0

    def rec(node):
        nonlocal offset
        if isinstance(node, torch.Tensor):
            leaf = PackedLeaf(offset, tuple(node.shape), node.dtype)
            flats.append(node.detach().reshape(-1).to(dtype))
            offset += node.numel()
            return leaf
        if isinstance(node, dict):
            return {k: rec(v) for k, v in node.items()}
        if isinstance(node, (list, tuple)):
            return type(node)(rec(v) for v in node)
        return node

    offsets = rec(tree)
    flat = torch.cat(flats) if flats else torch.zeros(0, dtype=dtype)
    return offsets, flat


def unpack_pytree(offset_tree, packed: torch.Tensor):
    """Inverse of :func:`pack_pytree`."""
    def rec(node):
        if isinstance(node, PackedLeaf):
            n = 1
            for s in node.shape:
                n *= s
            return packed[node.offset:node.offset + n].reshape(node.shape).to(node.dtype)
        if isinstance(node, dict):
            return {k: rec(v) for k, v in node.items()}
        if isinstance(node, (list, tuple)):
            return type(node)(rec(v) for v in node)
        return node

    return rec(offset_tree)
