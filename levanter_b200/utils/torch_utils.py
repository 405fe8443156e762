"""Device / process helpers that the reference keeps in ``utils/jax_utils.py`` (src/levanter/utils/jax_utils.py:33-469),
restated for PyTorch with one process per GPU."""
from __future__ import annotations

import contextlib
from typing import Any, Iterator, Optional

import torch
import torch.nn as nn

from ..distributed import barrier_sync, broadcast_one_to_all, process_index  # noqa: F401  (re-exported)
from .tree_utils import leaf_key_paths  # noqa: F401


def to_python(a):
    """Tensor -> Python scalar / list; anything else unchanged."""
    if isinstance(a, torch.Tensor):
        return a.item() if a.dim() == 0 else a.tolist()
    return a


@contextlib.contextmanager
def use_cpu_device():
    """Create tensors on the CPU inside the block (checkpoint conversion, dataset statistics)."""
    with torch.device("cpu"):
        yield


def parameter_count(model, need_grad_only: bool = False) -> int:
    """Number of parameters; shared tensors count once (src/levanter/utils/jax_utils.py:71-78)."""
    seen, n = set(), 0
    params = model.parameters() if isinstance(model, nn.Module) else [t for t in leaf_key_paths(model).values() if isinstance(t, torch.Tensor)]
    for p in params:
        if id(p) in seen or (need_grad_only and not p.requires_grad):
            continue
        seen.add(id(p))
        n += p.numel()
    return n


def multihost_broadcast_sync(obj, is_source: Optional[bool] = None, timeout: float = 200.0):
    """Rank 0's ``obj`` on every rank (pickled through the process group)."""
    return broadcast_one_to_all(obj, 0)


def key_iterator(seed: int) -> Iterator[int]:
    """An endless stream of derived seeds (the reference splits a PRNG key)."""
    from ..data.dataset import _fold_in

    i = 0
    while True:
        yield _fold_in(seed, i)
        i += 1


def is_inexact_arrayish(x) -> bool:
    return isinstance(x, torch.Tensor) and (x.is_floating_point() or x.is_complex())


def estimated_free_device_memory(device=None) -> Optional[float]:
    """Free memory of the GPU in GiB, or None without one (src/levanter/utils/jax_utils.py:351-370)."""
    if not torch.cuda.is_available():
        return None
    free, _total = torch.cuda.mem_get_info(device)
    return free / (1 << 30)


def zeros_like_tree(tree, dtype: Optional[torch.dtype] = None):
    if isinstance(tree, torch.Tensor):
        return torch.zeros_like(tree, dtype=dtype or tree.dtype)
    if isinstance(tree, dict):
        return {k: zeros_like_tree(v, dtype) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)):
        return type(tree)(zeros_like_tree(v, dtype) for v in tree)
    return tree


def tree_broadcast_to(prefix, tree):
    """Expand a prefix tree (for example one bool) to the structure of ``tree``."""
    if isinstance(tree, dict):
        return {k: tree_broadcast_to(prefix[k] if isinstance(prefix, dict) else prefix, v) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)):
        return type(tree)(tree_broadcast_to(prefix[i] if isinstance(prefix, (list, tuple)) else prefix, v) for i, v in enumerate(tree))
    return prefix
