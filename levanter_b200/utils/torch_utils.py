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


def broadcast_shard(tree, source: int = 0, *, shard_dim: Optional[int] = None, group=None, device=None):
    """A tree of tensors that exists on one process (``source``) arrives on every process of ``group``
    (src/levanter/utils/jax_utils.py:399-455; used by the evaluation harness to ship a packed batch from the process that
    talks to the harness).  The other processes pass a tree of the same structure (contents ignored; shapes and dtypes come
    from the source) or ``None``.  With ``shard_dim`` every process keeps only its equal slice of that axis (its part of the
    batch), otherwise the whole tensor.  Tensors travel over the process group's own transport (NCCL on GPUs, gloo on CPU)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return tree
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    src_global = dist.get_global_rank(group, source) if group is not None else source
    is_src = rank == source
    leaves, rebuild = _flatten_tensors(tree) if is_src else (None, None)
    box = [[(tuple(t.shape), t.dtype) for t in leaves], _structure_of(tree)] if is_src else [None, None]
    dist.broadcast_object_list(box, src=src_global, group=group)
    shapes, structure = box
    backend = dist.get_backend(group)
    dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu"))
    out = []
    for i, (shape, dtype) in enumerate(shapes):
        buf = leaves[i].to(dev).contiguous() if is_src else torch.empty(shape, dtype=dtype, device=dev)
        if buf.numel() > 0:  # as bytes: the transports do not take every dtype
            dist.broadcast(buf.view(-1).view(torch.uint8), src=src_global, group=group)
        if shard_dim is not None and buf.dim() > shard_dim and buf.shape[shard_dim] % world == 0:
            n = buf.shape[shard_dim] // world
            buf = buf.narrow(shard_dim, rank * n, n).contiguous()
        out.append(buf)
    return _rebuild(structure, out)


def _flatten_tensors(tree):
    leaves = []

    def walk(x):
        if isinstance(x, torch.Tensor):
            leaves.append(x)
        elif isinstance(x, dict):
            for k in x:
                walk(x[k])
        elif isinstance(x, (list, tuple)):
            for v in x:
                walk(v)

    walk(tree)
    return leaves, None


def _structure_of(tree):
    """The tree with every tensor replaced by its position in depth-first order (picklable, small)."""
    counter = [0]

    def walk(x):
        if isinstance(x, torch.Tensor):
            counter[0] += 1
            return ("__leaf__", counter[0] - 1)
        if isinstance(x, dict):
            return {k: walk(v) for k, v in x.items()}
        if isinstance(x, tuple):
            return tuple(walk(v) for v in x)
        if isinstance(x, list):
            return [walk(v) for v in x]
        return x

    return walk(tree)


def _rebuild(structure, leaves):
    def walk(x):
        if isinstance(x, tuple) and len(x) == 2 and x[0] == "__leaf__":
            return leaves[x[1]]
        if isinstance(x, dict):
            return {k: walk(v) for k, v in x.items()}
        if isinstance(x, tuple):
            return tuple(walk(v) for v in x)
        if isinstance(x, list):
            return [walk(v) for v in x]
        return x

    return walk(structure)


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
