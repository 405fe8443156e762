"""Write / read a state tree as one zarr array per leaf, at ``<path>/<key path with '.' -> '/'>``
(src/levanter/tensorstore_serialization.py:36-215).

Key paths follow the reference's ``leaf_key_paths``: dataclass / NamedTuple field names, tuple and list indices, dict keys.
Model parameters and the optimizer moments that mirror them are converted to the reference's layout on the way out:
per-layer tensors ``transformer.layers.<i>.x`` are stacked under ``transformer/layers/stacked/x`` with a leading layer
axis, 2-D ``[out, in]`` Linear weights are reshaped to their articulated axes (and transposed for ``out_first=False``
modules).  Loading inverts this, accepts arbitrary chunk grids, and reshards to whatever mesh is running.

Leaves may be ``DeferredLeaf`` objects (sharded tensors gathered only while they are being written); every rank resolves
every leaf in the same order (the gathers are collectives) and leaf ``i`` is written by rank ``i mod world``."""
from __future__ import annotations

import json
import logging
import re
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass, fields, is_dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from .store.zarr_array import ZarrArray, default_chunks
from .utils import fsspec_utils

logger = logging.getLogger(__name__)
_LAYER_RE = re.compile(r"^(.*?\.)?(layers|blocks|h)\.(\d+)\.(.*)$")


class DeferredLeaf:
    """A tensor produced on demand (e.g. an all-gather of optimizer-state shards)."""

    def __init__(self, fn: Callable[[], torch.Tensor], shape: Tuple[int, ...], dtype: torch.dtype):
        self.fn = fn
        self.shape = tuple(shape)
        self.dtype = dtype

    def resolve(self) -> torch.Tensor:
        return self.fn()


@dataclass
class ParamLayout:
    """How one torch parameter maps to the reference's array: articulated shape and whether it is stored transposed."""

    lev_shape: Tuple[int, ...]
    transposed: bool = False
    permute: Optional[Tuple[int, ...]] = None  # reference array = param.permute(permute).reshape(lev_shape)


def layouts_of(model: torch.nn.Module) -> Dict[str, ParamLayout]:
    out = {}
    for name, p in model.named_parameters():
        shape = tuple(getattr(p, "lev_shape", tuple(p.shape)))
        out[name] = ParamLayout(shape, bool(getattr(p, "lev_transposed", False)), getattr(p, "lev_permute", None))
    return out


# ------------------------------------------------------------------------------------------------ key paths
_LEAF_TYPES = (torch.Tensor, np.ndarray, int, float, bool, np.generic)


def keyed_children(x) -> Optional[List[Tuple[Any, Any]]]:
    """``[(key, child)]`` of a container node of a state tree, ``None`` for leaves and static values.  Keys are NamedTuple /
    dataclass field names, dict keys and sequence indices; an object with ``checkpoint_children()`` chooses its own keys."""
    if x is None or isinstance(x, _LEAF_TYPES) or isinstance(x, DeferredLeaf):
        return None
    if hasattr(x, "checkpoint_children"):
        return list(x.checkpoint_children())
    if isinstance(x, tuple) and hasattr(x, "_fields"):
        return [(f, getattr(x, f)) for f in x._fields]
    if is_dataclass(x) and not isinstance(x, type):
        return [(f.name, getattr(x, f.name)) for f in fields(x)]
    if isinstance(x, dict):
        return list(x.items())
    if isinstance(x, (list, tuple)):
        return list(enumerate(x))
    return None


def rebuild_from_children(x, values: Sequence[Any]):
    """The container ``x`` with its children (in :func:`keyed_children` order) replaced by ``values``."""
    values = list(values)
    if hasattr(x, "with_checkpoint_children"):
        return x.with_checkpoint_children(values)
    if isinstance(x, tuple) and hasattr(x, "_fields"):
        return type(x)(*values)
    if is_dataclass(x) and not isinstance(x, type):
        import dataclasses

        return dataclasses.replace(x, **{f.name: v for f, v in zip(fields(x), values)})
    if isinstance(x, dict):
        return {k: v for k, v in zip(x.keys(), values)}
    if isinstance(x, tuple):
        return tuple(values)
    if isinstance(x, list):
        return values
    raise TypeError(f"not a container: {type(x)}")


def leaf_key_paths(tree: Any, prefix: str = "") -> List[Tuple[str, Any]]:
    """Flatten ``tree`` into ``(dotted key path, leaf)`` pairs; ``None`` leaves are skipped
    (src/levanter/utils/jax_utils.py:150-223)."""
    out: List[Tuple[str, Any]] = []

    def rec(x, p):
        if x is None:
            return
        if isinstance(x, _LEAF_TYPES) or isinstance(x, DeferredLeaf):
            out.append((p, x))
            return
        children = keyed_children(x)
        # anything else (callables, strings) is static configuration, not state
        for k, v in children or ():
            rec(v, f"{p}.{k}" if p else str(k))

    rec(tree, prefix)
    return out


def _fs_path(base: str, key_path: str) -> str:
    return fsspec_utils.join_path(base, key_path.replace(".", "/")) if key_path else base


# ------------------------------------------------------------------------------------------------ layout conversion
def _is_param_dict(d) -> bool:
    return isinstance(d, dict) and len(d) > 0 and all(isinstance(k, str) for k in d) and \
        all(v is None or isinstance(v, (torch.Tensor, DeferredLeaf)) for v in d.values()) and \
        any(k.endswith((".weight", ".bias")) or k in ("weight", "bias") or "." in k for k in d)


def to_reference_layout(params: Dict[str, Any], layouts: Optional[Dict[str, ParamLayout]]) -> Dict[str, Any]:
    """torch-named flat dict -> nested dict in the reference's layout (stacked layers, articulated axes)."""
    groups: Dict[str, Dict[int, Tuple[str, Any]]] = {}
    singles: Dict[str, Any] = {}
    for name, t in params.items():
        if t is None:
            continue
        m = _LAYER_RE.match(name)
        if m:
            pre, coll, idx, rest = m.group(1) or "", m.group(2), int(m.group(3)), m.group(4)
            groups.setdefault(f"{pre}{coll}.stacked.{rest}", {})[idx] = (name, t)
        else:
            singles[name] = t

    def articulate(name, t):
        lay = layouts.get(name) if layouts else None

        def conv(x: torch.Tensor) -> torch.Tensor:
            if lay is None:
                return x
            if lay.permute is not None:
                x = x.permute(*lay.permute)
            elif lay.transposed and x.dim() == 2:
                x = x.t()
            return x.reshape(lay.lev_shape)

        if isinstance(t, DeferredLeaf):
            shape = lay.lev_shape if lay is not None else t.shape
            return DeferredLeaf(lambda t=t: conv(t.resolve()), shape, t.dtype)
        return conv(t)

    flat: Dict[str, Any] = {}
    for name, t in singles.items():
        flat[name] = articulate(name, t)
    for key, members in groups.items():
        idxs = sorted(members)
        items = [articulate(*members[i]) for i in idxs]
        shape = (len(items),) + tuple(items[0].shape)
        dtype = items[0].dtype

        def stack(items=items):
            return torch.stack([(x.resolve() if isinstance(x, DeferredLeaf) else x) for x in items])

        flat[key] = DeferredLeaf(stack, shape, dtype)
    return _nest(flat)


def _nest(flat: Dict[str, Any]) -> Dict[str, Any]:
    root: Dict[str, Any] = {}
    for k, v in flat.items():
        cur = root
        parts = k.split(".")
        for p in parts[:-1]:
            cur = cur.setdefault(p, {})
        cur[parts[-1]] = v
    return root


def convert_state_for_save(state: Any, layouts: Optional[Dict[str, ParamLayout]]) -> Any:
    """Apply :func:`to_reference_layout` to every parameter-shaped dict inside ``state``."""
    if _is_param_dict(state):
        return to_reference_layout(state, layouts)
    if isinstance(state, tuple) and hasattr(state, "_fields"):
        return type(state)(*[convert_state_for_save(v, layouts) for v in state])
    if isinstance(state, tuple):
        return tuple(convert_state_for_save(v, layouts) for v in state)
    if isinstance(state, list):
        return [convert_state_for_save(v, layouts) for v in state]
    if isinstance(state, dict):
        return {k: convert_state_for_save(v, layouts) for k, v in state.items()}
    return state


def reference_key_for(name: str) -> Tuple[str, Optional[int]]:
    """torch parameter name -> (reference key path, layer index or None)."""
    m = _LAYER_RE.match(name)
    if m:
        pre, coll, idx, rest = m.group(1) or "", m.group(2), int(m.group(3)), m.group(4)
        return f"{pre}{coll}.stacked.{rest}", idx
    return name, None


# ------------------------------------------------------------------------------------------------ save
class AsyncSerializer:
    """Background writer: ``serialize`` returns once every leaf has been copied to host memory; chunk compression and
    file writes proceed on a thread pool.  A committer thread joins each save's writes as soon as they finish, agrees with
    the other ranks that all of them are done, and then runs the save's commit callback, so a save made in the middle of a
    run becomes discoverable shortly after its writes complete, not when the run ends (the reference commits from its async
    manager's background thread, src/levanter/tensorstore_serialization.py:36-96).

    The ranks agree through marker files under ``<sync_dir>/.commit/`` (collectives must not be issued off the main
    thread): every rank drops ``rank-<r>-<save id>`` when its own writes are durable; rank 0 waits for all of them, runs its callback
    (which writes ``metadata.json``) and drops ``done-<save id>``; the other ranks run theirs once that file exists."""

    COMMIT_TIMEOUT_S = 1800.0

    def __init__(self, max_workers: int = 8):
        self._pool = ThreadPoolExecutor(max_workers=max_workers)
        self._lock = threading.Lock()
        self._idle = threading.Condition(self._lock)
        self._queue: List[Tuple[List[Future], Optional[Callable[[], None]], Optional[str], int, int, str, frozenset]] = []
        self._in_flight = 0
        self._busy_paths: set = set()  # leaf directories that a queued or running save still writes
        self._errors: List[BaseException] = []
        self._committer: Optional[threading.Thread] = None

    def serialize(self, leaves: Sequence[Tuple[str, Any]], on_commit: Optional[Callable[[], None]] = None,
                  sync_dir: Optional[str] = None) -> None:
        rank = dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0
        world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
        futures: List[Future] = []
        leaves = list(leaves)
        mine = frozenset(str(path) for i, (path, _) in enumerate(leaves) if i % world == rank)
        with self._lock:
            # a second save into the same directory (the same step saved again) starts by clearing each leaf's directory:
            # it must not do that under the first save's writers
            while self._in_flight > 0 and (mine & self._busy_paths):
                self._idle.wait(timeout=1.0)
            self._busy_paths |= mine
        for i, (path, leaf) in enumerate(leaves):
            t = leaf.resolve() if isinstance(leaf, DeferredLeaf) else leaf
            if i % world != rank:
                continue
            if isinstance(t, (int, float, bool, np.generic)):
                t = torch.tensor(t)
            elif isinstance(t, np.ndarray):
                t = torch.from_numpy(np.ascontiguousarray(t))
            host = t.detach().to("cpu", copy=True) if t.device.type != "cpu" else t.detach().clone()
            futures.append(self._pool.submit(_write_leaf, path, host))
        nonce = ""
        if world > 1 and sync_dir is not None:
            # a name for this save that every rank knows (a directory can be written more than once, e.g. after a resume)
            import uuid

            box = [uuid.uuid4().hex[:12] if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            nonce = box[0]
        with self._lock:
            self._queue.append((futures, on_commit, sync_dir, rank, world, nonce, mine))
            self._in_flight += 1
            if self._committer is None or not self._committer.is_alive():
                self._committer = threading.Thread(target=self._commit_loop, name="checkpoint-committer", daemon=True)
                self._committer.start()
            self._idle.notify_all()

    def _commit_loop(self) -> None:
        while True:
            with self._lock:
                while not self._queue:
                    if not self._idle.wait(timeout=5.0) and not self._queue:
                        self._committer = None
                        return
                item = self._queue.pop(0)
            try:
                self._commit_one(*item[:6])
            except BaseException as e:  # noqa: BLE001 - reported to the thread that calls wait_until_finished
                logger.exception("checkpoint commit failed")
                with self._lock:
                    self._errors.append(e)
            finally:
                with self._lock:
                    self._in_flight -= 1
                    self._busy_paths -= item[6]
                    self._idle.notify_all()

    def _commit_one(self, futures, cb, sync_dir, rank, world, nonce) -> None:
        import time

        for f in futures:
            f.result()
        if world > 1 and sync_dir is not None:
            from fsspec.core import url_to_fs

            fs, plain = url_to_fs(str(sync_dir))
            cdir = plain.rstrip("/") + "/.commit"
            fs.makedirs(cdir, exist_ok=True)
            with fs.open(f"{cdir}/rank-{rank}-{nonce}", "w") as fh:
                fh.write("ok")
            deadline = time.monotonic() + self.COMMIT_TIMEOUT_S
            want = [f"{cdir}/rank-{r}-{nonce}" for r in range(world)] if rank == 0 else [f"{cdir}/done-{nonce}"]
            while not all(fs.exists(w) for w in want):
                if time.monotonic() > deadline:
                    raise TimeoutError(f"ranks did not all finish writing {sync_dir} within {self.COMMIT_TIMEOUT_S:.0f} s")
                time.sleep(0.05)
                try:
                    fs.invalidate_cache(cdir)
                except Exception:  # noqa: BLE001
                    pass
            if rank == 0:
                if cb is not None:
                    cb()
                with fs.open(f"{cdir}/done-{nonce}", "w") as fh:
                    fh.write("ok")
                for r in range(world):
                    try:
                        fs.rm(f"{cdir}/rank-{r}-{nonce}")
                    except Exception:  # noqa: BLE001
                        pass
                return
        if cb is not None:
            cb()

    def drain(self) -> None:
        """Non-blocking: raise an error a finished commit left behind (called from the step loop)."""
        with self._lock:
            errs, self._errors = self._errors, []
        if errs:
            raise errs[0]

    def wait_until_finished(self) -> None:
        with self._lock:
            while self._in_flight > 0:
                self._idle.wait(timeout=1.0)
            errs, self._errors = self._errors, []
        if errs:
            raise errs[0]


def _write_leaf(path: str, t: torch.Tensor) -> None:
    itemsize = t.element_size()
    arr = ZarrArray.create(path, list(t.shape), default_chunks(list(t.shape), itemsize), t.dtype)
    arr.write_tensor(t)


def tree_serialize_leaves_tensorstore(checkpoint_dir: str, tree: Any, manager: Optional[AsyncSerializer] = None, *,
                                      commit_callback: Optional[Callable[[], None]] = None,
                                      layouts: Optional[Dict[str, ParamLayout]] = None) -> None:
    own = manager is None
    manager = manager or AsyncSerializer()
    tree = convert_state_for_save(tree, layouts)
    leaves = [(_fs_path(checkpoint_dir, kp), leaf) for kp, leaf in leaf_key_paths(tree)]
    manager.serialize(leaves, on_commit=commit_callback, sync_dir=checkpoint_dir)
    if own:
        manager.wait_until_finished()


# ------------------------------------------------------------------------------------------------ load
def read_leaf(checkpoint_dir: str, key_path: str) -> Optional[torch.Tensor]:
    p = _fs_path(checkpoint_dir, key_path)
    if not ZarrArray.exists(p):
        return None
    return ZarrArray.open(p).read_tensor()


def read_param(checkpoint_dir: str, prefix: str, name: str, layout: Optional[ParamLayout], shape: Tuple[int, ...]) -> Optional[torch.Tensor]:
    """Read torch parameter ``name`` from a reference-layout checkpoint under ``prefix`` (e.g. ``model``): picks the
    layer row of a stacked array and undoes the articulated reshape / transpose."""
    key, layer = reference_key_for(name)
    p = _fs_path(checkpoint_dir, f"{prefix}.{key}" if prefix else key)
    if not ZarrArray.exists(p):
        return None
    arr = ZarrArray.open(p)
    if layer is not None:
        lo = [layer] + [0] * (len(arr.shape) - 1)
        hi = [layer + 1] + list(arr.shape[1:])
        t = arr.read_tensor(lo, hi)[0]
    else:
        t = arr.read_tensor()
    if layout is not None and layout.permute is not None:
        perm = layout.permute
        permuted_shape = [shape[i] for i in perm]
        inv = [perm.index(i) for i in range(len(perm))]
        return t.reshape(permuted_shape).permute(*inv).contiguous()
    if layout is not None and layout.transposed and len(shape) == 2:
        t = t.reshape(shape[1], shape[0]).t()
    return t.reshape(shape)


def tree_deserialize_leaves_tensorstore(checkpoint_dir: str, tree: Any, *, allow_missing: bool = False) -> Any:
    """Read every leaf of ``tree`` (used as a structure exemplar) from ``checkpoint_dir``; with ``allow_missing`` leaves
    absent on disk keep their exemplar value (src/levanter/tensorstore_serialization.py:119-215)."""

    def rec(x, p):
        if x is None:
            return None
        if isinstance(x, (torch.Tensor, np.ndarray, int, float, bool, np.generic)):
            t = read_leaf(checkpoint_dir, p)
            if t is None:
                if allow_missing:
                    return x
                raise FileNotFoundError(f"Missing checkpoint leaf {p} in {checkpoint_dir}")
            if isinstance(x, bool):
                return bool(t.item())
            if isinstance(x, int):
                return int(t.item())
            if isinstance(x, float):
                return float(t.item())
            if isinstance(x, torch.Tensor):
                return t.to(dtype=x.dtype).reshape(x.shape).to(x.device)
            return t.numpy()
        children = keyed_children(x)
        if children is None:
            return x
        return rebuild_from_children(x, [rec(v, f"{p}.{k}" if p else str(k)) for k, v in children])

    return rec(tree, "")
