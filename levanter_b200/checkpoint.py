"""Checkpointing (src/levanter/checkpoint.py): save policies, asynchronous writes, discovery, resume.

Layout: ``<base_path>/<run_id>/step-<N>/`` holds ``metadata.json`` = ``{"step", "timestamp", "is_temporary"}`` and one
zarr array per leaf of the saveable state (``step``, ``model/...``, ``opt_state/...``, ``training_key``,
``model_averaging/...``), written in the reference's key-path and array layout
(:348-400, src/levanter/tensorstore_serialization.py:91-96).

Policies: *permanent* checkpoints every ``every`` steps (per ``keep`` interval list) and *temporary* time-based
checkpoints every ``save_interval`` that are deleted once the next checkpoint commits (:170-245).  Process 0 decides
and broadcasts the decision so clock skew cannot split the processes.  A checkpoint written on N GPUs loads on any other
count: parameters and optimizer moments are full arrays on disk and every rank keeps only its slices."""
from __future__ import annotations

import dataclasses
import datetime
import json
import logging
import os
import queue
import threading
import time
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Any, Callable, Dict, List, Optional, Sequence

import fsspec
import torch
import torch.distributed as dist
from fsspec.core import url_to_fs

from . import tensorstore_serialization as tss
from .distributed import broadcast_one_to_all
from .utils import fsspec_utils

logger = logging.getLogger(__name__)
PathLike = Any


def _rank() -> int:
    return dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0


@dataclass(frozen=True)
class CheckpointInterval:
    every: int
    until: Optional[int] = None  # None = forever


class Checkpointer:
    def __init__(self, base_path: PathLike, save_interval: Optional[datetime.timedelta],
                 step_policies: Sequence[CheckpointInterval], *, dt_now_injection: Optional[Callable[[], datetime.datetime]] = None,
                 delete_old_temp_checkpoints: bool = True):
        self.base_path = str(base_path)
        self.save_interval = save_interval
        self.step_policies = list(step_policies)
        self._dt_now_injection = dt_now_injection or datetime.datetime.now
        self._last_save_time = self._dt_now_injection()
        self._last_save_step = 0
        for i in range(1, len(self.step_policies)):
            prev_until, until = self.step_policies[i - 1].until, self.step_policies[i].until
            if prev_until is None:
                raise ValueError("Only the last step policy can have an 'until' value of None")
            if until is None:
                continue
            if prev_until >= until:
                raise ValueError("Step policies must be sorted by 'until' value")
        self._manager = tss.AsyncSerializer()
        self._remover_queue: "queue.Queue[str]" = queue.Queue()
        self._being_removed: Optional[str] = None
        if _rank() == 0:
            self._remover_thread = threading.Thread(target=self._async_checkpoint_remover, daemon=True)
            self._remover_thread.start()
        self._last_temporary_checkpoint: Optional[str] = None
        latest = discover_latest_checkpoint(self.base_path)
        if latest is not None and delete_old_temp_checkpoints:
            try:
                if _load_metadata(latest).get("is_temporary", False):
                    logger.info(f"Found prior temporary checkpoint {latest}. We will delete it after saving a new checkpoint.")
                    self._last_temporary_checkpoint = latest
            except FileNotFoundError:
                pass

    def load_checkpoint(self, state, path: Optional[str] = None, *, discover_latest: bool = True, **kw):
        return load_checkpoint(state, path or self.base_path, discover_latest=discover_latest, **kw)

    def load_model(self, model: torch.nn.Module, path: Optional[str] = None, *, discover_latest: bool = True, **kw):
        """Only the model, from the ``model`` sub-tree of the (newest) checkpoint under ``path`` (src/levanter/checkpoint.py:150-168)."""
        return load_checkpoint(model, path or self.base_path, subpath="model", discover_latest=discover_latest, **kw)

    def on_step(self, info, force: bool = False):
        step = info.step
        self._manager.drain()  # surface an error from a commit that finished in the background
        if step == 0:
            self._last_save_time = self._dt_now_injection()
            if not force:
                return
        if step == self._last_save_step and not force:
            return
        my_should_save = force
        my_permanent = force
        every = self._get_current_step_save_interval(step)
        elapsed = self._dt_now_injection() - self._last_save_time
        if every is not None and step % every == 0:
            my_should_save, my_permanent = True, True
        elif self.save_interval and elapsed >= self.save_interval:
            my_should_save, my_permanent = True, False
        should_save, permanent = broadcast_one_to_all((bool(my_should_save), bool(my_permanent)))
        if not should_save:
            return
        logger.info(f"Saving {'' if permanent else 'temporary '}checkpoint at step {step}.")
        last = self._last_temporary_checkpoint
        destination = f"step-{step}"
        self._last_temporary_checkpoint = None if permanent else os.path.join(self.base_path, destination)

        def callback():
            if last is not None:
                try:
                    if _load_metadata(last).get("is_temporary", False):
                        logger.info(f"Deleting old temporary checkpoint {last} after saving new checkpoint.")
                        self._rm_checkpoint(last)
                    else:
                        logger.info(f"Not deleting old temporary checkpoint {last} because it is no longer temporary.")
                except FileNotFoundError:
                    logger.warning(f"Could not load metadata for last temporary checkpoint {last}.")

        self.save_checkpoint(info, destination, commit_callback=callback, is_temporary=not permanent)

    def _get_current_step_save_interval(self, step: int) -> Optional[int]:
        pol = next((p for p in self.step_policies if p.until is None or p.until >= step), None)
        return None if pol is None else pol.every

    def wait_until_finished(self):
        self._manager.wait_until_finished()
        if _rank() == 0:
            while self._being_removed is not None or not self._remover_queue.empty():
                time.sleep(0.05)

    def _rm_checkpoint(self, checkpoint: str):
        if _rank() == 0:
            self._remover_queue.put(checkpoint)

    def _async_checkpoint_remover(self):
        while True:
            ckpt = self._remover_queue.get(block=True)
            self._being_removed = ckpt
            try:
                fs, plain = url_to_fs(ckpt)
                fs.rm(plain, recursive=True)
                logger.info(f"Deleted checkpoint {ckpt}")
            except Exception:  # noqa: BLE001
                logger.exception(f"Failed to delete checkpoint {ckpt}")
            finally:
                self._being_removed = None

    def save_checkpoint(self, info, destination: str, commit_callback: Optional[Callable[[], None]] = None, *,
                        is_temporary: bool = False):
        path = os.path.join(self.base_path, destination)
        logger.info(f"Saving checkpoint at step {info.step} to {path}")
        state = info.state
        save_checkpoint(state.saveable_state, step=info.step, checkpoint_path=path, manager=self._manager,
                        commit_callback=commit_callback, is_temporary=is_temporary, layouts=tss.layouts_of(state.model))
        self._last_save_step = info.step
        self._last_save_time = self._dt_now_injection()


class EpochCheckpointer:
    """Checkpoint every ``every_n_epochs`` epochs of a finite dataset (src/levanter/checkpoint.py:311-345)."""

    def __init__(self, checkpointer: Checkpointer, every_n_epochs: int = 1, total_dataset_size: Optional[int] = None,
                 batch_size: int = 1):
        self.checkpointer = checkpointer
        self.every_n_epochs = every_n_epochs
        self.total_dataset_size = total_dataset_size
        self.batch_size = batch_size
        self._last_saved_epoch = -1

    def on_step(self, info, force: bool = False):
        if self.total_dataset_size is None:
            return
        epoch = (self.batch_size * info.step) // self.total_dataset_size
        if epoch % self.every_n_epochs == 0 and epoch != self._last_saved_epoch:
            self.checkpointer.save_checkpoint(info, f"epoch-{epoch}", is_temporary=True)
            self._last_saved_epoch = epoch


def save_checkpoint(tree: Any, step: int, checkpoint_path: PathLike, manager: Optional[tss.AsyncSerializer] = None, *,
                    commit_callback: Optional[Callable[[], None]] = None, is_temporary: bool = False,
                    layouts: Optional[Dict[str, tss.ParamLayout]] = None):
    """Write ``tree`` under ``checkpoint_path``; ``metadata.json`` is written by process 0 once every leaf is durable."""
    checkpoint_path = str(checkpoint_path)
    fsspec_utils.mkdirs(checkpoint_path)

    def my_callback():
        if _rank() == 0:
            _save_metadata(checkpoint_path, step, is_temporary)
        logger.info("Saved checkpoint to %s", checkpoint_path)
        if commit_callback is not None:
            commit_callback()

    own = manager is None
    manager = manager or tss.AsyncSerializer()
    tss.tree_serialize_leaves_tensorstore(checkpoint_path, tree, manager, commit_callback=my_callback, layouts=layouts)
    if own:
        manager.wait_until_finished()
    return checkpoint_path


def _save_metadata(checkpoint_path: str, step: int, is_temporary: bool):
    metadata = {"step": int(step), "timestamp": datetime.datetime.now().isoformat(), "is_temporary": bool(is_temporary)}
    fs, plain = url_to_fs(checkpoint_path)
    with fs.open(os.path.join(plain, "metadata.json"), "w") as f:
        json.dump(metadata, f)


def _load_metadata(checkpoint_path: str) -> dict:
    fs, plain = url_to_fs(str(checkpoint_path))
    with fs.open(os.path.join(plain, "metadata.json"), "r") as f:
        return json.load(f)


def is_checkpoint_path(path: PathLike) -> bool:
    fs, plain = url_to_fs(str(path))
    return fs.exists(os.path.join(plain, "metadata.json"))


def discover_latest_checkpoint(checkpoint_path: PathLike) -> Optional[str]:
    """Newest checkpoint under ``checkpoint_path`` by ``(timestamp, step)`` of its metadata; ``checkpoint_path`` itself if
    it is a checkpoint (src/levanter/checkpoint.py:571-603)."""
    checkpoint_path = str(checkpoint_path)
    fs, plain = url_to_fs(checkpoint_path)
    if not fs.exists(plain):
        return None
    if fs.exists(os.path.join(plain, "metadata.json")):
        return checkpoint_path
    candidates = []
    try:
        metas = fs.glob(os.path.join(plain, "*", "metadata.json"))
    except Exception:
        metas = []
    for m in metas:
        try:
            with fs.open(m, "r") as f:
                md = json.load(f)
            ts = datetime.datetime.fromisoformat(md["timestamp"])
            candidates.append(((ts, md["step"]), os.path.dirname(m)))
        except Exception:  # noqa: BLE001
            logger.exception(f"Error reading metadata {m}")
    if not candidates:
        logger.warning(f"No checkpoints found in {checkpoint_path}")
        return None
    best = max(candidates, key=lambda c: c[0])[1]
    if "://" in checkpoint_path and "://" not in best:
        best = checkpoint_path.split("://")[0] + "://" + best
    return best


# ------------------------------------------------------------------------------------------------ loading
def load_checkpoint(state, checkpoint_path: PathLike, *, subpath: Optional[str] = None, discover_latest: bool = True,
                    allow_partial: bool = False):
    """Restore a ``TrainerState`` (or, with ``subpath="model"``, just a model) in place from a checkpoint directory.

    ``state`` may be a ``TrainerState``, an ``nn.Module``, or any tree of tensors and scalars written by
    :func:`save_checkpoint` (returned as a new tree; with ``allow_partial`` leaves that are not in the checkpoint keep their
    value).  Raises ``FileNotFoundError`` when nothing is found."""
    checkpoint_path = str(checkpoint_path)
    if discover_latest:
        found = discover_latest_checkpoint(checkpoint_path)
        if found is None:
            raise FileNotFoundError(f"Could not find checkpoint at {checkpoint_path}")
        checkpoint_path = found
    logger.info(f"Loading checkpoint from {checkpoint_path}")
    if isinstance(state, torch.nn.Module):
        prefix = subpath or ""
        load_model_params(state, checkpoint_path, prefix, allow_partial=allow_partial)
        return state
    if not hasattr(state, "engine"):
        where = checkpoint_path if not subpath else fsspec_utils.join_path(checkpoint_path, subpath.replace(".", "/"))
        return tss.tree_deserialize_leaves_tensorstore(where, state, allow_missing=allow_partial)
    return _load_trainer_state(state, checkpoint_path, allow_partial=allow_partial)


def load_model_params(model: torch.nn.Module, checkpoint_path: str, prefix: str = "model", *, allow_partial: bool = False,
                      only: Optional[Callable[[str], bool]] = None) -> List[str]:
    """Copy parameters from a reference-layout checkpoint into ``model``.  Returns the names that were missing."""
    layouts = tss.layouts_of(model)
    missing = []
    with torch.no_grad():
        for name, p in model.named_parameters():
            if only is not None and not only(name):
                continue
            t = tss.read_param(checkpoint_path, prefix, name, layouts.get(name), tuple(p.shape))
            if t is None:
                missing.append(name)
                continue
            p.data.copy_(t.to(device=p.device, dtype=p.dtype))
    if missing and not allow_partial:
        raise FileNotFoundError(f"Missing parameters in checkpoint {checkpoint_path}: {missing[:5]}{'...' if len(missing) > 5 else ''}")
    return missing


def _load_trainer_state(state, checkpoint_path: str, *, allow_partial: bool):
    from .optim import transforms as T
    from .parallel.engine import _is_param_tree

    engine = state.engine
    layouts = tss.layouts_of(state.model)
    shapes = {s.name: s.shape for s in engine.slots}
    slot_of = {s.name: s for s in engine.slots}

    def read_own(prefix: str, name: str):
        """This rank's part of a saved parameter-shaped leaf: all of it, or (expert-parallel parameters, which checkpoints hold
        with every expert) its slice of the experts."""
        slot = slot_of[name]
        full = tss.read_param(checkpoint_path, prefix, name, layouts.get(name), engine._full_shape(slot))
        return None if full is None else engine._own_part(slot, full)
    missing: List[str] = []

    def fill_shard(prefix: str, shard: torch.Tensor, names: Optional[Sequence[str]] = None):
        for name in (names if names is not None else engine.segments.keys()):
            seg = engine.segments.get(name)
            if seg is None:
                continue
            full = read_own(prefix, name)
            if full is None:
                missing.append(f"{prefix}.{name}")
                continue
            lo, fo, n = seg
            slot = next(s for s in engine.slots if s.name == name)
            a = fo - slot.offset
            shard[lo:lo + n].copy_(full.reshape(-1)[a:a + n].to(device=shard.device, dtype=shard.dtype))

    with torch.no_grad():
        # parameters: master slices, then the compute-dtype copies everywhere
        for s in engine.slots:
            full = read_own("model", s.name)
            if full is None:
                missing.append(f"model.{s.name}")
                continue
            if not s.streamed:  # (a streamed matrix is a view of a staging slot, filled when its layer is assembled)
                s.param.data.copy_(full.to(device=engine.device, dtype=s.param.dtype))
            seg = engine.segments.get(s.name)
            if seg is not None and not engine.master_is_param:
                lo, fo, n = seg
                a = fo - s.offset
                engine.master[lo:lo + n].copy_(full.reshape(-1)[a:a + n].to(device=engine.device, dtype=engine.master.dtype))
        # optimizer state
        if engine.fused_adam is not None:
            fa = engine.fused_adam
            cnt = tss.read_leaf(checkpoint_path, "opt_state.count")
            if cnt is not None:
                fa.count = int(cnt.item())
            idx = 1 if fa.cfg.max_grad_norm else 0
            fill_shard(f"opt_state.inner_state.{idx}.mu", fa.m)
            fill_shard(f"opt_state.inner_state.{idx}.nu", fa.v)
        elif engine.opt_state is not None:
            def rec(x, p):
                if _is_param_tree(x):
                    for name, leaf in x.items():
                        if leaf is None:
                            continue
                        full = read_own(p, name)
                        if full is None:
                            missing.append(f"{p}.{name}")
                            continue
                        lo, fo, n = engine.segments[name]
                        slot = next(s for s in engine.slots if s.name == name)
                        a = fo - slot.offset
                        leaf.copy_(full.reshape(-1)[a:a + n].to(device=leaf.device, dtype=leaf.dtype).reshape(leaf.shape))
                    return x
                children = tss.keyed_children(x)
                if children is not None:
                    return tss.rebuild_from_children(x, [rec(v, f"{p}.{k}" if p else str(k)) for k, v in children])
                if isinstance(x, (int, float, bool)) or isinstance(x, torch.Tensor):
                    t = tss.read_leaf(checkpoint_path, p)
                    if t is None:
                        missing.append(p)
                        return x
                    if isinstance(x, bool):
                        return bool(t.item())
                    if isinstance(x, int):
                        return int(t.item())
                    if isinstance(x, float):
                        return float(t.item())
                    return t.to(dtype=x.dtype).reshape(x.shape)
                return x

            engine.opt_state = rec(engine.opt_state, "opt_state")
        if state.model_averaging is not None:
            for name, leaf in state.model_averaging.model_params.items():
                full = read_own("model_averaging.model", name)
                if full is None:
                    missing.append(f"model_averaging.model.{name}")
                    continue
                lo, fo, n = engine.segments[name]
                slot = next(s for s in engine.slots if s.name == name)
                a = fo - slot.offset
                leaf.copy_(full.reshape(-1)[a:a + n].to(device=leaf.device, dtype=leaf.dtype).reshape(leaf.shape))
            if hasattr(state.model_averaging, "tot_weight"):  # the running weight of the decay phase is state too
                w = tss.read_leaf(checkpoint_path, "model_averaging.tot_weight")
                if w is not None:
                    state.model_averaging.tot_weight = float(w.item())
                else:
                    missing.append("model_averaging.tot_weight")
    engine.sync_streamed_from_master()  # fully sharded layers: peers gather from the compute-dtype rows, refresh them
    step = tss.read_leaf(checkpoint_path, "step")
    if step is None:
        step = torch.tensor(_load_metadata(checkpoint_path)["step"] + 1)
    state.step = int(step.item())
    key = tss.read_leaf(checkpoint_path, "training_key")
    if key is not None:
        state.training_key = key.to(torch.int64).reshape(-1)[:2]
    # a checkpoint written without the skip-step wrapper has no window: it starts empty
    missing = [m for m in missing if not m.rsplit(".", 1)[-1].startswith("_skipstep_")]
    if missing and not allow_partial:
        raise FileNotFoundError(f"Checkpoint {checkpoint_path} is missing leaves: {missing[:5]}{'...' if len(missing) > 5 else ''}")
    if missing:
        logger.warning(f"{len(missing)} leaves were not in the checkpoint and keep their initial values")
    return state


def load_checkpoint_or_initialize(state, checkpoint_search_paths, *, force_load: Optional[bool] = None,
                                  allow_partial: bool = False, initialize_from: Optional[str] = None):
    """Resume ``state`` from the newest checkpoint under the search path(s) when there is one; otherwise keep the
    freshly initialised state (optionally seeding it from ``initialize_from``).  ``force_load=True`` makes a missing
    checkpoint an error; ``False`` skips loading (src/levanter/checkpoint.py:462-560)."""
    if isinstance(checkpoint_search_paths, (str, os.PathLike)):
        checkpoint_search_paths = [checkpoint_search_paths]
    if force_load is not False:
        for p in checkpoint_search_paths:
            try:
                return load_checkpoint(state, p, discover_latest=True, allow_partial=allow_partial)
            except FileNotFoundError as e:
                if "missing leaves" in str(e) or "Missing parameters" in str(e):
                    raise
                continue
        if force_load is True:
            raise FileNotFoundError(f"Could not find a checkpoint in {list(checkpoint_search_paths)}")
    if initialize_from is not None:
        load_checkpoint(state, initialize_from, discover_latest=True, allow_partial=allow_partial)
        state.step = 0
    return state


@dataclass
class CheckpointerConfig:
    base_path: str = "checkpoints/"
    save_interval: timedelta = timedelta(minutes=15)
    keep: List[dict] = field(default_factory=lambda: [dict(every=10000)])
    append_run_id_to_base_path: bool = True
    delete_old_temp_checkpoints: bool = True

    def expanded_path(self, run_id: str) -> str:
        if self.append_run_id_to_base_path:
            return os.path.expanduser(os.path.join(self.base_path, run_id))
        return os.path.expanduser(self.base_path)

    def create(self, run_id: str) -> Checkpointer:
        keeps = [CheckpointInterval(**k) for k in self.keep]
        return Checkpointer(base_path=self.expanded_path(run_id), save_interval=self.save_interval, step_policies=keeps,
                            delete_old_temp_checkpoints=self.delete_old_temp_checkpoints)

    def __post_init__(self):
        self.base_path = os.path.expanduser(self.base_path) if "://" not in self.base_path else self.base_path
        for k in self.keep:
            if "every" not in k:
                raise ValueError(f"keep entries must have an 'every' key: {k}")
        prev = None
        for k in self.keep:
            until = k.get("until")
            if prev is None and k is not self.keep[0] and self.keep[self.keep.index(k) - 1].get("until") is None:
                raise ValueError("Only the last keep entry may omit 'until'")
            prev = until
