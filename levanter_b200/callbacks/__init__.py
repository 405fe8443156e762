"""Trainer hooks (src/levanter/callbacks/__init__.py, _metrics.py): validation loss, profiler, step logging,
throughput / MFU, progress bar, epoch progress."""
from __future__ import annotations

import contextlib
import cProfile
import io
import logging as pylogging
import os
import pstats
import threading
import time
from typing import Callable, Iterable, Optional

import torch
import torch.distributed as dist

from .. import tracker as trk
from ..utils.flop_utils import device_hardware_flops, device_kind
from ._core import Callback, JitCallback, LambdaCallback, StepInfo  # noqa: F401
from ._metrics import get_total_dataset_tokens, log_epoch_progress, log_performance_stats, log_step_info, pbar_logger  # noqa: F401

logger = pylogging.getLogger(__name__)


def eval_loss_loop(loss_fn, model, dataset: Iterable, max_batches: Optional[int] = None, name: Optional[str] = None,
                   device=None) -> float:
    """Mean loss of ``model`` over ``dataset`` (at most ``max_batches`` batches), averaged over ranks."""
    total = torch.zeros((), dtype=torch.float64, device=device)
    n = 0
    was_training = model.training
    model.eval()
    desc = f"eval {name}" if name else "eval"
    t0 = time.time()
    try:
        from tqdm import tqdm

        it = tqdm(dataset, desc=desc, total=max_batches, leave=False, disable=_rank() != 0)
    except Exception:
        it = dataset
    with torch.no_grad():
        for batch in it:
            if hasattr(batch, "to"):
                batch = batch.to(device)
            loss = loss_fn(model, batch)
            total += loss.detach().double().mean()
            n += 1
            if max_batches is not None and n >= max_batches:
                break
    if was_training:
        model.train()
    if n > 0:
        total /= n
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(total, op=dist.ReduceOp.AVG)
    logger.info(f"{desc} loss: {float(total):.3f} ({time.time() - t0:.1f}s)")
    return float(total)


def compute_validation_loss(loss_fn: Callable, dataset: Iterable, max_batches: Optional[int] = None,
                            name: Optional[str] = None, device=None):
    def compute_loss(info: StepInfo):
        loss = eval_loss_loop(loss_fn, info.eval_model, dataset, max_batches=max_batches, name=name, device=device)
        prefix = "eval" if not name else f"eval/{name}"
        trk.log({f"{prefix}/loss": loss}, step=info.step)
        return loss

    return compute_loss


def _rank() -> int:
    return dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0


def profile(path: str, start_step: int, num_steps: int, create_perfetto_link: bool = False) -> Callable[[StepInfo], None]:
    """Trace steps ``[start_step, start_step + num_steps)`` with ``torch.profiler`` (CPU + CUDA activities, Chrome trace
    in ``path``) and log the directory as a ``profile`` artifact, then barrier
    (counterpart of src/levanter/callbacks/__init__.py:110-139)."""
    state = {"prof": None}

    def profiler_callback_fn(step: StepInfo):
        if step.step == start_step - 1 and state["prof"] is None:
            os.makedirs(path, exist_ok=True)
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            prof = torch.profiler.profile(activities=acts, record_shapes=False)
            prof.__enter__()
            state["prof"] = prof
        elif step.step == start_step + num_steps - 1 and state["prof"] is not None:
            prof = state["prof"]
            prof.__exit__(None, None, None)
            state["prof"] = None
            out = os.path.join(path, f"trace_rank{_rank()}.json")
            try:
                prof.export_chrome_trace(out)
                trk.current_tracker().log_artifact(path, type="profile")
            except Exception:  # noqa: BLE001
                logger.exception("could not export the profiler trace")
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                dist.barrier()

    return profiler_callback_fn


@contextlib.contextmanager
def profile_ctx(path: str, *, create_perfetto_link: bool = False, host_profile: bool = False, host_profile_topn: int = 40):
    """Profile a block: ``torch.profiler`` device trace plus an optional host ``cProfile`` (``.pstats`` and top-N text)
    (src/levanter/callbacks/__init__.py:156-253)."""
    os.makedirs(path, exist_ok=True)
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    pr = cProfile.Profile() if host_profile else None
    prof = torch.profiler.profile(activities=acts)
    prof.__enter__()
    if pr is not None:
        pr.enable()
    try:
        yield
    finally:
        if pr is not None:
            pr.disable()
            pr.dump_stats(os.path.join(path, "host_profile.pstats"))
            s = io.StringIO()
            pstats.Stats(pr, stream=s).sort_stats("cumulative").print_stats(host_profile_topn)
            with open(os.path.join(path, "host_profile.txt"), "w") as f:
                f.write(s.getvalue())
        prof.__exit__(None, None, None)
        try:
            prof.export_chrome_trace(os.path.join(path, f"trace_rank{_rank()}.json"))
        except Exception:  # noqa: BLE001
            logger.exception("could not export the profiler trace")
        try:
            trk.current_tracker().log_artifact(path, type="profile")
        except Exception:
            pass
