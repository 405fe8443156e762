"""Step / throughput metrics (src/levanter/callbacks/_metrics.py:26-178)."""
from __future__ import annotations

import logging as pylogging
import time
from typing import Callable, Optional

import torch

from .. import tracker as trk
from ..utils.flop_utils import device_hardware_flops, device_kind
from ._core import StepInfo

logger = pylogging.getLogger(__name__)


def get_total_dataset_tokens(ds, seq_length: int):
    """A future for ``len(ds) * seq_length``, computed on a helper thread (the length of a cache that is still being built is
    slow to get) and logged as the summary ``dataset/total_tokens``.  ``ds`` may be an epoch wrapper: its ``dataset`` is counted."""
    import asyncio
    from concurrent.futures import ThreadPoolExecutor

    inner = getattr(ds, "dataset", ds)

    def log_length():
        total = asyncio.run(inner.async_len()) * seq_length
        trk.log_summary({"dataset/total_tokens": total})
        return total

    executor = ThreadPoolExecutor(max_workers=1)
    future = executor.submit(log_length)
    executor.shutdown(wait=False)
    return future


def log_epoch_progress(total_tokens_future, tokens_per_example: int, batch_size: int, max_epochs: Optional[int] = None):
    """Log ``train/current_epoch`` once the dataset's total token count is known (a number, a callable returning one or None,
    or a future as returned by :func:`get_total_dataset_tokens`)."""
    total = {"v": None}

    def log_epoch(step_info: StepInfo):
        if total["v"] is None:
            if hasattr(total_tokens_future, "done"):
                v = total_tokens_future.result() if total_tokens_future.done() else None
            else:
                v = total_tokens_future() if callable(total_tokens_future) else total_tokens_future
            if v is None:
                return
            total["v"] = v
        if not total["v"]:
            return
        processed = tokens_per_example * batch_size * step_info.next_step
        cur = processed / total["v"]
        if max_epochs is not None and cur > max_epochs:
            cur = max_epochs
        trk.log({"train/current_epoch": cur}, step=step_info.step)

    return log_epoch


def log_step_info(total_steps: Optional[int]):
    def log_step_info_inner(step: StepInfo):
        metrics = {"train/loss": step.loss, "global_step": step.step}
        if total_steps:
            metrics["run_progress"] = step.step / total_steps
        trk.log(metrics, step=step.step)

    return log_step_info_inner


def log_performance_stats(tokens_per_example: int, batch_schedule, flops_per_example: Optional[float] = None,
                          prefix: Optional[str] = "throughput", device_count: Optional[int] = None):
    """tokens/s, examples/s, GFLOP/s and MFU from host step durations (src/levanter/callbacks/_metrics.py:83-150).
    MFU = achieved FLOP/s / (device peak x devices)."""
    import torch.distributed as dist

    from ..schedule import BatchSchedule

    if isinstance(batch_schedule, int):
        batch_schedule = BatchSchedule(batch_schedule)
    if device_count is None:
        device_count = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
    peak = device_hardware_flops()
    state = {"logged_static": False}

    def wrap_key(key):
        return f"{prefix}/{key}" if prefix else key

    def log_performance_stats_inner(step_info: StepInfo):
        if not state["logged_static"]:
            state["logged_static"] = True
            summ = {wrap_key("device_kind"): device_kind()}
            if flops_per_example:
                summ[wrap_key("flops_per_example")] = flops_per_example
            if peak is not None:
                summ[wrap_key("theoretical_flops_per_device")] = peak
                summ[wrap_key("theoretical_flops")] = peak * device_count
            trk.log_summary(summ)
        bs = batch_schedule.batch_size_at_step(step_info.step)
        total_examples = batch_schedule.global_data_offset_by_step(step_info.step) + bs
        total_tokens = total_examples * tokens_per_example
        d = {wrap_key("total_tokens"): total_tokens}
        if flops_per_example:
            d[wrap_key("total_gflops")] = flops_per_example / 1e9 * total_examples
        dur = step_info.step_duration
        if dur and dur > 0:
            d[wrap_key("examples_per_second")] = bs / dur
            d[wrap_key("tokens_per_second")] = bs * tokens_per_example / dur
            d[wrap_key("duration")] = dur
            if flops_per_example is not None:
                fps = flops_per_example * bs / dur
                d[wrap_key("gflops_per_second")] = fps / 1e9
                if peak is not None:
                    d[wrap_key("mfu")] = fps / (peak * device_count) * 100.0
        trk.log(d, step=step_info.step)

    return log_performance_stats_inner


def pbar_logger(iterable=None, desc: str = "train", **tqdm_mkwargs) -> Callable[[StepInfo], None]:
    """Progress bar that refreshes its postfix at most once a minute (src/levanter/callbacks/_metrics.py:153-177)."""
    try:
        from tqdm import tqdm
    except ImportError:
        return lambda step: None
    import torch.distributed as dist

    kwargs = dict(tqdm_mkwargs)
    not_rank0 = dist.is_available() and dist.is_initialized() and dist.get_rank() != 0
    disable = bool(kwargs.pop("disable", False)) or not_rank0  # only process 0 draws; a caller may silence it too
    kwargs.setdefault("mininterval", 10.0)
    pbar = tqdm(iterable, desc=desc, disable=disable, **kwargs)
    last = {"t": 0.0}

    def update_pbar(step: StepInfo):
        pbar.update(step.next_step - pbar.n)
        now = time.time()
        if now - last["t"] > 60 or step.next_step == kwargs.get("total"):
            pbar.set_postfix(loss=f"{step.loss:.3f}")
            last["t"] = now

    return update_pbar
