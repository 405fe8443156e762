"""Job-level retry: run a training function (or command) again after a failure or a preemption, relying on checkpoint
resume; separate budgets for the two, as in the reference's ``run_on_pod_resumable`` (src/levanter/infra/ray_tpu.py:1081-1137)."""
from __future__ import annotations

import logging
import signal
import subprocess
import time
from typing import Callable, List, Optional, Sequence, TypeVar

logger = logging.getLogger(__name__)
T = TypeVar("T")


class Preempted(RuntimeError):
    """The job was asked to stop by the scheduler (SIGTERM, exit code 143 / 130)."""


PREEMPTION_EXIT_CODES = (143, 130, -signal.SIGTERM, -signal.SIGINT)


def classify(exc: BaseException) -> str:
    """"preemption" or "failure"."""
    if isinstance(exc, (Preempted, KeyboardInterrupt)):
        return "preemption"
    if isinstance(exc, subprocess.CalledProcessError) and exc.returncode in PREEMPTION_EXIT_CODES:
        return "preemption"
    return "failure"


def run_resumable(fn: Callable[[], T], *, max_retries_failure: int = 10, max_retries_preemption: int = 1_000_000,
                  backoff_seconds: float = 0.0, on_retry: Optional[Callable[[str, int, BaseException], None]] = None) -> T:
    """Call ``fn`` until it returns.  Failures and preemptions are counted separately; when a budget runs out the last
    exception is raised."""
    n_fail = n_preempt = 0
    while True:
        try:
            return fn()
        except BaseException as e:  # noqa: BLE001
            if isinstance(e, (SystemExit, GeneratorExit)):
                raise
            kind = classify(e)
            if kind == "preemption":
                n_preempt += 1
                if n_preempt > max_retries_preemption:
                    raise
            else:
                n_fail += 1
                if n_fail > max_retries_failure:
                    raise
            logger.warning("run %s (%s); retry %d", kind, e, n_fail + n_preempt)
            if on_retry is not None:
                on_retry(kind, n_fail + n_preempt, e)
            if backoff_seconds:
                time.sleep(backoff_seconds)


def run_command_resumable(cmd: Sequence[str], **kw) -> int:
    """``run_resumable`` around a subprocess (for example the ``torch.distributed.run`` line of the launcher)."""
    def once() -> int:
        rc = subprocess.call(list(cmd))
        if rc != 0:
            raise subprocess.CalledProcessError(rc, list(cmd))
        return rc

    return run_resumable(once, **kw)
