"""Failure detection on the host: per-rank heartbeat files, a watchdog that notices a stalled or failed peer (or a stalled
step of this rank) and a check the training loop calls between steps, so that a rank learns of a failure *before* it
launches kernels or collectives that would wait for the missing peer.

The reference relies on JAX's coordination service and on job-level retries for this (src/levanter/distributed.py:357-363,
src/levanter/utils/jax_utils.py:107-134, src/levanter/infra/ray_tpu.py:1081-1137).  Here every rank writes
``<dir>/rank-<r>.hb`` (JSON: time, step, phase) every ``interval`` seconds from a background thread; a rank that fails
writes ``<dir>/rank-<r>.failed`` with the reason on its way out.  Nothing here touches a GPU."""
from __future__ import annotations

import faulthandler
import json
import logging
import os
import sys
import threading
import time
import traceback
from dataclasses import dataclass
from typing import Callable, Dict, Optional

logger = logging.getLogger(__name__)


class PeerFailure(RuntimeError):
    """Another rank failed or stopped sending heartbeats."""


class StepStalled(RuntimeError):
    """This rank's own step did not finish within the limit."""


@dataclass
class WatchdogConfig:
    enabled: bool = False
    dir: Optional[str] = None          # shared directory; default <log_dir>/<run_id>/heartbeats
    interval: float = 5.0              # seconds between heartbeats
    peer_timeout: float = 120.0        # a peer without a heartbeat for this long counts as failed
    step_timeout: Optional[float] = None  # this rank's step taking longer than this counts as stalled (None: off)
    dump_stacks_on_stall: bool = True

    def build(self, rank: int, world: int, default_dir: str) -> Optional["Watchdog"]:
        if not self.enabled:
            return None
        return Watchdog(self.dir or default_dir, rank, world, interval=self.interval, peer_timeout=self.peer_timeout,
                        step_timeout=self.step_timeout, dump_stacks_on_stall=self.dump_stacks_on_stall)


class Watchdog:
    def __init__(self, directory: str, rank: int, world: int, *, interval: float = 5.0, peer_timeout: float = 120.0,
                 step_timeout: Optional[float] = None, dump_stacks_on_stall: bool = True, clock: Callable[[], float] = time.time):
        self.dir, self.rank, self.world = directory, rank, world
        self.interval, self.peer_timeout, self.step_timeout = interval, peer_timeout, step_timeout
        self.dump_stacks_on_stall = dump_stacks_on_stall
        self._clock = clock
        self._step, self._phase, self._last_beat = -1, "init", clock()
        self._failure: Optional[BaseException] = None
        self._stop = threading.Event()
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self._started_at = clock()
        os.makedirs(directory, exist_ok=True)
        for suffix in ("hb", "failed"):  # a previous incarnation of this rank may have left files behind
            try:
                os.remove(self._path(self.rank, suffix))
            except FileNotFoundError:
                pass

    # -- files ---------------------------------------------------------------------------------------------------
    def _path(self, rank: int, suffix: str) -> str:
        return os.path.join(self.dir, f"rank-{rank}.{suffix}")

    def _write_heartbeat(self) -> None:
        tmp = self._path(self.rank, "hb.tmp")
        with open(tmp, "w") as f:
            json.dump({"time": self._clock(), "step": self._step, "phase": self._phase, "pid": os.getpid()}, f)
        os.replace(tmp, self._path(self.rank, "hb"))

    def _read(self, rank: int, suffix: str) -> Optional[dict]:
        try:
            with open(self._path(rank, suffix)) as f:
                return json.load(f)
        except (FileNotFoundError, json.JSONDecodeError):
            return None

    # -- public --------------------------------------------------------------------------------------------------
    def start(self) -> "Watchdog":
        self._write_heartbeat()
        self._thread = threading.Thread(target=self._run, name=f"watchdog-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval + 1.0)

    def beat(self, step: int, phase: str = "step") -> None:
        """Called by the training loop when a step (or a phase of it) completes."""
        with self._lock:
            self._step, self._phase, self._last_beat = step, phase, self._clock()

    def mark_failed(self, reason: str) -> None:
        """Tell the peers that this rank is going down (called from an exception handler)."""
        try:
            with open(self._path(self.rank, "failed"), "w") as f:
                json.dump({"time": self._clock(), "step": self._step, "reason": reason[:2000]}, f)
        except OSError:
            pass

    def check_once(self) -> Optional[BaseException]:
        """One scan of the peers' files and of this rank's own progress; returns the failure found, if any."""
        now = self._clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            failed = self._read(r, "failed")
            if failed is not None and failed.get("time", 0) >= self._started_at - 1.0:
                return PeerFailure(f"rank {r} failed at step {failed.get('step')}: {failed.get('reason')}")
            hb = self._read(r, "hb")
            last = hb["time"] if hb is not None else self._started_at
            if now - last > self.peer_timeout:
                what = "never sent a heartbeat" if hb is None else f"sent its last heartbeat {now - last:.0f} s ago (step {hb.get('step')}, {hb.get('phase')})"
                return PeerFailure(f"rank {r} {what}; limit {self.peer_timeout:.0f} s")
        if self.step_timeout is not None and self._step >= 0 and now - self._last_beat > self.step_timeout:
            return StepStalled(f"rank {self.rank}: step {self._step + 1} has been running for {now - self._last_beat:.0f} s; limit {self.step_timeout:.0f} s")
        return None

    def raise_if_failed(self) -> None:
        """Called between steps, before anything is launched that would wait for a peer."""
        if self._failure is None:
            self._failure = self.check_once()
        if self._failure is not None:
            raise self._failure

    @property
    def failure(self) -> Optional[BaseException]:
        return self._failure

    # -- thread --------------------------------------------------------------------------------------------------
    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._write_heartbeat()
                if self._failure is None:
                    f = self.check_once()
                    if f is not None:
                        self._failure = f
                        logger.error("watchdog: %s", f)
                        if isinstance(f, StepStalled) and self.dump_stacks_on_stall:
                            faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
            except Exception:  # noqa: BLE001  (the watchdog must not die of a full disk or a race on a file)
                logger.warning("watchdog scan failed:\n%s", traceback.format_exc())

    def __enter__(self):
        return self.start()

    def __exit__(self, exc_type, exc, tb):
        if exc is not None and not isinstance(exc, PeerFailure):
            self.mark_failed(f"{exc_type.__name__}: {exc}")
        self.stop()
        return False
