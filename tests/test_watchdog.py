"""Watchdog and job-level retry on one process (injected clock, fail-once functions)."""
import subprocess

import pytest

from levanter_b200.infra.resumable import Preempted, classify, run_resumable
from levanter_b200.utils.watchdog import PeerFailure, StepStalled, Watchdog


def test_stale_peer_and_stalled_step_with_injected_clock(tmp_path):
    now = [1000.0]
    a = Watchdog(str(tmp_path), 0, 2, peer_timeout=30.0, step_timeout=60.0, clock=lambda: now[0])
    b = Watchdog(str(tmp_path), 1, 2, peer_timeout=30.0, clock=lambda: now[0])
    a._write_heartbeat(); b._write_heartbeat()
    a.beat(0)
    assert a.check_once() is None
    now[0] += 20
    b._write_heartbeat()
    now[0] += 20
    assert a.check_once() is None            # b's last heartbeat is 20 s old
    now[0] += 15
    f = a.check_once()
    assert isinstance(f, PeerFailure) and "rank 1" in str(f)
    b._write_heartbeat()
    now[0] += 10                              # 65 s since a's own last beat
    assert isinstance(a.check_once(), StepStalled)
    a.beat(1)
    assert a.check_once() is None
    b.mark_failed("out of memory")
    with pytest.raises(PeerFailure, match="out of memory"):
        a.raise_if_failed()


def test_missing_peer_counts_from_start(tmp_path):
    now = [0.0]
    a = Watchdog(str(tmp_path), 0, 2, peer_timeout=10.0, clock=lambda: now[0])
    assert a.check_once() is None
    now[0] = 11.0
    assert "never sent a heartbeat" in str(a.check_once())


def test_run_resumable_budgets():
    calls = {"n": 0}

    def fail_twice():
        calls["n"] += 1
        if calls["n"] <= 2:
            raise RuntimeError("node lost")
        return "done"

    assert run_resumable(fail_twice, max_retries_failure=2) == "done" and calls["n"] == 3
    calls["n"] = 0
    with pytest.raises(RuntimeError):
        run_resumable(fail_twice, max_retries_failure=1)

    seen = []

    def preempted_then_ok():
        if not seen:
            seen.append(1)
            raise Preempted("SIGTERM")
        return 7

    assert run_resumable(preempted_then_ok, max_retries_failure=0, max_retries_preemption=1) == 7
    assert classify(subprocess.CalledProcessError(143, ["x"])) == "preemption" and classify(ValueError()) == "failure"
