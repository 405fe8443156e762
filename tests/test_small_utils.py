"""Small utilities other layers rely on (levanter_b200/utils/*, distributed.py node-list expansion; scenarios after the
reference's tests/test_distributed.py, test_py_utils.py, test_logging.py and the behaviours its utilities document)."""
import asyncio
import dataclasses
import json
import random
import time
import uuid

import numpy as np
import pytest
import torch

from levanter_b200.distributed import _square_brace_expand
from levanter_b200.utils import fsspec_utils
from levanter_b200.utils.index import Index
from levanter_b200.utils.json_utils import ConfigJSONEncoder
from levanter_b200.utils.py_utils import (Stopwatch, actual_sizeof, dataclass_with_default_init, logical_cpu_core_count, non_caching_cycle,
                                          set_global_rng_seeds)
from levanter_b200.utils.stat_utils import RunningMean
from levanter_b200.utils.thread_utils import AsyncIteratorWrapper, ExceptionTrackingThread, blocking_wait


def test_slurm_node_lists_expand():
    assert _square_brace_expand("node[001-004]") == ["node001", "node002", "node003", "node004"]
    assert _square_brace_expand("prefix[001-002]node[005-006]suffix") == ["prefix001node005suffix", "prefix001node006suffix",
                                                                            "prefix002node005suffix", "prefix002node006suffix"]
    assert _square_brace_expand("node[1-11]suffix") == [f"node{i}suffix" for i in range(1, 12)]
    assert _square_brace_expand("node[1-11,21]suffix") == [f"node{i}suffix" for i in range(1, 12)] + ["node21suffix"]
    assert _square_brace_expand("single-host") == ["single-host"]


def test_sizes_cycles_and_stopwatch():
    d1 = {"a": 1, "b": 2, "c": 3}
    d2 = {"a": 1, "b": 2, "c": 3, "d": {"a": 1, "b": 2, "c": 3}}
    assert actual_sizeof(d1) < actual_sizeof(d2)
    shared = [0] * 100
    assert actual_sizeof([shared, shared]) < 2 * actual_sizeof(shared)  # an object is counted once

    calls = []

    class Source:
        def __iter__(self):
            calls.append(1)
            return iter([1, 2, 3])

    it = non_caching_cycle(Source())
    assert [next(it) for _ in range(7)] == [1, 2, 3, 1, 2, 3, 1] and len(calls) == 3  # re-iterated, not cached
    assert list(non_caching_cycle([])) == []

    sw = Stopwatch()
    for _ in range(2):
        with sw:
            time.sleep(0.01)
    assert 0.02 <= sw.elapsed() < 1.0 and sw.average() == pytest.approx(sw.elapsed() / 2)
    sw.reset()
    assert sw.elapsed() == 0.0
    assert logical_cpu_core_count() >= 1


def test_seeding_is_scoped_and_reproducible():
    before = (random.random(), float(np.random.rand()), float(torch.rand(())))
    random.seed(5), np.random.seed(5), torch.manual_seed(5)
    outer_next = (random.random(), float(np.random.rand()), float(torch.rand(())))
    random.seed(5), np.random.seed(5), torch.manual_seed(5)
    with set_global_rng_seeds(123):
        a = (random.random(), float(np.random.rand()), float(torch.rand(())))
    with set_global_rng_seeds(123):
        b = (random.random(), float(np.random.rand()), float(torch.rand(())))
    assert a == b and a != before
    assert (random.random(), float(np.random.rand()), float(torch.rand(()))) == outer_next  # the outer streams were not disturbed


def test_dataclass_that_keeps_its_own_init():
    @dataclass_with_default_init(frozen=True)
    class Point:
        x: int
        y: int = 2

        def __init__(self, both: int):
            self.__default_init__(x=both, y=both)

    p = Point(3)
    assert (p.x, p.y) == (3, 3) and dataclasses.is_dataclass(p)
    with pytest.raises(dataclasses.FrozenInstanceError):
        p.x = 1


def test_coroutines_run_from_sync_code_even_inside_a_running_loop():
    async def answer():
        await asyncio.sleep(0)
        return 42

    assert blocking_wait(answer()) == 42

    async def outer():
        return blocking_wait(answer())  # a loop is running in this thread

    assert asyncio.run(outer()) == 42


def test_async_iterators_as_plain_iterators_and_threads_that_report_their_errors():
    async def numbers():
        for i in range(5):
            await asyncio.sleep(0)
            yield i

    assert list(AsyncIteratorWrapper(numbers())) == [0, 1, 2, 3, 4]

    def boom():
        raise KeyError("from the thread")

    t = ExceptionTrackingThread(target=boom)
    t.start()
    with pytest.raises(KeyError, match="from the thread"):
        t.join()
    ok = ExceptionTrackingThread(target=lambda: None)
    ok.start()
    ok.join()
    ok.check_raise()


def test_running_mean_merges_by_weight_and_survives_zero_weight():
    m = RunningMean.zeros_like(0.0).add(2.0, 1.0).add(4.0, 3.0)
    assert m.mean == pytest.approx(3.5) and m.total == 4.0
    assert (m + RunningMean(10.0, 4.0)).mean == pytest.approx(6.75)
    empty = RunningMean.zeros_like(0.0)
    assert (empty + empty).mean == 0.0 and (empty + m).mean == pytest.approx(3.5)
    t = RunningMean.zeros_like(torch.zeros(2)).add(torch.tensor([1.0, 5.0]), torch.tensor([0.0, 2.0]))
    assert t.mean.tolist() == [0.0, 5.0] and t.total.tolist() == [0.0, 2.0]  # no division by the zero weight


def test_index_maps_objects_and_positions_both_ways():
    idx = Index(["a", "b"])
    assert idx.append("c") == 2 and idx.append("a") == 0 and len(idx) == 3
    assert idx.get_index("b") == 1 and idx.get_index("zzz") is None and idx.get_obj(2) == "c" and idx.get_obj(9) is None
    assert idx[1] == "b" and "c" in idx and "q" not in idx and list(idx) == ["a", "b", "c"] and idx.index("c") == 2
    with pytest.raises((KeyError, ValueError)):
        idx.index("missing")


def test_config_json_encoder_writes_enums_paths_and_dataclasses():
    from pathlib import Path

    from levanter_b200.utils.activation import ActivationFunctionEnum

    @dataclasses.dataclass
    class C:
        act: ActivationFunctionEnum
        path: Path

    text = json.dumps({"cfg": C(ActivationFunctionEnum.gelu_new, Path("/tmp/x")), "dt": torch.float32}, cls=ConfigJSONEncoder)
    back = json.loads(text)
    assert back["cfg"]["act"] == "gelu_new" and back["cfg"]["path"] == "/tmp/x"


def test_fsspec_helpers_on_a_memory_filesystem(tmp_path):
    base = f"memory://lvb-fs/{uuid.uuid4().hex}"
    assert not fsspec_utils.exists(base + "/a")
    fsspec_utils.mkdirs(base + "/a")
    import fsspec

    for name in ("x-0.jsonl", "x-1.jsonl", "y-0.jsonl"):
        with fsspec.open(f"{base}/a/{name}", "w") as f:
            f.write("{}")
    assert fsspec_utils.exists(f"{base}/a/x-0.jsonl")
    assert list(fsspec_utils.expand_glob(f"{base}/a/x-{{0,1}}.jsonl")) == [f"{base}/a/x-0.jsonl", f"{base}/a/x-1.jsonl"]
    assert list(fsspec_utils.expand_glob(f"{base}/a/x-{{0..1}}.jsonl")) == [f"{base}/a/x-0.jsonl", f"{base}/a/x-1.jsonl"]
    assert sorted(fsspec_utils.expand_glob(f"{base}/a/*-0.jsonl")) == [f"{base}/a/x-0.jsonl", f"{base}/a/y-0.jsonl"]  # protocol kept
    fsspec_utils.remove(f"{base}/a/y-0.jsonl")
    assert not fsspec_utils.exists(f"{base}/a/y-0.jsonl")
    asyncio.run(fsspec_utils.async_remove(f"{base}/a", recursive=True))
    assert not fsspec_utils.exists(f"{base}/a/x-0.jsonl")

    assert fsspec_utils.join_path("gs://bucket/run", "step-5") == "gs://bucket/run/step-5"
    assert fsspec_utils.join_path("/local/run", "gs://bucket/abs") == "gs://bucket/abs"  # a right side with a protocol is absolute
    assert fsspec_utils.join_path("gs://bucket/run", "gs://bucket/run/step-5") == "gs://bucket/run/step-5"
    with pytest.raises(ValueError):
        fsspec_utils.join_path("gs://bucket/run", "s3://other/x")


def test_git_root_of_the_experiment_is_found():
    import os

    from levanter_b200.tracker.helpers import infer_experiment_git_root

    root = infer_experiment_git_root()
    assert root is not None and os.path.isdir(os.path.join(root, ".git"))


def test_slurm_environment_gives_coordinator_ranks_and_local_devices(monkeypatch):
    from levanter_b200.distributed import LevanterSlurmCluster as S

    for k in list(__import__("os").environ):
        if k.startswith("SLURM"):
            monkeypatch.delenv(k)
    assert not S.is_env_present()
    env = {"SLURM_JOB_ID": "123456", "SLURM_PROCID": "5", "SLURM_NTASKS": "8", "SLURM_LOCALID": "1", "SLURM_STEP_NODELIST": "gpu[07-08,11]",
           "SLURM_STEP_TASKS_PER_NODE": "4(x2)", "SLURMD_NODENAME": "gpu08", "CUDA_VISIBLE_DEVICES": "0,1,2,3,4,5,6,7"}
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    assert S.is_env_present()
    host, port = S.get_coordinator_address().split(":")
    assert host == "gpu07" and 61440 <= int(port) <= 65535 and int(port) == 123456 % 4096 + 61440  # a port every task derives alike
    assert S.get_process_count() == 8 and S.get_process_id() == 5 and S.get_local_process_id() == 1
    assert S.get_tasks_per_node() == [4, 4]
    assert S.get_local_device_ids_for_process() == [2, 3]  # eight visible devices over four local tasks
    monkeypatch.setenv("SLURM_STEP_TASKS_PER_NODE", "2(x3),1")
    assert S.get_tasks_per_node() == [2, 2, 2, 1]
    monkeypatch.setenv("SLURM_STEP_TASKS_PER_NODE", "3")
    monkeypatch.setenv("SLURM_LOCALID", "0")
    assert S.get_local_device_ids_for_process() is None  # 8 devices do not divide over 3 tasks
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES")
    assert S.get_local_device_ids_for_process() is None
    monkeypatch.setenv("SLURM_STEP_TASKS_PER_NODE", "two")
    with pytest.raises(ValueError):
        S.get_tasks_per_node()
