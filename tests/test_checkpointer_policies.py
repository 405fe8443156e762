"""Checkpointer policies on a real directory: step policies that change over a run, time-based temporary checkpoints and their
clean-up, discovery, and partial loads (levanter_b200/checkpoint.py; scenarios after the reference's tests/test_checkpoint.py)."""
import datetime
import json
import os
from datetime import timedelta

import pytest
import torch

from levanter_b200.checkpoint import (Checkpointer, CheckpointerConfig, CheckpointInterval, discover_latest_checkpoint, load_checkpoint,
                                      save_checkpoint)


class _State:
    """The little a checkpointer needs of a trainer state."""

    def __init__(self, step):
        self.model = torch.nn.Linear(2, 2)
        self.saveable_state = {"model": {k: v.detach() for k, v in self.model.state_dict().items()}, "step": step}


class _Info:
    def __init__(self, step):
        self.step, self.state = step, _State(step)


def _steps(path):
    out = []
    for d in os.listdir(path):
        meta = os.path.join(path, d, "metadata.json")
        if os.path.exists(meta):
            out.append(json.load(open(meta))["step"])
    return sorted(out)


class _Clock:
    def __init__(self):
        self.now = datetime.datetime(2021, 1, 1)

    def __call__(self):
        return self.now

    def advance(self, seconds):
        self.now += timedelta(seconds=seconds)


POLICIES = [CheckpointInterval(every=2, until=10), CheckpointInterval(every=5, until=20), CheckpointInterval(every=10, until=None)]


def test_step_policies_that_change_over_the_run(tmp_path):
    ck = Checkpointer(str(tmp_path), None, POLICIES)
    for step in range(1, 50):
        ck.on_step(_Info(step))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [2, 4, 6, 8, 10, 15, 20, 30, 40]


def test_time_policy_keeps_only_the_newest_temporary_checkpoint(tmp_path):
    clock = _Clock()
    ck = Checkpointer(str(tmp_path), timedelta(seconds=10), [], dt_now_injection=clock)
    ck.on_step(_Info(0))
    clock.advance(10)
    ck.on_step(_Info(1))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [1]
    clock.advance(9)
    ck.on_step(_Info(2))  # not yet
    ck.wait_until_finished()
    assert _steps(tmp_path) == [1]
    clock.advance(1)
    ck.on_step(_Info(3))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [3]  # the temporary checkpoint of step 1 is gone
    assert json.load(open(tmp_path / "step-3" / "metadata.json"))["is_temporary"] is True


def test_step_and_time_policies_together(tmp_path):
    clock = _Clock()
    ck = Checkpointer(str(tmp_path), timedelta(seconds=10), POLICIES, dt_now_injection=clock)
    ck.on_step(_Info(0))
    clock.advance(10)
    ck.on_step(_Info(1))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [1]
    clock.advance(9)
    ck.on_step(_Info(2))  # too early for the clock, but a step policy asks for it; the temporary one of step 1 goes
    ck.wait_until_finished()
    assert _steps(tmp_path) == [2]
    clock.advance(1)
    ck.on_step(_Info(3))  # ten seconds since step 1's save, but only one since step 2's
    ck.wait_until_finished()
    assert _steps(tmp_path) == [2]
    for step in range(4, 11):
        clock.advance(10)
        ck.on_step(_Info(step))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [2, 4, 6, 8, 10]
    clock.advance(9)
    ck.on_step(_Info(11))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [2, 4, 6, 8, 10]
    for step in range(12, 50):
        ck.on_step(_Info(step))
        clock.advance(10)
    ck.wait_until_finished()
    assert _steps(tmp_path) == [2, 4, 6, 8, 10, 15, 20, 30, 40, 49]  # 49: the last temporary one


def test_a_new_checkpointer_cleans_up_the_temporary_checkpoint_of_an_earlier_run(tmp_path):
    clock = _Clock()
    policies = [CheckpointInterval(every=5, until=20), CheckpointInterval(every=10, until=None)]
    ck = Checkpointer(str(tmp_path), timedelta(seconds=10), policies, dt_now_injection=clock)
    ck.on_step(_Info(0))
    clock.advance(10)
    for i in range(1, 6):
        ck.on_step(_Info(i))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [5]
    clock.advance(10)
    ck.on_step(_Info(6))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [5, 6]

    ck = Checkpointer(str(tmp_path), timedelta(seconds=10), policies, dt_now_injection=clock)  # a restart
    ck.on_step(_Info(7))
    clock.advance(10)
    ck.on_step(_Info(8))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [5, 8]  # 6 was temporary and is replaced by 8

    ck = Checkpointer(str(tmp_path), timedelta(seconds=10), [CheckpointInterval(every=20, until=None)], dt_now_injection=clock,
                      delete_old_temp_checkpoints=False)
    ck.on_step(_Info(9))
    clock.advance(10)
    ck.on_step(_Info(10))
    ck.wait_until_finished()
    assert _steps(tmp_path) == [5, 8, 10]  # told to leave the earlier run's temporary checkpoint alone


def test_forced_saves_are_permanent_and_step_zero_is_only_saved_when_forced(tmp_path):
    ck = Checkpointer(str(tmp_path), None, [CheckpointInterval(every=100)])
    ck.on_step(_Info(0))
    ck.on_step(_Info(7))
    ck.wait_until_finished()
    assert _steps(tmp_path) == []
    ck.on_step(_Info(7), force=True)
    ck.on_step(_Info(7), force=True)  # the same step again: written once more, still one directory
    ck.wait_until_finished()
    assert _steps(tmp_path) == [7] and json.load(open(tmp_path / "step-7" / "metadata.json"))["is_temporary"] is False


def test_policy_lists_are_validated():
    with pytest.raises(ValueError):
        Checkpointer("unused", None, [CheckpointInterval(every=5, until=None), CheckpointInterval(every=20, until=100)])
    with pytest.raises(ValueError):
        Checkpointer("unused", None, [CheckpointInterval(every=5, until=100), CheckpointInterval(every=20, until=50)])
    cfg = CheckpointerConfig(base_path="/tmp/x", keep=[dict(every=5, until=10), dict(every=20)])
    assert cfg.expanded_path("run") == "/tmp/x/run"
    assert CheckpointerConfig(base_path="/tmp/x", append_run_id_to_base_path=False).expanded_path("run") == "/tmp/x"
    with pytest.raises(ValueError):
        CheckpointerConfig(keep=[dict(until=10)])


def test_discovery_picks_the_newest_complete_checkpoint(tmp_path):
    assert discover_latest_checkpoint(str(tmp_path)) is None
    assert discover_latest_checkpoint(str(tmp_path / "does-not-exist")) is None
    for step in (10, 20, 30):
        save_checkpoint({"w": torch.full((2,), float(step))}, step, str(tmp_path / f"step-{step}"))
    os.makedirs(tmp_path / "step-40")  # no metadata: an interrupted save
    latest = discover_latest_checkpoint(str(tmp_path))
    assert latest.endswith("step-30")
    # "newest" goes by the time of writing first: a run that was rolled back and re-saved an earlier step wins
    save_checkpoint({"w": torch.zeros(2)}, 15, str(tmp_path / "step-15"))
    assert discover_latest_checkpoint(str(tmp_path)).endswith("step-15")
    assert discover_latest_checkpoint(latest) == latest  # a checkpoint directory itself


def test_trees_load_fully_or_partially(tmp_path):
    tree = {"model": {"a.weight": torch.arange(6.0).reshape(2, 3), "a.bias": torch.ones(2)}, "step": 5}
    save_checkpoint(tree, 5, str(tmp_path / "step-5"))
    like = {"model": {"a.weight": torch.zeros(2, 3), "a.bias": torch.zeros(2)}, "step": 0}
    got = load_checkpoint(like, str(tmp_path), discover_latest=True)
    assert torch.equal(got["model"]["a.weight"], tree["model"]["a.weight"]) and got["step"] == 5
    bigger = {"model": {"a.weight": torch.zeros(2, 3), "a.bias": torch.zeros(2), "b.weight": torch.full((2,), 7.0)}, "step": 0}
    with pytest.raises(FileNotFoundError):
        load_checkpoint(bigger, str(tmp_path / "step-5"), discover_latest=False)
    got = load_checkpoint(bigger, str(tmp_path / "step-5"), discover_latest=False, allow_partial=True)
    assert torch.equal(got["model"]["a.bias"], torch.ones(2)) and torch.equal(got["model"]["b.weight"], torch.full((2,), 7.0))
    with pytest.raises(FileNotFoundError):
        load_checkpoint(like, str(tmp_path / "nothing-here"))


def test_checkpointer_loads_just_the_model_of_the_newest_checkpoint(tmp_path):
    ck = Checkpointer(str(tmp_path), None, [CheckpointInterval(every=1)])
    infos = [_Info(1), _Info(2)]
    for info in infos:
        ck.on_step(info)
    ck.wait_until_finished()
    fresh = torch.nn.Linear(2, 2)
    assert not torch.equal(fresh.weight, infos[1].state.model.weight)
    ck.load_model(fresh)
    assert torch.equal(fresh.weight, infos[1].state.model.weight) and torch.equal(fresh.bias, infos[1].state.model.bias)
    ck.load_model(fresh, str(tmp_path / "step-1"), discover_latest=False)
    assert torch.equal(fresh.weight, infos[0].state.model.weight)
