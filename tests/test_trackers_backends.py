"""The tensorboard and trackio trackers against fake back ends (neither service is contacted), and the flat packing of trees."""
import pytest
import os
import numpy as np
import torch

from levanter_b200.tracker.tensorboard import TensorboardTracker
from levanter_b200.tracker.trackio import TrackioTracker
from levanter_b200.utils.tree_utils import pack_pytree, unpack_pytree


class _Writer:
    def __init__(self, log_dir):
        self.log_dir, self.scalars, self.texts, self.hists, self.closed = str(log_dir), [], [], [], False

    def add_scalar(self, k, v, global_step=None):
        self.scalars.append((k, v, global_step))

    def add_text(self, k, v, global_step=None):
        self.texts.append((k, v, global_step))

    def add_histogram(self, k, v, global_step=None):
        self.hists.append((k, np.asarray(v), global_step))

    def add_histogram_raw(self, k, **kw):
        self.hists.append((k, kw, kw.get("global_step")))

    def close(self):
        self.closed = True


def test_tensorboard_tracker_routes_scalars_text_arrays_histograms_and_artifacts(tmp_path):
    from levanter_b200.tracker.histogram import Histogram

    w = _Writer(tmp_path / "tb")
    t = TensorboardTracker(w)
    t.log_hyperparameters({"model": {"hidden_dim": 64}, "lr": 1e-3})
    assert ("config/model/hidden_dim", "64", None) in w.texts or any(k.endswith("hidden_dim") for k, _, _ in w.texts)
    h = Histogram.from_array(torch.randn(1000)) if hasattr(Histogram, "from_array") else None
    metrics = {"train/loss": 2.5, "note": "hello", "grad": {"norm": torch.tensor(0.3)}, "vec": np.arange(4.0)}
    if h is not None:
        metrics["hist"] = h
    t.log(metrics, step=7)
    assert ("train/loss", 2.5, 7) in w.scalars and any(k.endswith("norm") and s == 7 for k, _, s in w.scalars)
    assert ("note", "hello", 7) in w.texts
    assert any(k == "vec" for k, _, _ in w.hists) and (h is None or any(k == "hist" for k, _, _ in w.hists))
    t.log_summary({"final_loss": 1.25, "status": "done"})
    assert ("summary/final_loss", 1.25, None) in w.scalars and any(k == "summary/status" for k, _, _ in w.texts)
    art = tmp_path / "a.txt"
    art.write_text("x")
    t.log_artifact(str(art), name="kept.txt")
    assert (tmp_path / "tb" / "artifacts" / "kept.txt").read_text() == "x"
    t.finish()
    assert w.closed


def test_trackio_tracker_sends_floats_and_strings_to_the_run():
    class Run:
        def __init__(self):
            self.config, self.logged, self.finished = {}, [], False

        def log(self, payload, step=None):
            self.logged.append((payload, step))

        def finish(self):
            self.finished = True

    run = Run()
    t = TrackioTracker(run)
    t._trackio = None  # whatever is installed, talk to the fake run
    t.log_hyperparameters({"lr": 3e-4})
    assert run.config == {"lr": 3e-4}
    t.log({"loss": torch.tensor(1.5), "tag": "abc"}, step=3)
    assert run.logged[-1] == ({"loss": 1.5, "tag": "abc"}, 3)
    t.log_summary({"best": 0.9})
    assert run.logged[-1] == ({"summary/best": 0.9}, None)
    t.finish()
    assert run.finished


def test_pack_and_unpack_trees():
    tree = {"a": torch.arange(3, dtype=torch.float32), "b": [torch.arange(4, dtype=torch.float64).reshape(2, 2), torch.tensor(5, dtype=torch.int32)],
            "meta": "kept as is"}
    offsets, flat = pack_pytree(tree)
    assert flat.dtype == torch.float32 and flat.numel() == 3 + 4 + 1
    back = unpack_pytree(offsets, flat)
    assert back["meta"] == "kept as is"
    assert torch.equal(back["a"], tree["a"]) and torch.equal(back["b"][0], tree["b"][0]) and back["b"][0].dtype == torch.float64
    assert int(back["b"][1]) == 5 and back["b"][1].dtype == torch.int32 and back["b"][1].shape == ()
    offsets, flat = pack_pytree({})
    assert flat.numel() == 0 and unpack_pytree(offsets, flat) == {}


class _FakeWandbRun:
    def __init__(self):
        self.step, self.logged, self.summary, self.artifacts, self.finished, self.code = 0, [], {}, [], False, None
        self.config = self

    def update(self, values, allow_val_change=False):  # run.config.update
        self.hparams = dict(values)

    def log(self, metrics, step=None, commit=None):
        self.logged.append((step, dict(metrics), commit))
        if step is not None:
            self.step = step

    def log_artifact(self, path, name=None, type=None):
        self.artifacts.append((os.path.basename(path), name, type))

    def log_code(self, root):
        self.code = root

    def finish(self):
        self.finished = True


def test_wandb_tracker_logs_steps_in_order_histograms_summaries_and_artifacts(monkeypatch, tmp_path, caplog):
    wandb = pytest.importorskip("wandb")
    from levanter_b200.tracker.histogram import Histogram
    from levanter_b200.tracker.wandb import WandbTracker

    run = _FakeWandbRun()
    run.summary = {}
    t = WandbTracker(run)
    t.log_hyperparameters({"lr": 0.1})
    t.log({"loss": 1.0}, step=3)
    t.log({"loss": 0.5, "hist": Histogram.from_array(torch.arange(10.0))}, step=4)
    t.log({"late": 1.0}, step=2)  # a step the run is already past: refused with a warning, not an error
    t.log({"auto": 2.0}, step=None)
    assert run.hparams == {"lr": 0.1} and [s for s, _, _ in run.logged] == [3, 4, 4]
    assert isinstance(run.logged[1][1]["hist"], wandb.Histogram) and run.logged[2][1] == {"auto": 2.0}
    assert "Cowardly refusing" in caplog.text
    t.log_summary({"best": 0.5})
    (tmp_path / "a.txt").write_text("x")
    t.log_artifact(str(tmp_path / "a.txt"), name="a", type="text")
    t.finish()
    assert run.summary == {"best": 0.5} and run.artifacts == [("a.txt", "a", "text")] and run.finished


def test_wandb_config_chooses_the_run_id_mode_and_records_the_commit(monkeypatch):
    wandb = pytest.importorskip("wandb")
    from levanter_b200.tracker.wandb import WandbConfig, WandbTracker

    calls = []

    def fake_init(**kw):
        calls.append(kw)
        return _FakeWandbRun()

    monkeypatch.setattr(wandb, "init", fake_init)
    monkeypatch.delenv("WANDB_API_KEY", raising=False)
    monkeypatch.delenv("WANDB_MODE", raising=False)
    monkeypatch.setenv("RANK", "0")
    tracker = WandbConfig(project="proj", tags=["t"], save_code=False).init("run-1")
    assert isinstance(tracker, WandbTracker)
    kw = calls[-1]
    assert kw["id"] == "run-1" and kw["project"] == "proj" and kw["tags"] == ["t"] and kw["resume"] == "allow"
    assert kw["mode"] == "offline"  # no credentials and no explicit mode: usable without a network
    assert len(kw["config"]["git_commit"]) == 40
    WandbConfig(id="mine", mode="online").init("run-1")
    assert calls[-1]["id"] == "mine" and calls[-1]["mode"] == "online"  # the tracker's own id wins
    monkeypatch.setenv("WANDB_API_KEY", "k")
    WandbConfig(save_code=False).init("r")
    assert calls[-1]["mode"] is None
    monkeypatch.setenv("RANK", "3")
    WandbConfig(save_code=False).init("r")
    assert calls[-1]["mode"] == "offline"  # only process 0 talks to the service
