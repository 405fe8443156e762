"""Trackers: global tracker context, deferred in-step logging, composite fan-out, JSON logger, histograms."""
import json
import logging

import numpy as np
import torch

from levanter_b200 import config as C
from levanter_b200 import tracker as trk
from levanter_b200.tracker.histogram import Histogram
from levanter_b200.tracker.tracker import CompositeTracker, DictTracker, NoopTracker, TrackerConfig


def test_current_tracker_context_and_log():
    t = DictTracker()
    with trk.current_tracker(t):
        trk.log({"a": 1, "b": torch.tensor(2.5)}, step=3)
        trk.log_summary({"params": 10})
        trk.log_hyperparameters({"lr": 0.1})
    assert t.metrics["a"] == 1 and abs(t.metrics["b"] - 2.5) < 1e-9 and t.summary["params"] == 10 and t.hparams["lr"] == 0.1
    assert t.history[0]["step"] == 3


def test_deferred_logging_collects_metrics_logged_inside_a_step():
    t = DictTracker()
    with trk.current_tracker(t):
        with trk.defer_tracker_for_jit() as captured:
            trk.jit_log({"grad_norm": torch.tensor(1.5)})
        assert "grad_norm" in captured and "grad_norm" not in t.metrics
        trk.log(captured, step=0)
    assert float(t.metrics["grad_norm"]) == 1.5


def test_composite_fans_out():
    a, b = DictTracker(), DictTracker()
    c = CompositeTracker([a, b, NoopTracker()])
    c.log({"x": 1}, step=0)
    c.log_summary({"y": 2})
    assert a.metrics["x"] == b.metrics["x"] == 1 and a.summary["y"] == 2


def test_json_logger_emits_one_json_object_per_event(caplog):
    cfg = C.decode(TrackerConfig, {"type": "json_logger", "logger_name": "lvb.test.metrics"})
    t = cfg.init("run1")
    with caplog.at_level(logging.INFO, logger="lvb.test.metrics"):
        t.log({"loss": 1.25}, step=7)
        t.log_summary({"done": True})
        t.finish()
    events = [json.loads(r.getMessage()) for r in caplog.records if r.name == "lvb.test.metrics"]
    assert any(e.get("event") == "log" and e.get("step") == 7 and e["metrics"]["loss"] == 1.25 for e in events)
    assert any(e.get("event") == "summary" for e in events)


def test_tracker_list_in_config_becomes_composite():
    from levanter_b200.trainer import TrainerConfig

    cfg = C.decode(TrainerConfig, {"tracker": [{"type": "noop"}, {"type": "json_logger"}]})
    assert isinstance(cfg.tracker, (list, tuple)) and len(cfg.tracker) == 2


def test_histogram_matches_numpy():
    x = torch.randn(1000, generator=torch.Generator().manual_seed(0))
    h = Histogram.from_array(x, num_bins=20)
    counts, edges = np.histogram(x.numpy(), bins=20)
    assert h.num == 1000 and abs(h.sum - float(x.sum())) < 1e-3 and abs(h.sum_squares - float((x * x).sum())) < 1e-2
    assert np.allclose(h.bucket_limits, edges, atol=1e-5) and np.abs(h.bucket_counts - counts).sum() <= 2
    assert h.min == float(x.min()) and h.max == float(x.max())


# ---------------------------------------------------------------- scenarios after the reference's tests/test_tracker.py
import pytest  # noqa: E402


def test_tracker_registry_default_choice_and_unknown_names():
    import dataclasses as dc

    import yaml

    from levanter_b200 import config as C
    from levanter_b200.tracker import TrackerConfig

    assert TrackerConfig.get_choice_class("wandb") is not None
    with pytest.raises(KeyError):
        TrackerConfig.get_choice_class("foo")
    with pytest.raises(C.ConfigError, match="known:.*noop"):
        TrackerConfig.get_choice_class("foo")

    @dc.dataclass
    class Holder:
        tracker: TrackerConfig

    t = C.decode(Holder, yaml.safe_load("tracker:\n  entity: foo\n")).tracker  # no type: the default choice
    assert isinstance(t, TrackerConfig.get_choice_class("wandb")) and t.entity == "foo"


def test_one_tracker_or_a_list_of_trackers_in_a_config():
    import dataclasses as dc
    from typing import Tuple, Union

    import yaml

    from levanter_b200 import config as C
    from levanter_b200.tracker import TrackerConfig
    from levanter_b200.tracker.tracker import NoopConfig

    @dc.dataclass
    class Holder:
        tracker: Union[TrackerConfig, Tuple[TrackerConfig, ...]]

    assert isinstance(C.decode(Holder, yaml.safe_load("tracker:\n  type: noop\n")).tracker, NoopConfig)
    both = C.decode(Holder, yaml.safe_load("tracker:\n  - type: noop\n  - type: wandb\n")).tracker
    assert both == (NoopConfig(), TrackerConfig.get_choice_class("wandb")())


def test_trackers_are_found_by_name_inside_a_composite():
    import levanter_b200.tracker as T
    from levanter_b200.tracker import CompositeTracker, NoopTracker
    from levanter_b200.tracker.json_logger import JsonLoggerTracker

    import logging

    inner = JsonLoggerTracker(logging.getLogger("test-json-tracker"))
    with CompositeTracker([inner, NoopTracker()]):
        assert T.get_tracker("json_logger") is inner
        assert T.get_tracker("noop") is not None
        with pytest.raises(KeyError):
            T.get_tracker("foo")
