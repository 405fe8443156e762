"""Hooks: tree statistics, the watch hook through a real trainer, throughput metrics, the profiler hooks, the epoch checkpointer and
validation loss (levanter_b200/callbacks/, analysis/tree_stats.py)."""
import math
import os

import pytest
import torch

import levanter_b200.tracker as T
from levanter_b200 import callbacks
from levanter_b200 import config as C
from levanter_b200.analysis.tree_stats import summary_statistics_for_tree
from levanter_b200.checkpoint import EpochCheckpointer
from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
from levanter_b200.optim import AdamConfig
from levanter_b200.tracker.histogram import Histogram
from levanter_b200.trainer import Trainer, TrainerConfig


class Recorder(T.NoopTracker):
    def __init__(self):
        self.logged, self.summary, self.artifacts = {}, {}, []

    def log(self, metrics, *, step, commit=None):
        self.logged.setdefault(step, {}).update(metrics)

    def log_summary(self, metrics):
        self.summary.update(metrics)

    def log_artifact(self, artifact_path, *, name=None, type=None):
        self.artifacts.append((str(artifact_path), name, type))


def test_tree_statistics_per_parameter_per_layer_and_stacked():
    tree = {"transformer.layers.0.mlp.up.weight": torch.full((2, 2), 1.0), "transformer.layers.1.mlp.up.weight": torch.full((2, 2), 2.0),
            "embeddings.token_embeddings.weight": torch.full((3,), 2.0), "unused": None}
    split = summary_statistics_for_tree("params", tree, split_scan_layers=True)
    assert float(split["params/norm/transformer/layers/0/mlp/up/weight"]) == pytest.approx(2.0)
    assert float(split["params/norm/transformer/layers/1/mlp/up/weight"]) == pytest.approx(4.0)
    assert float(split["params/norm/total"]) == pytest.approx(math.sqrt(4 + 16 + 12))
    stacked = summary_statistics_for_tree("params", tree, split_scan_layers=False)
    layer_keys = [k for k in stacked if "mlp" in k]
    assert len(layer_keys) == 1 and float(stacked[layer_keys[0]]) == pytest.approx(math.sqrt(4 + 16))  # both layers under one path
    only_total = summary_statistics_for_tree("g", tree, include_per_parameter_norms=False)
    assert list(only_total) == ["g/norm/total"]
    hist = summary_statistics_for_tree("g", tree, include_norms=False, include_histogram=True)
    h = hist["g/hist/embeddings/token_embeddings/weight"]
    assert isinstance(h, Histogram) and float(h.num) == 3 and float(h.sum) == pytest.approx(6.0)
    assert summary_statistics_for_tree("g", {"a": None}) == {}


VOCAB = 64


def _data(n=128):
    g = torch.Generator().manual_seed(0)
    starts = torch.randint(0, VOCAB, (n,), generator=g)
    return ListAsyncDataset([LmExample.causal(((s + torch.arange(16)) % VOCAB).to(torch.int32)) for s in starts], is_complete=True)


def test_watch_hook_and_default_metrics_through_a_trainer(tmp_path):
    rec = Recorder()
    cfg = C.decode(TrainerConfig, {"num_train_steps": 4, "train_batch_size": 8, "require_accelerator": False, "tracker": {"type": "noop"},
                                   "log_dir": f"{tmp_path}/logs", "id": "w", "steps_per_eval": 2, "max_eval_batches": 2, "per_device_eval_parallelism": 4,
                                   "checkpointer": {"base_path": f"{tmp_path}/ckpt", "save_interval": "10h"},
                                   "watch": {"watch_targets": "grads,params,opt_state,updates", "interval": 2, "include_histograms": True}})
    mc = LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, gradient_checkpointing=False)
    with T.current_tracker(rec):
        with Trainer(cfg, AdamConfig(learning_rate=1e-3, warmup=0.0, max_grad_norm=None), compute_next_token_loss) as trainer:
            state = trainer.initial_state(0, model_init=lambda: mc.build(VOCAB, seed=3))
            trainer.add_eval_hook(_data(32), name="tiny")
            trainer.add_hook(callbacks.log_performance_stats(16, cfg.batch_schedule, flops_per_example=1e6), every=1)
            trainer.train(state, trainer.data_loader(_data()).iter_from_step(0))
    assert sorted(rec.logged) == [0, 1, 2, 3]
    watched = rec.logged[2]
    assert float(watched["grad/norm/total"]) > 0 and float(watched["params/norm/total"]) > 0
    assert any(k.startswith("params/norm/transformer/layers/1/") for k in watched)
    assert any(k.startswith("opt_state/") and k.endswith("/norm/total") for k in watched)
    assert isinstance(watched["grad/hist/transformer/layers/0/self_attn/q_proj/weight"], Histogram)
    # the change of the weights in that step: with Adam and no decay every element moves by about the learning rate
    upd = float(watched["updates/norm/total"])
    n_params = sum(p.numel() for p in state.model.parameters())
    assert 0.2e-3 * n_params ** 0.5 < upd < 1.01e-3 * n_params ** 0.5
    assert any(k.startswith("updates/norm/transformer/layers/0/") for k in watched)
    assert "grad/norm/total" not in rec.logged[1] and "updates/norm/total" not in rec.logged[1]  # every second step only
    assert "eval/tiny/loss" in rec.logged[2] and "eval/tiny/loss" not in rec.logged[1] and rec.logged[2]["eval/tiny/loss"] > 0
    for step in (1, 2, 3):
        m = rec.logged[step]
        assert m["train/loss"] > 0 and m["global_step"] == step
        assert m["throughput/tokens_per_second"] > 0 and m["throughput/examples_per_second"] > 0 and m["throughput/duration"] > 0
        assert m["throughput/total_tokens"] == 16 * 8 * (step + 1) and "throughput/loading_time" in m
    assert rec.summary["throughput/flops_per_example"] == 1e6 and "throughput/device_kind" in rec.summary
    with pytest.raises(ValueError, match="Invalid watch target"):
        C.decode(TrainerConfig, {"watch": {"watch_targets": "gradients"}}).watch.build()


def test_profiler_hook_traces_the_configured_steps_and_logs_an_artifact(tmp_path):
    rec = Recorder()
    hook = callbacks.profile(str(tmp_path / "prof"), start_step=2, num_steps=2)
    with T.current_tracker(rec):
        for step in range(6):
            torch.ones(8) * 2
            hook(_Info(step))
    assert os.path.exists(tmp_path / "prof" / "trace_rank0.json") and rec.artifacts == [(str(tmp_path / "prof"), None, "profile")]

    with T.current_tracker(rec):
        with callbacks.profile_ctx(str(tmp_path / "block"), host_profile=True, host_profile_topn=5):
            sum(i * i for i in range(1000))
    assert sorted(os.listdir(tmp_path / "block")) == ["host_profile.pstats", "host_profile.txt", "trace_rank0.json"]
    assert "cumulative" in open(tmp_path / "block" / "host_profile.txt").read()


class _Info:
    def __init__(self, step, state=None):
        self.step, self.next_step, self.state = step, step + 1, state
        self.loss = 0.0


def test_epoch_checkpointer_saves_once_per_epoch():
    saved = []

    class FakeCheckpointer:
        def save_checkpoint(self, info, destination, **kw):
            saved.append((info.step, destination, kw.get("is_temporary")))

    ec = EpochCheckpointer(FakeCheckpointer(), every_n_epochs=1, total_dataset_size=100, batch_size=10)
    for step in range(0, 31):
        ec.on_step(_Info(step))
    assert saved == [(0, "epoch-0", True), (10, "epoch-1", True), (20, "epoch-2", True), (30, "epoch-3", True)]
    saved.clear()
    every_two = EpochCheckpointer(FakeCheckpointer(), every_n_epochs=2, total_dataset_size=100, batch_size=10)
    for step in range(0, 41):
        every_two.on_step(_Info(step))
    assert [d for _, d, _ in saved] == ["epoch-0", "epoch-2", "epoch-4"]
    EpochCheckpointer(FakeCheckpointer(), total_dataset_size=None).on_step(_Info(5))  # unknown size: nothing to do


def test_progress_bar_hook_runs_quietly():
    hook = callbacks.pbar_logger(total=3, disable=True)
    for step in range(3):
        hook(_Info(step))
