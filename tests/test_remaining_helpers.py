"""Small public helpers that the larger scenario tests do not reach: checkpoint path test, the cache's async accessors, datasource
factories, the entropy / top-2-gap hooks, process helpers, trainer batch helpers and a few tree / config utilities."""
import asyncio
import json
import math
from types import SimpleNamespace
from typing import Iterator, Sequence

import numpy as np
import pytest
import torch

from levanter_b200 import tracker as T
from levanter_b200.data.sharded_datasource import ShardedDataSource, datasource_from_json, datasource_from_parquet
from levanter_b200.store.cache import BatchProcessor, TreeCache
from levanter_b200.store.jagged_array import JaggedArrayStore


class _Processor(BatchProcessor):
    def __call__(self, batch):
        return [{"ids": np.asarray(x, np.int64)} for x in batch]

    @property
    def output_exemplar(self):
        return {"ids": np.zeros(0, np.int64)}

    @property
    def metadata(self):
        return {}

    @property
    def num_cpus(self):
        return 1


class _Shards(ShardedDataSource):
    @property
    def shard_names(self) -> Sequence[str]:
        return ["a", "b"]

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[list]:
        base = 0 if shard_name == "a" else 100
        return ([base + i] * (i + 1) for i in range(row, 5))


def test_cache_is_built_in_the_background_and_read_through_its_async_store(tmp_path):
    cache = TreeCache.build_or_load(str(tmp_path / "c"), _Shards(), _Processor())  # returns before the build is finished
    store = asyncio.run(cache.store_async())
    cache.await_finished()
    assert cache.is_finished and len(cache) == 10
    assert store is not None and [int(x["ids"][0]) for x in cache] == [0, 1, 2, 3, 4, 100, 101, 102, 103, 104]
    assert [len(x["ids"]) for x in cache[:5]] == [1, 2, 3, 4, 5]
    again = TreeCache.load(str(tmp_path / "c"), {"ids": np.zeros(0, np.int64)})
    assert len(again) == 10


def test_jagged_store_async_open_and_reload_see_rows_appended_by_another_handle(tmp_path):
    async def scenario():
        writer = await JaggedArrayStore.open_async(str(tmp_path / "j"), mode="a", item_rank=1, dtype=np.int32)
        writer.append(np.arange(3, dtype=np.int32))
        reader = await JaggedArrayStore.open_async(str(tmp_path / "j"), mode="r", item_rank=1, dtype=np.int32)
        assert reader.num_rows == 1
        writer.extend([np.arange(5, dtype=np.int32), np.arange(2, dtype=np.int32)])
        reader = await reader.reload_async()
        return reader

    reader = asyncio.run(scenario())
    assert reader.num_rows == 3 and reader[1].tolist() == [0, 1, 2, 3, 4] and reader[2].tolist() == [0, 1]


def test_datasource_factories_for_json_and_parquet(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq

    rows = [{"text": f"doc {i}", "n": i} for i in range(7)]
    (tmp_path / "d.json").write_text(json.dumps(rows))
    pq.write_table(pa.Table.from_pylist(rows), tmp_path / "d.parquet", row_group_size=3)
    for source in (datasource_from_json([str(tmp_path / "d.json")]), datasource_from_parquet([str(tmp_path / "d.parquet")])):
        (shard,) = source.shard_names
        assert [r["n"] for r in source.open_shard(shard)] == list(range(7))
        assert [r["text"] for r in source.open_shard_at_row(shard, 4)] == ["doc 4", "doc 5", "doc 6"]  # resuming inside a row group too


def test_entropy_and_top2_gap_hooks_log_histograms_of_the_evaluated_model():
    from levanter_b200.analysis.entropy import cb_compute_entropies, cb_compute_top2_gap
    from levanter_b200.data.dataset import ListAsyncDataset
    from levanter_b200.models.llama import LlamaConfig
    from levanter_b200.models.lm_model import LmExample
    from levanter_b200.tracker.histogram import Histogram

    vocab = 24
    model = LlamaConfig(seq_len=8, hidden_dim=16, intermediate_dim=32, num_layers=1, num_heads=2, num_kv_heads=2).build(vocab, seed=0)
    data = ListAsyncDataset([LmExample.causal(torch.randint(0, vocab, (8,), generator=torch.Generator().manual_seed(i), dtype=torch.int32))
                             for i in range(8)], is_complete=True)

    class Recorder(T.NoopTracker):
        def __init__(self):
            self.logged = {}

        def log(self, metrics, *, step, commit=None):
            self.logged.setdefault(step, {}).update(metrics)

    def logits(m, batch):
        return m(batch.tokens, attn_mask=batch.attn_mask)

    rec = Recorder()
    info = SimpleNamespace(step=5, eval_model=model)
    with T.current_tracker(rec):
        cb_compute_entropies(logits, vocab, data, prefix="probe", batch_size=4)(info)
        cb_compute_top2_gap(logits, vocab, data, prefix=None, batch_size=4)(info)
        cb_compute_entropies(logits, vocab, ListAsyncDataset([], is_complete=True), prefix="none", batch_size=4)(info)  # warns, logs nothing
    ent, gap = rec.logged[5]["probe/entropy"], rec.logged[5]["analysis/top2_gap"]
    assert isinstance(ent, Histogram) and isinstance(gap, Histogram) and "none/entropy" not in rec.logged[5]
    assert int(ent.num) == 8 * 8 and 0.0 <= float(ent.min) <= float(ent.max) <= math.log(vocab) + 1e-4
    assert int(gap.num) == 8 * 8 and float(gap.min) >= 0.0


def test_process_helpers_follow_the_launcher_variables(monkeypatch, tmp_path):
    from levanter_b200 import distributed as D

    for k in ("LOCAL_RANK", "SLURM_LOCALID", "RANK", "WORLD_SIZE", "SLURM_PROCID", "SLURM_NTASKS"):
        monkeypatch.delenv(k, raising=False)
    assert D.process_count() == 1 and D.process_index() == 0
    monkeypatch.setenv("SLURM_NTASKS", "16")
    monkeypatch.setenv("SLURM_PROCID", "5")
    assert D.process_count() == 16 and D.process_index() == 5
    monkeypatch.setenv("WORLD_SIZE", "8")
    monkeypatch.setenv("RANK", "3")
    assert D.process_count() == 8 and D.process_index() == 3  # torchrun's variables win
    monkeypatch.setenv("LOCAL_RANK", "2")
    assert not D.is_local_leader()
    monkeypatch.setenv("LOCAL_RANK", "0")
    assert D.is_local_leader()
    monkeypatch.delenv("LOCAL_RANK")
    monkeypatch.setenv("SLURM_LOCALID", "1")
    assert not D.is_local_leader()
    # no launcher variable: the first process on the node to take the lock leads
    monkeypatch.delenv("SLURM_LOCALID")
    monkeypatch.setenv("SLURM_JOB_ID", f"test-{tmp_path.name}")
    assert D.is_local_leader()


def test_trainer_config_batch_helpers():
    from levanter_b200 import config as C
    from levanter_b200.trainer import TrainerConfig

    cfg = C.decode(TrainerConfig, {"train_batch_size": [{"start": 0, "value": 8}, {"start": 10, "value": 32}], "per_device_parallelism": 4,
                                   "require_accelerator": False})
    assert [cfg.batch_size_at_step(s) for s in (0, 9, 10, 500)] == [8, 8, 32, 32]
    assert cfg.microbatch_size == 4 * cfg.data_axis_size
    assert C.decode(TrainerConfig, {"require_accelerator": False}).microbatch_size is None  # -1: the whole per-GPU batch at once


def test_checkpoint_path_test_and_small_tree_and_config_utilities(tmp_path, monkeypatch):
    from levanter_b200 import tensorstore_serialization as tss
    from levanter_b200.checkpoint import is_checkpoint_path
    from levanter_b200.optim.skipstep import SkipStepConfig
    from levanter_b200.utils.py_utils import logical_cpu_memory_size
    from levanter_b200.utils.remat import ScanCheckpointPolicy
    from levanter_b200.utils.tree_utils import tree_flatten_one_level_with_keys

    assert not is_checkpoint_path(tmp_path)
    tss.tree_serialize_leaves_tensorstore(str(tmp_path / "step-1"), {"w": torch.ones(2)})
    assert not is_checkpoint_path(tmp_path / "step-1")  # arrays alone are not a checkpoint: the metadata file marks a finished save
    (tmp_path / "step-1" / "metadata.json").write_text(json.dumps({"step": 1, "timestamp": "2024-01-01T00:00:00", "is_temporary": False}))
    assert is_checkpoint_path(tmp_path / "step-1") and is_checkpoint_path(f"file://{tmp_path}/step-1")

    children, kind = tree_flatten_one_level_with_keys({"a": torch.zeros(1), "b": {"c": torch.ones(1)}})
    assert [k for k, _ in children] == ["a", "b"] and kind is dict and isinstance(dict(children)["b"], dict)

    monkeypatch.setenv("SLURM_MEM_PER_NODE", "64000")
    assert logical_cpu_memory_size() == pytest.approx(64.0)
    monkeypatch.setenv("SLURM_MEM_PER_NODE", "lots")
    assert logical_cpu_memory_size() > 0  # falls back to what the machine reports

    assert ScanCheckpointPolicy.from_config_value(False).recompute is False and ScanCheckpointPolicy.from_config_value(True).recompute
    assert ScanCheckpointPolicy.from_config_value("nested").nested
    assert SkipStepConfig.from_config_value(64).rolling_interval_length == 64 and SkipStepConfig.from_config_value(False) is None


def test_converter_reads_the_config_of_a_local_checkpoint_and_merges_overrides(tmp_path):
    from levanter_b200.compat.hf_checkpoints import HFCheckpointConverter
    from levanter_b200.models.llama import LlamaConfig

    small = LlamaConfig(seq_len=32, hidden_dim=16, intermediate_dim=48, num_layers=2, num_heads=4, num_kv_heads=2)
    (tmp_path / "config.json").write_text(json.dumps(small.to_hf_config(100)))
    conv = HFCheckpointConverter(LlamaConfig, str(tmp_path))
    got = conv.config_from_hf_checkpoint()
    assert (got.hidden_dim, got.intermediate_dim, got.num_layers, got.num_heads, got.num_kv_heads) == (16, 48, 2, 4, 2)
    assert conv.default_hf_config["vocab_size"] == 100
    a = conv.with_config_overrides({"rope_theta": 5.0})
    b = a.with_config_overrides({"max_position_embeddings": 64})
    c = a.with_config_overrides({"max_position_embeddings": 64}, merge=False)
    assert b.config_overrides == {"rope_theta": 5.0, "max_position_embeddings": 64} and c.config_overrides == {"max_position_embeddings": 64}
    assert conv.config_overrides in (None, {})  # the original is untouched


def test_gemma3_local_rope_and_tied_unembedding():
    from levanter_b200.models.gemma import Gemma3Config
    from levanter_b200.models.llama import LlamaConfig

    cfg = Gemma3Config(seq_len=16, hidden_dim=16, intermediate_dim=32, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=8,
                       rope_local_base_freq=1234.0)
    assert cfg.local_rope.theta == 1234.0 and cfg.rope.theta != 1234.0 and type(cfg.local_rope) is type(cfg.rope)
    # the embedding module scores hidden states against its own rows (the head of a model with tied embeddings)
    model = LlamaConfig(seq_len=8, hidden_dim=16, intermediate_dim=32, num_layers=1, num_heads=2, num_kv_heads=2,
                        tie_word_embeddings=True).build(20, seed=0)
    x = torch.randn(2, 3, 16)
    emb = model.embeddings
    assert torch.allclose(emb.unembed(x), x @ emb.token_embeddings.weight.t(), atol=1e-5)
    assert all("lm_head" not in n for n, _ in model.named_parameters())
