"""CPU tests of the data pipeline: stores, cache build/resume, permutations, mixtures, packing and the text configs."""
import asyncio
import json
import os

import numpy as np
import pytest
import torch

from levanter_b200 import config as cfg
from levanter_b200.data._prp import Permutation
from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.data.mixture import MixtureDataset, StopStrategy
from levanter_b200.data.packing import (GreedyPrepackedDataset, PromptCompletion, greedy_pack_prompt_completions, pack_documents,
                                        pack_prompt_completions, per_segment_correct, per_segment_loss)
from levanter_b200.data.passthrough_tokenizer import PassthroughTokenizer
from levanter_b200.data.sharded_datasource import UrlDataSource
from levanter_b200.data.text import (BatchTokenizer, LMMixtureDatasetConfig, SupervisedDataset, SupervisedLmDatasetFormat,
                                     UrlSingleDatasetLMConfig, cached_token_count)
from levanter_b200.store.cache import CacheLedger, CacheOptions, SerialCacheWriter, TreeCache, build_or_load_cache
from levanter_b200.store.jagged_array import JaggedArrayStore
from levanter_b200.store.tree_store import TreeStore


def run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


def _write_shards(d, n_shards=3, rows=40, vocab=1000):
    rng = np.random.default_rng(0)
    docs = []
    for s in range(n_shards):
        with open(f"{d}/shard{s}.jsonl", "w") as f:
            for i in range(rows + s):
                ids = rng.integers(0, vocab - 1, size=int(rng.integers(3, 50)))
                docs.append(ids)
                f.write(json.dumps({"text": " ".join(map(str, ids))}) + "\n")
    return docs


@pytest.mark.parametrize("kind", ["feistel", "linear"])
@pytest.mark.parametrize("n", [1, 2, 17, 100, 1000])
def test_permutation_is_bijection(kind, n):
    p = Permutation.make(kind, n, 1234)
    img = p(np.arange(n))
    assert sorted(img.tolist()) == list(range(n))
    assert all(int(p(i)) == int(img[i]) for i in range(min(n, 20)))
    if n >= 100:
        assert not np.array_equal(img, np.arange(n))
        assert not np.array_equal(img, Permutation.make(kind, n, 99)(np.arange(n)))
    with pytest.raises(IndexError):
        p(n)


def test_jagged_store_roundtrip_and_trim(tmp_path):
    s = JaggedArrayStore.open(str(tmp_path / "j"), mode="w", dtype=np.int32)
    rows = [np.arange(i + 1, dtype=np.int32) * (i + 1) for i in range(60)]
    s.extend(rows[:25])
    s.extend(rows[25:])
    assert len(s) == 60 and s.data_size == sum(len(r) for r in rows)
    for i, r in zip([59, 0, 31, 31], s.get_batch_sync([59, 0, 31, 31])):
        np.testing.assert_array_equal(r, rows[i])
    s.trim_to_size(10)
    assert len(s) == 10
    s.append(rows[10])
    np.testing.assert_array_equal(s[10], rows[10])
    r = JaggedArrayStore.open(str(tmp_path / "j"), mode="r", dtype=np.int32, cache_metadata=True)
    assert len(r) == 11
    np.testing.assert_array_equal(r[3], rows[3])


def test_tree_store_rank2_leaf(tmp_path):
    ex = {"ids": np.zeros(0, np.int32), "feat": np.zeros((0, 3), np.float32)}
    t = TreeStore.open(ex, str(tmp_path / "t"), mode="w")
    items = [{"ids": np.arange(i + 2, dtype=np.int32), "feat": np.full((i + 1, 3), i, np.float32)} for i in range(9)]
    t.extend(items)
    assert len(t) == 9
    g = t[4]
    np.testing.assert_array_equal(g["ids"], items[4]["ids"])
    assert g["feat"].shape == (5, 3) and (g["feat"] == 4).all()


def test_cache_build_is_deterministic_and_resumes(tmp_path):
    d = str(tmp_path)
    docs = _write_shards(d)
    tok = PassthroughTokenizer(1000)
    src = UrlDataSource([f"{d}/shard{{0..2}}.jsonl"])
    proc = BatchTokenizer(tok, enforce_bos=False, enforce_eos=False)
    c = build_or_load_cache(d + "/cache", src, proc, options=CacheOptions(batch_size=7))
    assert len(c) == len(docs)
    for got, want in zip(c.get_batch_sync(range(len(docs))), docs):
        np.testing.assert_array_equal(got["input_ids"], want)
    assert cached_token_count(d + "/cache") == sum(len(x) for x in docs)

    # simulate an interrupted build: ledger says shard0 finished and shard1 consumed 10 rows; extra rows are on disk
    ledger = CacheLedger.load(d + "/cache")
    n0 = ledger.shard_rows["shard0_jsonl"]
    ledger.is_finished = False
    ledger.finished_shards = ["shard0_jsonl"]
    ledger.shard_rows = {"shard0_jsonl": n0, "shard1_jsonl": 10, "shard2_jsonl": 0}
    ledger.total_num_rows = n0 + 10
    ledger._serialize_and_commit(d + "/cache")
    c2 = build_or_load_cache(d + "/cache", src, proc, options=CacheOptions(batch_size=5))
    assert c2._builder is not None and len(c2) == len(docs)
    for got, want in zip(c2.get_batch_sync(range(len(docs))), docs):
        np.testing.assert_array_equal(got["input_ids"], want)


def test_cache_readable_while_building(tmp_path):
    d = str(tmp_path)
    docs = _write_shards(d, n_shards=2, rows=30)
    src = UrlDataSource([f"{d}/shard{{0..1}}.jsonl"])
    proc = BatchTokenizer(PassthroughTokenizer(1000), enforce_bos=False, enforce_eos=False)
    c = build_or_load_cache(d + "/c", src, proc, await_finished=False, options=CacheOptions(batch_size=4, target_size_per_flush=1))
    np.testing.assert_array_equal(c.get_batch_sync([5])[0]["input_ids"], docs[5])
    c.await_finished()
    assert len(c) == len(docs)


def test_builder_error_reaches_reader(tmp_path):
    d = str(tmp_path)
    with open(f"{d}/bad.jsonl", "w") as f:
        f.write(json.dumps({"text": "1 2 x"}) + "\n")
    proc = BatchTokenizer(PassthroughTokenizer(10), enforce_bos=False, enforce_eos=False)
    with pytest.raises(ValueError, match="whitespace-separated integers"):
        build_or_load_cache(d + "/c", UrlDataSource([f"{d}/bad.jsonl"]), proc)


def test_serial_cache_writer(tmp_path):
    ex = {"input_ids": np.zeros(0, np.int32)}
    with SerialCacheWriter(str(tmp_path / "c"), ex) as w:
        w.write_batch([{"input_ids": np.arange(4, dtype=np.int32)}] * 3)
    c = w.result()
    assert len(c) == 3 and c.is_finished
    np.testing.assert_array_equal(c[1]["input_ids"], np.arange(4))


def test_mixture_block_counts_and_stability():
    a = ListAsyncDataset(list(range(0, 1000)), is_complete=True)
    b = ListAsyncDataset(list(range(10000, 10100)), is_complete=True)
    m = MixtureDataset({"a": a, "b": b}, {"a": 0.75, "b": 0.25}, block_size=16, key=3)
    got = run(m.get_batch(list(range(64))))
    for blk in range(4):
        chunk = got[blk * 16:(blk + 1) * 16]
        assert sum(1 for x in chunk if x >= 10000) == 4
    # each source is consumed in order, no repeats
    assert sorted(x for x in got if x < 10000) == list(range(48))
    # random access agrees with batch access
    assert run(m.getitem_async(37)) == got[37]
    # restart strategy wraps the short dataset
    far = run(m.get_batch(list(range(16 * 30, 16 * 30 + 16))))
    assert all(10000 <= x < 10100 for x in far if x >= 10000)


def test_mixture_stages_and_first_exhausted():
    a = ListAsyncDataset(list(range(100)), is_complete=True)
    b = ListAsyncDataset(list(range(1000, 1100)), is_complete=True)
    m = MixtureDataset({"a": a, "b": b}, [(0, {"a": 1.0, "b": 0.0}), (32, {"a": 0.0, "b": 1.0})], block_size=16, key=0)
    got = run(m.get_batch(list(range(48))))
    assert all(x < 100 for x in got[:32]) and all(x >= 1000 for x in got[32:])
    assert sorted(got[32:]) == list(range(1000, 1016))
    with pytest.raises(ValueError):
        MixtureDataset({"a": a}, [(0, {"a": 1.0}), (10, {"a": 1.0})], block_size=16, key=0)
    m2 = MixtureDataset({"a": a, "b": b}, {"a": 0.5, "b": 0.5}, block_size=16, key=0, stop_strategy=StopStrategy.FIRST_STOP_STRATEGY)
    with pytest.raises((StopIteration, RuntimeError, IndexError)):
        run(m2.get_batch(list(range(16 * 20, 16 * 20 + 16))))


def test_pack_documents_matches_quadratic_reference():
    rng = np.random.default_rng(1)
    lens = rng.integers(1, 40, size=300)

    def slow(lens, cap, max_seg):
        out, i = [], 0
        while i < len(lens):
            start, segs = i, 0
            while i < len(lens) and segs < max_seg and sum(lens[start:i + 1]) <= cap:
                segs += 1
                i += 1
            if i == start:
                i += 1
            out.append(range(start, i))
        return out

    assert pack_documents(lens, 64, 5) == slow(lens, 64, 5)
    assert pack_documents(lens, 64, None) == slow(lens, 64, 1 << 30)
    with pytest.raises(ValueError):
        pack_documents(np.array([3, 100]), 64)
    assert pack_documents(np.array([3, 100, 2]), 64, slice_too_long_examples=True) == [range(0, 1), range(1, 2), range(2, 3)]


def test_prompt_completion_packers():
    seqs = [PromptCompletion(list(range(1, 6)), 2), PromptCompletion(list(range(10, 14)), 1), PromptCompletion(list(range(20, 29)), 4)]
    out = list(pack_prompt_completions(16, seqs, pad_token=0, max_segments_per_example=2))
    assert len(out) == 2
    e = out[0]
    assert e.tokens.tolist()[:9] == [1, 2, 3, 4, 5, 10, 11, 12, 13]
    assert e.loss_mask.tolist()[:9] == [0, 1, 1, 1, 0, 1, 1, 1, 0]
    assert e.attn_mask.segment_ids[0].tolist()[:10] == [0] * 5 + [1] * 4 + [-1]
    g = greedy_pack_prompt_completions(16, seqs, pad_token=0, max_segments_per_example=2)
    assert len(g) == 2 and g[1].attn_mask.segment_ids[0].tolist()[:9] == [2] * 9
    losses = torch.arange(16, dtype=torch.float32)
    ids, per = per_segment_loss(e, losses, 4)
    assert ids.tolist() == [-1, 0, 1, -1]
    assert per.tolist()[1] == 1 + 2 + 3 and per.tolist()[2] == 5 + 6 + 7
    correct = torch.ones(16, dtype=torch.bool)
    correct[6] = False
    _, ok = per_segment_correct(e, correct, 4)
    assert ok.tolist()[1] is True and ok.tolist()[2] is False


def test_supervised_sequence_mask():
    seg = np.array([5, 5, 5, 5, 9, 9, 9, -1, -1])
    m = SupervisedDataset._make_sequence_mask(seg, np.array([2, 1]))
    assert m.tolist() == [0, 0, 1, 1, 0, 1, 1, 0, 0]


def _cfg_for(d, **kw):
    return UrlSingleDatasetLMConfig(tokenizer="passthrough", vocab_size=1000, cache_dir=d + "/cache", train_urls=[f"{d}/shard{{0..2}}.jsonl"],
                                    validation_urls=[f"{d}/shard0.jsonl"], cache_options=CacheOptions(batch_size=8), **kw)


def test_single_dataset_config_end_to_end(tmp_path):
    d = str(tmp_path)
    docs = _write_shards(d)
    flat = np.concatenate([np.append(x, 999) for x in docs])  # eos appended by BatchTokenizer
    c = _cfg_for(d)
    ds = c.train_set(32, key=0).as_sync_dataset()
    assert len(ds) == len(flat) // 32
    ex = ds[3]
    np.testing.assert_array_equal(ex.tokens.numpy(), flat[96:128])
    assert ex.loss_mask[-1] == 0 and ex.attn_mask.segment_ids is not None
    seg = ex.attn_mask.segment_ids[0].numpy()
    eos_pos = np.nonzero(flat[96:127] == 999)[0]
    assert (np.diff(seg) == 1).sum() == len(eos_pos)
    val = c.validation_sets(32)
    assert list(val.keys()) == [""]
    shuffled = _cfg_for(d, shuffle=True, permutation_type="feistel").train_set(32, key=1).as_sync_dataset()
    toks = sorted(tuple(shuffled[i].tokens.tolist()) for i in range(len(shuffled)))
    assert toks == sorted(tuple(ds[i].tokens.tolist()) for i in range(len(ds)))
    tagged = c.tagged_eval_sets(32)
    assert tagged[0][1] == [""]


def test_mixture_config_from_yaml(tmp_path):
    d = str(tmp_path)
    _write_shards(d)
    y = f"""
tokenizer: passthrough
vocab_size: 1000
cache_dir: {d}/mix
mixture_block_size: 8
configs:
  a:
    train_urls: ["{d}/shard0.jsonl"]
    validation_urls: ["{d}/shard1.jsonl"]
    tags: [web]
  b:
    train_urls: ["{d}/shard{{1..2}}.jsonl"]
train_weights:
  a: 0.5
  b: 0.5
"""
    import yaml

    c = cfg.decode(LMMixtureDatasetConfig, yaml.safe_load(y))
    from levanter_b200.schedule import BatchSchedule

    ds = c.train_set(16, BatchSchedule(4), key=0).as_sync_dataset()
    batch = ds.get_batch(list(range(16)))
    assert all(b.tokens.shape == (16,) for b in batch)
    tagged = c.tagged_eval_sets(16)
    assert [t for _, t in tagged] == [["web", "a"]]


def test_supervised_format_packs(tmp_path):
    d = str(tmp_path)
    with open(f"{d}/sup.jsonl", "w") as f:
        for i in range(20):
            f.write(json.dumps({"prompt": " ".join(str(5 + j) for j in range(i % 4 + 1)) + " ", "response": " ".join(str(100 + j) for j in range(3))}) + "\n")
    c = UrlSingleDatasetLMConfig(tokenizer="passthrough", vocab_size=1000, cache_dir=d + "/c", train_urls=[f"{d}/sup.jsonl"],
                                 format=SupervisedLmDatasetFormat())
    ds = c.train_set(16, key=0).as_sync_dataset()
    ex = ds[0]
    seg = ex.attn_mask.segment_ids[0].numpy()
    toks, lm = ex.tokens.numpy(), ex.loss_mask.numpy()
    assert len(set(seg[seg >= 0].tolist())) >= 2  # packed
    # loss only where the *next* token is a response token of the same segment
    for t in range(15):
        if lm[t]:
            assert toks[t + 1] >= 100 and seg[t + 1] == seg[t]
    assert lm[seg == -1].sum() == 0


def test_any_step_of_a_shuffled_staged_mixture_can_be_reached_directly(tmp_path):
    """The batch of step k is a function of the configuration and k alone: iterating from 0, resuming at k, and asking a fresh
    dataset object built from the same config give the same tokens (mixture with stages, per-source shuffle, batch-size schedule)."""
    from levanter_b200.data.loader import DataLoader
    from levanter_b200.schedule import BatchSchedule, ScheduleStep

    d = str(tmp_path)
    rng = np.random.default_rng(0)
    for name, base in (("a", 100), ("b", 400), ("c", 700)):
        with open(f"{d}/{name}.jsonl", "w") as f:
            for _ in range(120):
                f.write(json.dumps({"text": " ".join(str(base + int(x)) for x in rng.integers(0, 250, size=int(rng.integers(3, 30))))}) + "\n")

    def build():
        return cfg.decode(LMMixtureDatasetConfig, {
            "tokenizer": "passthrough", "vocab_size": 1000, "cache_dir": f"{d}/cache", "mixture_block_size": 8, "shuffle": True,
            "configs": {n: {"train_urls": [f"{d}/{n}.jsonl"]} for n in "abc"},
            "train_weights": [[0, {"a": 0.75, "b": 0.25, "c": 0.0}], [6, {"a": 0.25, "b": 0.25, "c": 0.5}]]})

    sched = BatchSchedule([ScheduleStep(0, 4), ScheduleStep(4, 8)])
    ds = build().train_set(16, sched, key=5)
    loader = DataLoader(ds, sched, max_buffered_batches=0, pin_memory=False)
    it = iter(loader)
    straight = [next(it).tokens.clone() for _ in range(10)]
    assert [b.shape[0] for b in straight] == [4] * 4 + [8] * 6
    for k in (1, 4, 7, 9):
        resumed = loader.iter_from_step(k)
        assert torch.equal(next(resumed).tokens, straight[k]), k
    fresh = DataLoader(build().train_set(16, sched, key=5), sched, max_buffered_batches=4, pin_memory=False).iter_from_step(6)
    assert torch.equal(next(fresh).tokens, straight[6]) and torch.equal(next(fresh).tokens, straight[7])
    other_key = DataLoader(build().train_set(16, sched, key=6), sched, max_buffered_batches=0, pin_memory=False)
    assert not torch.equal(next(iter(other_key)).tokens, straight[0])
    # the stage change at step 6 (= sequence 4 * 4 + 2 * 8 = 32, a block boundary) shows in the sources of the tokens
    share_c = [float(((b >= 700) & (b < 950)).float().mean()) for b in straight]
    assert max(share_c[:6]) == 0.0 and min(share_c[6:]) > 0.2
