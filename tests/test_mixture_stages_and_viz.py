"""Mixtures whose weights change at stage boundaries (proportions, zero weights, block alignment, invalid stage lists) and the
HTML rendering of per-token log-probabilities."""
import asyncio

import numpy as np
import pytest

from levanter_b200.analysis.visualization import visualize_log_prob_diff, visualize_log_probs
from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.data.mixture import MixtureDataset


def run(coro):
    return asyncio.get_event_loop_policy().new_event_loop().run_until_complete(coro)


def _sources():
    return {"ones": ListAsyncDataset([1] * 500, is_complete=True), "tens": ListAsyncDataset([10] * 500, is_complete=True),
            "hundreds": ListAsyncDataset([100] * 500, is_complete=True)}


def _shares(batch):
    n = len(batch)
    return {v: sum(1 for x in batch if x == v) / n for v in (1, 10, 100)}


def test_proportions_follow_the_stage_a_block_belongs_to():
    stages = [(0, {"ones": 0.8, "tens": 0.2, "hundreds": 0.0}), (200, {"ones": 0.2, "tens": 0.6, "hundreds": 0.2}),
              (400, {"ones": 0.0, "tens": 0.2, "hundreds": 0.8})]
    m = MixtureDataset(_sources(), stages, block_size=20, key=42)
    first = _shares(run(m.get_batch(list(range(0, 200)))))
    mid = _shares(run(m.get_batch(list(range(200, 400)))))
    last = _shares(run(m.get_batch(list(range(400, 600)))))
    assert first[1] == pytest.approx(0.8, abs=0.05) and first[100] == 0.0
    assert mid[10] == pytest.approx(0.6, abs=0.05) and mid[1] == pytest.approx(0.2, abs=0.05)
    assert last[100] == pytest.approx(0.8, abs=0.05) and last[1] == 0.0
    # a batch that straddles a boundary takes each index from its own stage
    straddle = run(m.get_batch(list(range(190, 210))))
    assert 100 not in straddle[:10]


def test_a_zero_weight_source_is_never_read_and_missing_names_mean_zero():
    m = MixtureDataset(_sources(), [(0, {"ones": 1.0}), (40, {"tens": 1.0, "ones": 0.0})], block_size=10, key=0, randomize_blocks=False)
    assert set(run(m.get_batch(list(range(0, 40))))) == {1}
    assert set(run(m.get_batch(list(range(40, 90))))) == {10}


def test_stage_lists_are_validated():
    src = _sources()
    with pytest.raises(ValueError):
        MixtureDataset(src, [(10, {"ones": 1.0})], block_size=10, key=0)  # must start at 0
    with pytest.raises(ValueError):
        MixtureDataset(src, [(0, {"ones": 1.0}), (25, {"tens": 1.0})], block_size=10, key=0)  # not on a block boundary
    with pytest.raises(ValueError):
        MixtureDataset(src, [(0, {"ones": 1.0}), (20, {"tens": 1.0}), (20, {"hundreds": 1.0})], block_size=10, key=0)  # not increasing
    with pytest.raises(ValueError):
        MixtureDataset(src, [(0, {"nobody": 1.0})], block_size=10, key=0)  # unknown source
    with pytest.raises(ValueError):
        MixtureDataset(src, [], block_size=10, key=0)


def test_the_same_index_always_maps_to_the_same_item():
    stages = [(0, {"ones": 0.5, "tens": 0.5}), (60, {"tens": 0.5, "hundreds": 0.5})]
    m1 = MixtureDataset(_sources(), stages, block_size=20, key=7)
    m2 = MixtureDataset(_sources(), stages, block_size=20, key=7)
    idx = [5, 59, 60, 61, 119, 3]
    assert run(m1.get_batch(idx)) == run(m2.get_batch(idx)) == [run(m1.get_batch([i]))[0] for i in idx]


def test_log_probability_pages_are_written(tmp_path):
    toks = [["The", " cat", " <b>"], ["A", " dog", " ran"]]
    lps = np.array([[-0.1, -3.0, -9.5], [-0.5, -1.5, -2.5]])
    out = tmp_path / "lp.html"
    visualize_log_probs(toks, lps, str(out), argmaxes=[["The", " dog", " x"], ["A", " cat", " ran"]])
    html = out.read_text()
    assert html.count("<span") >= 6 and "data-lp='-3.000'" in html and "&lt;b&gt;" in html and "data-argmax" in html
    out2 = tmp_path / "diff.html"
    visualize_log_prob_diff(toks, lps, lps[::-1].copy(), str(out2))
    assert "diff" in out2.read_text()
