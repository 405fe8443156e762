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


def test_log_probability_pages_from_models_and_the_training_hook(tmp_path):
    """Per-token log-probabilities of a model over a loader end up in a page (position t shows the probability OF token t);
    a second model gives a difference page; the hook form writes one page per call and logs it as an artifact."""
    import torch

    import levanter_b200.tracker as T
    from levanter_b200.analysis.visualization import (cb_compute_and_visualize_log_probs, compute_and_diff_log_probs,
                                                      compute_and_visualize_log_probs)
    from levanter_b200.data.loader import DataLoader
    from levanter_b200.data.passthrough_tokenizer import PassthroughTokenizer
    from levanter_b200.models.llama import LlamaConfig
    from levanter_b200.models.lm_model import LmExample

    cfg = LlamaConfig(seq_len=8, hidden_dim=16, intermediate_dim=32, num_layers=1, num_heads=2, num_kv_heads=2)
    a, b = cfg.build(50, seed=0).eval(), cfg.build(50, seed=1).eval()
    data = ListAsyncDataset([LmExample.causal(torch.arange(i, i + 8, dtype=torch.int32)) for i in range(6)], is_complete=True)
    loader = DataLoader(data, 2, max_buffered_batches=0, pin_memory=False)
    tok = PassthroughTokenizer(50)

    def log_prob_fn(model, batch):
        logits = model(batch.tokens, batch.attn_mask).float()
        lp = torch.log_softmax(logits, -1)
        targets = torch.roll(batch.tokens, -1, dims=-1).long()
        return lp.gather(-1, targets.unsqueeze(-1)).squeeze(-1), logits.argmax(-1)

    page = tmp_path / "lp.html"
    compute_and_visualize_log_probs(str(page), a, tok, log_prob_fn, loader, max_docs=5)
    html = page.read_text()
    assert html.count("<br><br>") == 5 and html.count("<span") == 5 * 8 and "data-argmax" in html
    assert html.count("data-lp='0.000'") >= 5  # the first token of a document has nothing before it
    with torch.no_grad():
        first = LmExample.stack([data.as_sync_dataset()[0]])
        want = float(log_prob_fn(a, first)[0][0, 0])
    assert f"data-lp='{want:.3f}'" in html  # shown under token 1, which position 0 predicts

    diff = tmp_path / "diff.html"
    compute_and_diff_log_probs(str(diff), a, b, tok, log_prob_fn, loader, max_docs=4)
    assert diff.read_text().count("<br><br>") == 4 and "diff" in diff.read_text()
    same = tmp_path / "same.html"
    compute_and_diff_log_probs(str(same), a, a, tok, log_prob_fn, loader, max_docs=2)
    assert "diff 0.000" in same.read_text() and "diff 0.5" not in same.read_text()

    class Recorder(T.NoopTracker):
        def __init__(self):
            self.artifacts = []

        def log_artifact(self, artifact_path, *, name=None, type=None):
            self.artifacts.append((os.path.basename(str(artifact_path)), name, type))

    import os
    from types import SimpleNamespace

    rec = Recorder()
    hook = cb_compute_and_visualize_log_probs(loader, tok, log_prob_fn, str(tmp_path / "pages"), max_docs=2)
    with T.current_tracker(rec):
        hook(SimpleNamespace(step=7, eval_model=a))
    assert os.path.exists(tmp_path / "pages" / "step_7.html") and rec.artifacts == [("step_7.html", "log_probs_step_7.html", "html")]
