"""Generation engine: slot/page release and reuse with a dummy model, clones, and a real model whose paged greedy decoding
must equal re-running the full forward pass token by token."""
import logging

import numpy as np
import pytest
import torch

from levanter_b200.inference.engine import InferenceEngine, InferenceEngineConfig, Request
from levanter_b200.inference.jit_scheduler import SeqDecodingParams
from levanter_b200.layers.attention import AttentionMask, KvPageCache
from levanter_b200.models.llama import LlamaConfig


class DummyModel:
    """``decode`` always prefers token ``eos``; the cache is unused."""

    def __init__(self, vocab_size: int, eos_id: int = 3):
        self.vocab_size, self.eos = vocab_size, eos_id

    def initial_cache(self, page_table, *, dtype):
        return KvPageCache.init(page_table.num_pages, page_table.page_size, 1, 8, dtype=dtype)

    def decode(self, input_ids, kv_cache, batch_info, pos_ids):
        logits = torch.zeros(input_ids.shape[0], self.vocab_size)
        logits[:, self.eos] = 1.0
        return logits, kv_cache


def _service(**kw):
    return InferenceEngine.from_model(model=DummyModel(10), tokenizer=None, max_pages=64, max_seqs=8, page_size=8, max_pages_per_seq=4,
                                      compute_dtype=torch.float32, max_queued_tokens=64, max_seqs_in_prefill=4, **kw)


def _req(i, toks, n=1, extra=5, stop=(3,), temperature=0.0, key=None):
    params = SeqDecodingParams(max_num_tokens=len(toks) + extra, stop_tokens=None if stop is None else np.array([list(stop)], np.int32),
                               temperature=temperature, key=i if key is None else key)
    return Request(prompt_tokens=list(toks), request_id=i, decode_params=params, n_generations=n)


def test_release_on_finish_and_reuse_slots(caplog):
    caplog.set_level(logging.INFO)
    svc = _service()
    result = svc.generate([_req(0, [7, 7]), _req(1, [1])])
    assert result.tokens == [[3], [3]] and result.total_generated == 2
    pt = svc.gen_state.decode_state.page_table
    assert not pt.used_mask.any() and (pt.seq_lens == 0).all() and int(pt.page_ref_counts.sum()) == 0
    assert any("Releasing finished sequences" in r.message for r in caplog.records)
    result2 = svc.generate([_req(0, [5, 5, 5], extra=3)])
    assert result2.tokens == [[3]] and result2.total_generated == 1


def test_reuse_with_clones_and_slot_reassignment():
    svc = _service()
    for seed in (0, 100):
        out = svc.generate([_req(i, p, n=3, key=seed + i) for i, p in enumerate([[7, 7], [1, 2]])])
        assert len(out.tokens) == 6 and all(t == [3] for t in out.tokens)
    pt = svc.gen_state.decode_state.page_table
    assert not pt.used_mask.any() and int(pt.page_ref_counts.sum()) == 0


def test_length_limit_and_more_requests_than_slots():
    svc = _service()
    reqs = [_req(i, [1, 2, 3], extra=4, stop=None) for i in range(20)]  # no stop sequence: runs to the length limit
    out = svc.generate(reqs)
    assert all(t == [3, 3, 3, 3] for t in out.tokens) and out.total_generated == 80


def test_request_that_can_never_fit_is_rejected():
    svc = _service()
    with pytest.raises(ValueError):
        svc.generate([_req(0, list(range(40)))])  # 4 pages of 8 hold 32 tokens


def _tiny_llama():
    cfg = LlamaConfig(seq_len=64, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=4, num_kv_heads=2)
    return cfg.build(50, seed=0).eval()


def _greedy_full_forward(model, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        ids = torch.tensor([toks], dtype=torch.int32)
        with torch.no_grad():
            acts = model.activations(ids, AttentionMask.causal())
            logits = acts[0, -1] @ model.get_lm_head().t()
        toks.append(int(logits.argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("max_rounds", [1, 4])
def test_paged_greedy_decoding_matches_full_forward(max_rounds):
    model = _tiny_llama()
    cfg = InferenceEngineConfig(max_seqs=4, page_size=4, max_pages_per_seq=8, max_pages=24, compute_dtype=torch.float32,
                                max_rounds=max_rounds, max_seqs_in_prefill=2, enable_logprobs=True)
    eng = InferenceEngine.from_model_with_config(model, None, cfg)
    prompts = [[5, 9, 2], [7], [11, 12, 13, 14, 15, 16, 17], [3, 4], [20, 21, 22, 23, 24]]
    reqs = [_req(i, p, extra=6, stop=None) for i, p in enumerate(prompts)]
    out = eng.generate(reqs)
    for p, got, lps in zip(prompts, out.tokens, out.logprobs):
        assert got == _greedy_full_forward(model, p, 6)
        assert len(lps) == 6 and all(lp <= 0 for lp in lps)
    pt = eng.gen_state.decode_state.page_table
    assert not pt.used_mask.any() and int(pt.page_ref_counts.sum()) == 0


def test_clones_share_prefix_and_sample_independently():
    model = _tiny_llama()
    cfg = InferenceEngineConfig(max_seqs=6, page_size=4, max_pages_per_seq=8, compute_dtype=torch.float32, max_rounds=3)
    eng = InferenceEngine.from_model_with_config(model, None, cfg)
    prompt = [5, 9, 2, 8, 1, 6]  # ends inside a page: the clones get a private copy of the last page
    greedy = eng.generate([_req(0, prompt, n=3, extra=5, stop=None)])
    want = _greedy_full_forward(model, prompt, 5)
    assert all(t == want for t in greedy.tokens)
    sampled = eng.generate([_req(0, prompt, n=4, extra=8, stop=None, temperature=1.5, key=7)])
    assert len({tuple(t) for t in sampled.tokens}) > 1  # different keys, different continuations
    again = eng.generate([_req(0, prompt, n=4, extra=8, stop=None, temperature=1.5, key=7)])
    assert again.tokens == sampled.tokens  # same keys, same continuations


def test_stop_sequence_of_two_tokens():
    model = _tiny_llama()
    eng = InferenceEngine.from_model_with_config(model, None, InferenceEngineConfig(max_seqs=2, page_size=4, max_pages_per_seq=8,
                                                                                    compute_dtype=torch.float32, max_rounds=4))
    prompt = [5, 9, 2]
    full = _greedy_full_forward(model, prompt, 8)
    stop = full[2:4]
    out = eng.generate([_req(0, prompt, extra=8, stop=stop)])
    assert out.tokens[0] == full[:4]


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_workloads_on_a_small_page_pool_match_plain_greedy_decoding(seed):
    """Many requests of random prompt lengths, generation lengths, clone counts and stop sequences, served by an engine with
    few slots, few pages and small prefill batches, so that requests queue, prefill in pieces and reuse freed pages: every
    generation must equal token-by-token greedy decoding of the full forward pass, and nothing may leak."""
    rng = np.random.default_rng(seed)
    model = _tiny_llama()
    cfg = InferenceEngineConfig(max_seqs=3 + seed, page_size=4, max_pages_per_seq=6, max_pages=14 + 4 * seed, compute_dtype=torch.float32,
                                max_rounds=int(rng.integers(1, 5)), max_seqs_in_prefill=2, max_prefill_size=16, max_queued_tokens=16)
    eng = InferenceEngine.from_model_with_config(model, None, cfg)
    for wave in range(2):  # the second call starts from the state the first one left
        reqs, want = [], []
        for i in range(7):
            prompt = rng.integers(1, 50, size=int(rng.integers(1, 13))).tolist()
            n_new = int(rng.integers(1, 24 - len(prompt)))
            n = int(rng.integers(1, 3))
            full = _greedy_full_forward(model, prompt, n_new)
            stop = None
            if n_new >= 3 and rng.random() < 0.4:
                at = int(rng.integers(1, n_new - 1))
                stop = full[at:at + 2]
                first = next(j for j in range(len(full) - 1) if full[j:j + 2] == stop)
                full = full[:first + 2]  # generation ends with the first occurrence of the stop sequence
            reqs.append(_req(i, prompt, n=n, extra=n_new, stop=stop))
            want += [full] * n
        out = eng.generate(reqs)
        assert out.tokens == want, (seed, wave)
        assert out.total_generated == sum(len(w) for w in want)
        pt = eng.gen_state.decode_state.page_table
        assert not pt.used_mask.any() and int(pt.page_ref_counts.sum()) == 0 and pt.num_free_pages == pt.num_pages
