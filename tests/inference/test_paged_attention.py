"""Ragged paged attention and the attention module's paged path on CPU: every way of feeding tokens through the page cache
(token by token, whole prompt, prompt in chunks, several sequences advancing by different amounts) gives what full causal
attention gives (levanter_b200/layers/attention.py, ops/paged_attention.py; scenarios after the reference's
tests/inference/test_paged_attention.py)."""
import math

import numpy as np
import pytest
import torch

from levanter_b200.inference.page_table import PageTable
from levanter_b200.layers.attention import Attention, AttentionConfig, AttentionMask, KvPageCache, default_ragged_paged_attention
from levanter_b200.layers.rotary import DefaultRotaryEmbeddingsConfig

PAGE = 4
H, KV, D = 4, 2, 8


def _naive(q, k, v, scale, soft_cap=None):
    """Causal attention of one sequence whose ``q`` rows are the LAST ``len(q)`` positions of ``k``/``v``."""
    Tq, Tk = q.shape[0], k.shape[0]
    g = q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk.float()) * scale
    if soft_cap:
        s = torch.tanh(s / soft_cap) * soft_cap
    qpos = torch.arange(Tk - Tq, Tk)[:, None]
    s = s.masked_fill(torch.arange(Tk)[None, :] > qpos, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), vv.float())


def _paged_layout(kv_lens, seed=0, shuffle=True):
    """Random K/V per sequence scattered over pages in a shuffled order; returns (kv_pages, page_indices, ks, vs)."""
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = max(math.ceil(n / PAGE) for n in kv_lens)
    total = sum(math.ceil(n / PAGE) for n in kv_lens)
    order = torch.randperm(total + 3, generator=g).tolist() if shuffle else list(range(total + 3))
    kv_pages = torch.zeros(total + 3, PAGE, 2 * KV, D)
    page_indices = torch.full((len(kv_lens), pages_per_seq), -1, dtype=torch.int32)
    ks, vs = [], []
    for s, n in enumerate(kv_lens):
        k, v = torch.randn(n, KV, D, generator=g), torch.randn(n, KV, D, generator=g)
        ks.append(k)
        vs.append(v)
        for p in range(math.ceil(n / PAGE)):
            page = order.pop()
            page_indices[s, p] = page
            m = min(PAGE, n - p * PAGE)
            kv_pages[page, :m, 0::2] = k[p * PAGE:p * PAGE + m]
            kv_pages[page, :m, 1::2] = v[p * PAGE:p * PAGE + m]
    return kv_pages, page_indices, ks, vs


def _check_ragged(kv_lens, q_lens, soft_cap=None, seed=0):
    kv_pages, page_indices, ks, vs = _paged_layout(kv_lens, seed)
    g = torch.Generator().manual_seed(seed + 100)
    qs = [torch.randn(n, H, D, generator=g) for n in q_lens]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    pad = 3  # packed token slots past the last sequence
    q = torch.cat(qs + [torch.randn(pad, H, D, generator=g)])
    scale = 1.0 / math.sqrt(D)
    out = default_ragged_paged_attention(q, kv_pages, torch.tensor(kv_lens, dtype=torch.int32), page_indices, cu,
                                         torch.tensor(len(kv_lens), dtype=torch.int32), sm_scale=scale, soft_cap=soft_cap)
    assert out.shape == q.shape
    for s in range(len(kv_lens)):
        want = _naive(qs[s], ks[s], vs[s], scale, soft_cap)
        got = out[int(cu[s]):int(cu[s + 1])]
        assert torch.allclose(got.float(), want, atol=1e-5, rtol=1e-5), s


def test_one_sequence_whole_prompt_and_single_token():
    _check_ragged([9], [9])
    _check_ragged([9], [1])
    _check_ragged([8], [3])  # the cache ends exactly on a page boundary


@pytest.mark.parametrize("kv_lens,q_lens", [([5, 11, 2], [5, 11, 2]), ([8, 4, 13], [1, 1, 1]), ([7, 12, 3, 16], [2, 12, 1, 5])])
def test_several_sequences_with_ragged_query_and_cache_lengths(kv_lens, q_lens):
    _check_ragged(kv_lens, q_lens)
    _check_ragged(kv_lens, q_lens, soft_cap=20.0, seed=3)


def test_sequences_beyond_num_seqs_are_ignored():
    kv_pages, page_indices, ks, vs = _paged_layout([6, 9])
    q = torch.randn(4, H, D, generator=torch.Generator().manual_seed(1))
    cu = torch.tensor([0, 2, 4], dtype=torch.int32)
    lens = torch.tensor([6, 9], dtype=torch.int32)
    both = default_ragged_paged_attention(q, kv_pages, lens, page_indices, cu, torch.tensor(2), sm_scale=0.3)
    one = default_ragged_paged_attention(q, kv_pages, lens, page_indices, cu, torch.tensor(1), sm_scale=0.3)
    assert torch.allclose(one[:2], both[:2]) and float(one[2:].abs().sum()) == 0.0


# ---------------------------------------------------------------- the attention module over a page table

def _module():
    torch.manual_seed(0)
    cfg = AttentionConfig(hidden_dim=32, num_heads=H, num_kv_heads=KV, rope=DefaultRotaryEmbeddingsConfig(), use_bias=True)
    return Attention(cfg).eval()


def _full(attn, x):
    """Full causal attention of every sequence in ``x[B, S, E]``."""
    pos = torch.arange(x.shape[1])
    with torch.no_grad():
        return attn(x, AttentionMask.causal(), pos)


def _feed(attn, xs, schedule):
    """Push tokens through ``paged_decode`` following ``schedule``: a list of steps, each a list of ``(sequence, n_tokens)``.
    Returns the outputs per sequence, in position order."""
    n_seq = len(xs)
    table = PageTable.init(max_pages=64, max_seqs=n_seq + 1, page_size=PAGE, max_pages_per_seq=8)
    slots = []
    for _ in range(n_seq):
        table, s = table.assign_seq_id_to_seq()
        slots.append(s)
    cache = attn.empty_page_cache(64, PAGE, dtype=torch.float32)
    done = [0] * n_seq
    outs = [[] for _ in range(n_seq)]
    for step in schedule:
        slot_ids, pos_ids, chunks = [], [], []
        for s, n in step:
            slot_ids += [slots[s]] * n
            pos_ids += list(range(done[s], done[s] + n))
            chunks.append(xs[s][done[s]:done[s] + n])
        pad = 2
        slot_ids += [-1] * pad
        pos_ids += [-1] * pad
        x = torch.cat(chunks + [torch.zeros(pad, xs[0].shape[-1])])
        table, info = table.allocate_for_seq(np.array(slot_ids, np.int32), np.array(pos_ids, np.int32))
        with torch.no_grad():
            out, cache = attn.paged_decode(x, cache, info, torch.tensor(pos_ids).clamp(min=0))
        at = 0
        for s, n in step:
            outs[s].append(out[at:at + n])
            at += n
            done[s] += n
    return [torch.cat(o) for o in outs]


def _inputs(lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, 32, generator=g) for n in lengths]


def test_token_by_token_decode_matches_full_attention():
    attn = _module()
    xs = _inputs([7, 7])
    want = _full(attn, torch.stack(xs))
    got = _feed(attn, xs, [[(0, 1), (1, 1)] for _ in range(7)])
    for s in range(2):
        assert torch.allclose(got[s], want[s], atol=1e-5), s


def test_whole_prompt_prefill_matches_full_attention():
    attn = _module()
    xs = _inputs([10, 10, 10], seed=1)
    want = _full(attn, torch.stack(xs))
    got = _feed(attn, xs, [[(0, 10), (1, 10), (2, 10)]])
    for s in range(3):
        assert torch.allclose(got[s], want[s], atol=1e-5), s


@pytest.mark.parametrize("prefix,chunk", [(1, 1), (4, 3), (5, 4), (8, 8)])
def test_prefill_in_chunks_after_a_prefix_matches_full_attention(prefix, chunk):
    attn = _module()
    n = 16
    xs = _inputs([n, n], seed=2)
    want = _full(attn, torch.stack(xs))
    schedule = [[(0, prefix), (1, prefix)]]
    at = prefix
    while at < n:
        m = min(chunk, n - at)
        schedule.append([(0, m), (1, m)])
        at += m
    got = _feed(attn, xs, schedule)
    for s in range(2):
        assert torch.allclose(got[s], want[s], atol=1e-5), (s, prefix, chunk)


def test_sequences_that_advance_by_different_amounts_match_full_attention():
    attn = _module()
    xs = _inputs([12, 12], seed=3)
    want = _full(attn, torch.stack(xs))
    # sequence 0 in chunks of 4, 2, 6; sequence 1 in chunks of 3, 9, joining a step late
    got = _feed(attn, xs, [[(0, 4)], [(0, 2), (1, 3)], [(1, 9), (0, 6)]])
    for s in range(2):
        assert torch.allclose(got[s], want[s], atol=1e-5), s


def test_page_cache_update_drops_padding_tokens_and_copy_page_copies():
    cache = KvPageCache.init(4, PAGE, KV, D, dtype=torch.float32)
    table = PageTable.init(max_pages=4, max_seqs=2, page_size=PAGE, max_pages_per_seq=2)
    table, s = table.assign_seq_id_to_seq()
    table, info = table.allocate_for_seq(np.array([s, s, s, -1], np.int32), np.array([0, 1, 2, -1], np.int32))
    k, v = torch.ones(4, KV, D), 2 * torch.ones(4, KV, D)
    cache = cache.update(info, k, v)
    page = int(info.page_indices[0, 0])
    assert float(cache.kv_pages[page, :3, 0::2].sum()) == 3 * KV * D and float(cache.kv_pages[page, :3, 1::2].sum()) == 2 * 3 * KV * D
    assert float(cache.kv_pages.sum()) == 3 * 3 * KV * D  # the padding token went nowhere
    other = (page + 1) % 4
    cache = cache.copy_page(page, other)
    assert torch.equal(cache.kv_pages[other], cache.kv_pages[page])
