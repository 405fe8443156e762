"""Sequence packing: the online packer, prompt/completion packers, the packed view over jagged stores and the per-segment
reductions (levanter_b200/data/packing.py; scenarios after the reference's tests/test_packing.py)."""
import asyncio

import numpy as np
import pytest
import torch

from levanter_b200.data.packing import (GreedyPrepackedDataset, PromptCompletion, SequencePacker, greedy_pack_prompt_completions,
                                        pack_documents, pack_prompt_completions, per_segment_correct, per_segment_loss)
from levanter_b200.store.jagged_array import JaggedArrayStore


def _seg(ex):
    s = ex.attn_mask.segment_ids
    return (s[0] if isinstance(s, tuple) else s).tolist()


# ---------------------------------------------------------------- the online packer

def test_can_pack_counts_tokens_and_segments():
    p = SequencePacker(10, max_pack_size=2, pad_token=0)
    assert p.can_pack([1, 2, 3])
    p.add_example([1, 2, 3], [1, 1, 1])
    assert p.can_pack([4, 5]) and not p.can_pack(list(range(8)))
    p.add_example([4, 5], [1, 1])
    assert not p.can_pack([6])  # two segments already


def test_add_example_and_pack_pads_with_the_pad_token_and_segment_minus_one():
    p = SequencePacker(10, max_pack_size=2, pad_token=7)
    p.add_example([1, 2, 3], [1, 1, 1])
    ex = p.pack()
    assert ex.tokens.tolist() == [1, 2, 3] + [7] * 7
    assert _seg(ex) == [0, 0, 0] + [-1] * 7
    assert ex.loss_mask.tolist() == [1, 1, 1] + [0] * 7
    assert ex.attn_mask.is_causal


def test_adding_past_the_capacity_raises():
    p = SequencePacker(10, max_pack_size=2, pad_token=0)
    p.add_example([1, 2, 3], [1, 1, 1])
    with pytest.raises(ValueError, match="Too many tokens"):
        p.add_example(list(range(8)), [1] * 8)
    p.add_example([4], [1])
    with pytest.raises(ValueError, match="Too many segments"):
        p.add_example([5], [1])
    with pytest.raises(ValueError, match="same length"):
        SequencePacker(10, 2, 0).add_example([1, 2], [1])
    with pytest.raises(ValueError):
        SequencePacker(10, 2, None)


def test_an_empty_sequence_adds_nothing():
    p = SequencePacker(10, max_pack_size=2, pad_token=0)
    p.add_example([], [])
    assert p.num_segments == 0
    ex = p.pack()
    assert ex.tokens.tolist() == [0] * 10 and _seg(ex) == [-1] * 10 and ex.loss_mask.sum() == 0


def test_several_examples_share_a_row_with_their_own_segment_ids():
    p = SequencePacker(10, max_pack_size=3, pad_token=9)
    p.add_example([1, 2], [1, 1])
    p.add_example([3, 4, 5], [1, 0, 1], segment_id=41)
    ex = p.pack()
    assert ex.tokens.tolist() == [1, 2, 3, 4, 5, 9, 9, 9, 9, 9]
    assert _seg(ex) == [0, 0, 41, 41, 41, -1, -1, -1, -1, -1]
    assert ex.loss_mask.tolist() == [1, 1, 1, 0, 1, 0, 0, 0, 0, 0]


# ---------------------------------------------------------------- prompt / completion pairs

def test_prompt_completion_rejects_empty_and_prompt_only_sequences():
    with pytest.raises(ValueError):
        PromptCompletion([], 0)
    with pytest.raises(ValueError):
        PromptCompletion([1, 2], 2)


def test_pack_prompt_completions_masks_prompts_and_the_last_token():
    seqs = [PromptCompletion([1, 2, 3], 2), PromptCompletion([4, 5], 1), PromptCompletion([6, 7, 8], 1)]
    packed = list(pack_prompt_completions(10, seqs, pad_token=0, max_segments_per_example=2))
    assert len(packed) == 2
    first, second = packed
    assert first.tokens.tolist() == [1, 2, 3, 4, 5, 0, 0, 0, 0, 0]
    assert _seg(first) == [0, 0, 0, 1, 1, -1, -1, -1, -1, -1]
    # loss on the positions that PREDICT a completion token: from the last prompt token to the one before the sequence's end
    assert first.loss_mask.tolist() == [0, 1, 0, 1, 0, 0, 0, 0, 0, 0]
    assert second.tokens.tolist() == [6, 7, 8] + [0] * 7
    assert second.loss_mask.tolist() == [1, 1, 0] + [0] * 7


def test_pack_prompt_completions_emits_the_oldest_row_when_the_buffer_is_full():
    # every sequence fills more than half a row, so none share a row; at most two rows stay open
    seqs = [PromptCompletion([i] * 6, 2, segment_id=i) for i in range(1, 6)]
    packed = list(pack_prompt_completions(10, seqs, pad_token=0, max_segments_per_example=4, max_buffered_examples=2))
    assert len(packed) == 5
    assert [ex.tokens[0].item() for ex in packed] == [1, 2, 3, 4, 5]  # emitted in arrival order
    for i, ex in enumerate(packed, 1):
        assert _seg(ex) == [i] * 6 + [-1] * 4

    # a later short sequence still lands in the first open row that has room
    seqs = [PromptCompletion([1] * 6, 2), PromptCompletion([2] * 7, 2), PromptCompletion([3] * 4, 2), PromptCompletion([4] * 3, 1)]
    packed = list(pack_prompt_completions(10, seqs, pad_token=0, max_segments_per_example=4, max_buffered_examples=8))
    assert [sorted(set(ex.tokens.tolist()) - {0}) for ex in packed] == [[1, 3], [2, 4]]


def test_greedy_pack_prompt_completions_keeps_the_order_and_numbers_segments_by_position():
    seqs = [PromptCompletion([1, 2, 3], 2), PromptCompletion([4, 5], 1), PromptCompletion([6, 7, 8, 9, 10, 11], 3), PromptCompletion([12, 13], 1)]
    packed = greedy_pack_prompt_completions(10, seqs, pad_token=0, max_segments_per_example=8)
    assert len(packed) == 2
    assert packed[0].tokens.tolist() == [1, 2, 3, 4, 5, 0, 0, 0, 0, 0]
    assert _seg(packed[0]) == [0, 0, 0, 1, 1] + [-1] * 5
    assert packed[1].tokens.tolist() == [6, 7, 8, 9, 10, 11, 12, 13, 0, 0]
    assert _seg(packed[1]) == [2] * 6 + [3] * 2 + [-1] * 2
    assert packed[1].loss_mask.tolist() == [0, 0, 1, 1, 1, 0, 1, 0, 0, 0]


def test_greedy_pack_prompt_completions_respects_the_segment_limit():
    seqs = [PromptCompletion([i, i], 1) for i in range(1, 6)]
    packed = greedy_pack_prompt_completions(16, seqs, pad_token=0, max_segments_per_example=2)
    assert [sorted(set(_seg(ex)) - {-1}) for ex in packed] == [[0, 1], [2, 3], [4]]


def test_greedy_pack_prompt_completions_keeps_the_end_of_a_sequence_that_is_too_long():
    long = PromptCompletion(list(range(1, 15)), 3)
    packed = greedy_pack_prompt_completions(10, [PromptCompletion([50, 51], 1), long, PromptCompletion([60, 61], 1)], pad_token=0)
    assert len(packed) == 3
    assert packed[1].tokens.tolist() == list(range(5, 15))  # the last ten tokens: the completion is what is scored
    assert _seg(packed[1]) == [1] * 10
    assert packed[1].loss_mask.tolist() == [1] * 9 + [0]


def test_greedy_pack_prompt_completions_of_nothing_is_nothing():
    assert greedy_pack_prompt_completions(10, [], pad_token=0) == []


# ---------------------------------------------------------------- per-segment reductions

def _packed_example():
    p = SequencePacker(8, max_pack_size=3, pad_token=0)
    p.add_example([1, 2, 3], [1, 1, 0], segment_id=2)
    p.add_example([4, 5, 6, 7], [0, 1, 1, 1], segment_id=5)
    return p.pack()


def test_per_segment_loss_sums_masked_losses_by_segment():
    ex = _packed_example()
    losses = torch.arange(1, 9, dtype=torch.float32)
    ids, sums = per_segment_loss(ex, losses, 4)
    by_id = dict(zip(ids.tolist(), sums.tolist()))
    assert by_id[2] == 1 + 2 and by_id[5] == 5 + 6 + 7
    assert by_id[-1] == 0  # padding: masked out
    assert ids.shape == (4,) and sorted(ids.tolist()) == [-1, -1, 2, 5]


def test_per_segment_correct_is_true_when_every_scored_token_is_right():
    ex = _packed_example()
    correct = torch.tensor([1, 1, 0, 0, 1, 0, 1, 0], dtype=torch.bool)  # segment 2: wrong only where unscored; segment 5: one miss
    ids, ok = per_segment_correct(ex, correct, 4)
    by_id = dict(zip(ids.tolist(), ok.tolist()))
    assert by_id[2] is True and by_id[5] is False
    correct[5] = True
    ids, ok = per_segment_correct(ex, correct, 4)
    assert dict(zip(ids.tolist(), ok.tolist()))[5] is True


def test_per_segment_reductions_need_segment_ids():
    from levanter_b200.layers.attention import AttentionMask
    from levanter_b200.models.lm_model import LmExample

    ex = LmExample(tokens=torch.zeros(4, dtype=torch.int32), loss_mask=torch.ones(4, dtype=torch.int32), attn_mask=AttentionMask.causal())
    with pytest.raises(ValueError, match="segment_ids"):
        per_segment_loss(ex, torch.zeros(4), 2)


# ---------------------------------------------------------------- packing from lengths

def test_pack_documents_is_contiguous_and_greedy():
    assert pack_documents(np.array([3, 3, 3, 3]), 6) == [range(0, 2), range(2, 4)]
    assert pack_documents(np.array([5, 2, 2, 2, 5]), 6) == [range(0, 1), range(1, 4), range(4, 5)]
    assert pack_documents(np.array([], dtype=np.int64), 6) == []
    assert pack_documents(np.array([1] * 7), 100, max_segments_per_example=3) == [range(0, 3), range(3, 6), range(6, 7)]


def test_pack_documents_with_several_leaves_closes_a_pack_when_any_leaf_is_full():
    lengths = {"a": np.array([2, 2, 2, 2]), "b": np.array([1, 5, 1, 1])}
    assert pack_documents(lengths, {"a": 100, "b": 6}) == [range(0, 2), range(2, 4)]
    assert pack_documents(lengths, 6) == [range(0, 2), range(2, 4)]  # one capacity for every leaf
    assert pack_documents(lengths, {"a": 4, "b": 100}) == [range(0, 2), range(2, 4)]
    assert pack_documents(lengths, {"a": 3, "b": 100}) == [range(i, i + 1) for i in range(4)]


def test_pack_documents_argument_errors():
    with pytest.raises(ValueError, match="positive integer"):
        pack_documents(np.array([1, 2]), 4, max_segments_per_example=0)
    with pytest.raises(ValueError, match="positive integer"):
        pack_documents(np.array([1, 2]), 4, max_segments_per_example=-2)
    with pytest.raises(ValueError, match="same number of documents"):
        pack_documents({"a": np.array([1, 2]), "b": np.array([1, 2, 3])}, 4)
    with pytest.raises(ValueError, match="same number of leaves"):
        pack_documents({"a": np.array([1, 2])}, {"a": 4, "b": 4})
    with pytest.raises(ValueError, match="exceeds maximum allowed length"):
        pack_documents(np.array([1, 9]), 4)
    assert pack_documents(np.array([1, 9, 1]), 4, slice_too_long_examples=True) == [range(0, 1), range(1, 2), range(2, 3)]


# ---------------------------------------------------------------- the packed view over stores

def _store(path, rows, dtype=np.int32):
    s = JaggedArrayStore.open(str(path), mode="w", dtype=dtype)
    s.extend([np.asarray(r, dtype=dtype) for r in rows])
    return s


def _get(ds, idx):
    return asyncio.run(ds.get_batch(idx))


def test_packed_view_over_one_store(tmp_path):
    rows = [[1, 2, 3], [4, 5], [6, 7, 8, 9], [10], [11, 12]]
    ds = GreedyPrepackedDataset(_store(tmp_path / "s", rows), max_length=6)
    assert asyncio.run(ds.async_len()) == 3 and ds.is_finite()
    (d0, s0), (d1, s1), (d2, s2) = _get(ds, [0, 1, 2])
    assert d0.tolist() == [1, 2, 3, 4, 5, 0] and s0.tolist() == [0, 0, 0, 1, 1, -1]
    assert d1.tolist() == [6, 7, 8, 9, 10, 0] and s1.tolist() == [2, 2, 2, 2, 3, -1]
    assert d2.tolist() == [11, 12, 0, 0, 0, 0] and s2.tolist() == [4, 4, -1, -1, -1, -1]
    # any order, repeated indices
    (e2, _), (e0, _), (e2b, _) = _get(ds, [2, 0, 2])
    assert e2.tolist() == d2.tolist() == e2b.tolist() and e0.tolist() == d0.tolist()


def test_packed_view_without_padding_returns_ragged_rows(tmp_path):
    rows = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    ds = GreedyPrepackedDataset(_store(tmp_path / "s", rows), max_length=6, pad_with_zeros=False)
    (d0, s0), (d1, s1) = _get(ds, [0, 1])
    assert d0.tolist() == [1, 2, 3, 4, 5] and s0.tolist() == [0, 0, 0, 1, 1]
    assert d1.tolist() == [6, 7, 8, 9] and s1.tolist() == [2, 2, 2, 2]


def test_packed_view_respects_the_segment_limit(tmp_path):
    rows = [[i] for i in range(1, 8)]
    ds = GreedyPrepackedDataset(_store(tmp_path / "s", rows), max_length=10, max_segments_per_example=3)
    assert asyncio.run(ds.async_len()) == 3
    out = _get(ds, [0, 1, 2])
    assert [d[:3].tolist() for d, _ in out] == [[1, 2, 3], [4, 5, 6], [7, 0, 0]]
    assert out[2][1].tolist() == [6] + [-1] * 9


def test_packed_view_over_a_tree_of_stores(tmp_path):
    ids = [[1, 2, 3], [4, 5], [6, 7, 8, 9], [10]]
    aux = [[1.5], [2.5, 3.5, 4.5], [5.5], [6.5, 7.5]]
    tree = {"input_ids": _store(tmp_path / "a", ids), "aux": {"w": _store(tmp_path / "b", aux, np.float32)}}
    ds = GreedyPrepackedDataset(tree, max_length={"input_ids": 6, "aux": {"w": 4}})
    assert asyncio.run(ds.async_len()) == 2
    (d0, s0), (d1, s1) = _get(ds, [0, 1])
    assert d0["input_ids"].tolist() == [1, 2, 3, 4, 5, 0] and s0["input_ids"].tolist() == [0, 0, 0, 1, 1, -1]
    assert d0["aux"]["w"].tolist() == [1.5, 2.5, 3.5, 4.5] and s0["aux"]["w"].tolist() == [0, 1, 1, 1]
    assert d1["input_ids"].tolist() == [6, 7, 8, 9, 10, 0] and s1["aux"]["w"].tolist() == [2, 3, 3, -1]
    assert d1["aux"]["w"].dtype == np.float32

    # the auxiliary leaf's capacity closes packs earlier
    ds = GreedyPrepackedDataset(tree, max_length={"input_ids": 100, "aux": {"w": 3}})
    assert [len(set(s["input_ids"].tolist()) - {-1}) for _, s in _get(ds, range(asyncio.run(ds.async_len())))] == [1, 1, 2]


@pytest.mark.parametrize("strategy,kept", [("left", [1, 2, 3, 4]), ("right", [4, 5, 6, 7])])
def test_a_document_longer_than_the_capacity_is_cut_on_the_chosen_side(tmp_path, strategy, kept):
    rows = [[9, 9], [1, 2, 3, 4, 5, 6, 7], [8]]
    ds = GreedyPrepackedDataset(_store(tmp_path / "s", rows), max_length=4, slice_strategy=strategy)
    out = _get(ds, [0, 1, 2])
    assert out[0][0].tolist() == [9, 9, 0, 0]
    assert out[1][0].tolist() == kept and out[1][1].tolist() == [1, 1, 1, 1]
    assert out[2][0].tolist() == [8, 0, 0, 0] and out[2][1].tolist() == [2, -1, -1, -1]


def test_a_document_longer_than_the_capacity_is_refused_by_default(tmp_path):
    s = _store(tmp_path / "s", [[1, 2], [1, 2, 3, 4, 5, 6, 7]])
    with pytest.raises(ValueError, match="exceeds maximum allowed length"):
        GreedyPrepackedDataset(s, max_length=4)
    with pytest.raises(ValueError, match="slice_strategy"):
        GreedyPrepackedDataset(s, max_length=4, slice_strategy="middle")
    with pytest.raises(ValueError, match="positive integer"):
        GreedyPrepackedDataset(s, max_length=8, max_segments_per_example=0)
