"""Page table, token queue, decode state and the small inference helpers; the native (C++) and numpy paths must agree."""
import numpy as np
import pytest

from levanter_b200.inference import page_table as PT
from levanter_b200.inference.jit_scheduler import DecodeState, SeqDecodingParams, TokenQueue
from levanter_b200.inference.page_table import PageBatchInfo, PageTable
from levanter_b200.inference.utils import INVALID, get_unique_in_order, is_stop_signal, purge


def _make_table(pages=8, seqs=4, page_size=2, pages_per_seq=2):
    return PageTable.init(pages, seqs, page_size, pages_per_seq)


@pytest.fixture(params=["native", "numpy"])
def backend(request, monkeypatch):
    if request.param == "numpy":
        monkeypatch.setattr(PT, "_native", None)
        monkeypatch.setattr(PT, "_native_tried", True)
    elif PT._lib() is None:
        pytest.skip("native library not built")
    return request.param


def test_max_len_per_seq():
    assert _make_table(page_size=2, pages_per_seq=3).max_len_per_seq == 6


def test_free_pages(backend):
    pt = _make_table()
    pt.page_ref_counts[:2] = 1
    pt.page_indices[0, :2] = [0, 1]
    pt.seq_lens[0] = 4
    pt.used_mask[0] = True
    freed = pt.free_pages(0)
    assert (freed.page_ref_counts[:2] == 0).all() and (freed.page_indices[0] == INVALID).all()
    assert freed.seq_lens[0] == 0 and not freed.used_mask[0]
    assert pt.page_ref_counts[0] == 1  # value semantics: the original is untouched
    same = pt.free_pages(-1)
    assert same is pt


def test_allocate_single_token(backend):
    pt, sid = _make_table().assign_seq_id_to_seq()
    assert sid == 0
    new_pt, info = pt.allocate_for_seq(np.zeros(1, np.int32), np.zeros(1, np.int32))
    assert info.new_token_dests[0] == 0 and new_pt.seq_lens[0] == 1 and int(info.num_seqs) == 1
    assert isinstance(info, PageBatchInfo) and info.cu_q_lens.shape[0] == pt.max_seqs + 1


def test_allocate_updates_only_used_slots(backend):
    pt = _make_table(seqs=8, pages=16)
    pt.used_mask[:6] = True
    slots = np.array([2, 3, 3, 5, 5, 5], np.int32)
    pos = np.array([0, 0, 1, 0, 1, 2], np.int32)
    new_pt, info = pt.allocate_for_seq(slots, pos)
    assert new_pt.seq_lens[:6].tolist() == [0, 0, 1, 2, 0, 3] and (new_pt.seq_lens[6:] == 0).all()
    assert int(info.num_seqs) == 3
    assert info.slot_ids[:3].tolist() == [2, 3, 5] and info.cu_q_lens[:4].tolist() == [0, 1, 3, 6]
    pages, offs = info.pages_and_slots()
    # slot 5 has 3 tokens with page size 2: two pages, the third token starts the second one
    assert offs.tolist() == [0, 0, 1, 0, 1, 0] and pages[3] == pages[4] != pages[5]
    assert sorted(set(pages.tolist())) == [0, 1, 2, 3]
    assert new_pt.page_ref_counts[:4].tolist() == [1, 1, 1, 1]


def test_allocate_with_padding_tokens_and_growth(backend):
    pt, _ = _make_table(pages=4, seqs=2, page_size=2, pages_per_seq=2).assign_seq_id_to_seq()
    pt, info = pt.allocate_for_seq(np.array([0, 0, -1, INVALID], np.int32), np.array([0, 1, INVALID, INVALID], np.int32))
    assert info.new_token_dests.tolist()[:2] == [0, 1] and (info.new_token_dests[2:] == INVALID).all()
    pt, info = pt.allocate_for_seq(np.array([0], np.int32), np.array([2], np.int32))  # decode step: crosses into page two
    assert pt.seq_lens[0] == 3 and info.new_token_dests[0] == 2 and pt.page_ref_counts.tolist() == [1, 1, 0, 0]
    assert info.seq_lens[0] == 3


def test_out_of_pages_raises(backend):
    pt, _ = _make_table(pages=1, seqs=1, page_size=2, pages_per_seq=4).assign_seq_id_to_seq()
    with pytest.raises(RuntimeError, match="Out of free pages"):
        pt.allocate_for_seq(np.zeros(3, np.int32), np.arange(3, dtype=np.int32))


def test_assign_seq_id(backend):
    pt, a = _make_table(seqs=4).assign_seq_id_to_seq()
    assert a == 0
    pt, b = pt.assign_seq_id_to_seq(2)
    assert b == 2 and pt.used_mask[2] and (pt.seq_lens == 0).all()
    pt2, c = pt.assign_seq_id_to_seq(2)
    assert c == INVALID and pt2 is pt
    pt, d = pt.assign_seq_id_to_seq()
    assert d == 1


def test_clone_pages_partial_last_page_gets_fresh_page(backend):
    pt = _make_table(pages=8, seqs=4, page_size=4, pages_per_seq=3)
    pt, s = pt.assign_seq_id_to_seq()
    pt, _ = pt.allocate_for_seq(np.zeros(6, np.int32), np.arange(6, dtype=np.int32))  # pages 0 (full) and 1 (partial)
    c = pt.clone_pages_from(0, 1)
    assert c.page_indices[1, 0] == 0 and c.page_indices[1, 1] not in (0, 1, INVALID)
    assert c.page_ref_counts[0] == 2 and c.page_ref_counts[1] == 1 and c.page_ref_counts[c.page_indices[1, 1]] == 1
    assert c.seq_lens[1] == 6 and c.used_mask[1]


def test_clone_pages_at_boundary_shares_last_page(backend):
    pt = _make_table(pages=8, seqs=4, page_size=4, pages_per_seq=3)
    pt, _ = pt.assign_seq_id_to_seq()
    pt, _ = pt.allocate_for_seq(np.zeros(8, np.int32), np.arange(8, dtype=np.int32))
    c = pt.clone_pages_from(0, 2)
    assert c.page_indices[2, :2].tolist() == [0, 1] and c.page_ref_counts[:2].tolist() == [2, 2]
    freed = c.free_pages(0)
    assert freed.page_ref_counts[:2].tolist() == [1, 1]  # still referenced by the clone


def test_token_queue_pack_sorted_by_slot(backend):
    tq = TokenQueue.init(8)
    tq = tq.enqueue_tokens(np.array([10, 11, 12, 20, 21, 22, 23]), np.array([1, 1, 1, 0, 0, 0, 0]), np.array([0, 1, 2, 0, 1, 2, 3]), 6)
    assert tq.num_queued_tokens == 6
    tq2, packed = tq.pack_next_sequence(4)
    assert packed.num_tokens == 4 and tq2.num_queued_tokens == 2 and tq.num_queued_tokens == 6
    assert packed.slot_ids.tolist() == [0, 1, 1, 1] and packed.tokens.tolist() == [20, 10, 11, 12] and packed.pos_ids.tolist() == [0, 0, 1, 2]
    assert tq2.queued_tokens[:2].tolist() == [21, 22] and (tq2.queued_tokens[2:] == INVALID).all()
    tq3 = tq.purge_queue_of_slot(1)
    assert tq3.num_queued_tokens == 3 and tq3.queued_tokens[:3].tolist() == [20, 21, 22]
    tq4, p4 = tq2.pack_next_sequence(4)
    assert p4.num_tokens == 2 and p4.tokens.tolist() == [21, 22, INVALID, INVALID] and tq4.num_queued_tokens == 0


def test_pack_boundaries_match_page_table(backend):
    tq = TokenQueue.init(6).enqueue_tokens(np.array([10, 11, 12, 20, 21, 22, 23]), np.array([1, 1, 1, 0, 0, 0, 0]),
                                           np.array([0, 1, 2, 0, 1, 2, 3]), 6)
    _, packed = tq.pack_next_sequence(6)
    pt = PageTable.init(16, 4, 8, 4)
    pt, _ = pt.assign_seq_id_to_seq(1)
    pt, _ = pt.assign_seq_id_to_seq(0)
    pt, info = pt.allocate_for_seq(packed.slot_ids, packed.pos_ids)
    lens = {int(s): int(l) for s, l in zip(info.slot_ids[:2], info.seq_lens[:2])}
    boundary = [packed.pos_ids[i] == lens[int(packed.slot_ids[i])] - 1 for i in range(6)]
    assert boundary == [False, False, True, False, False, True]


def test_is_stop_signal():
    stops = np.array([[INVALID, 5, 6], [7, 8, 9]])
    assert is_stop_signal(np.array([1, 5, 6]), stops)
    assert is_stop_signal(np.array([7, 8, 9]), stops)
    assert not is_stop_signal(np.array([5, 6, 1]), stops)
    assert not is_stop_signal(np.array([1, 2, 3]), np.zeros((0, 3), int))
    assert not is_stop_signal(np.array([1, 2, 3]), np.full((2, 3), INVALID))
    assert not is_stop_signal(np.array([INVALID, INVALID, 6]), np.array([[INVALID, 5, 6]]))


def test_purge_and_unique():
    assert purge(np.array([1, 2, 3, 4]), np.array([False, True, False, True])).tolist() == [1, 3, INVALID, INVALID]
    u, d = get_unique_in_order(np.array([5, 5, 2, 9, 2]), size=4)
    assert u.tolist() == [5, 2, 9, INVALID] and d.tolist() == [0, 0, 1, 2, 1]


def test_decode_state_update_tokens_stop_and_length():
    pt = PageTable.init(16, 3, 4, 4)
    ds = DecodeState.init(pt, pad_token_id=0, max_stop_seqs=2, max_stop_tokens=3, max_queued_tokens=8, enable_logprobs=True)
    ds = ds.assign_seq(0, np.array([1, 2, 3]), 3, seq_params=SeqDecodingParams(10, np.array([[7, 8]]), 0.0, 1))
    ds = ds.assign_seq(1, np.array([4]), 1, seq_params=SeqDecodingParams(3, None, 0.5, 2))
    assert ds.stop_tokens[0, 0].tolist() == [INVALID, 7, 8]
    ds = ds.update_tokens(np.array([7, 5]), np.array([0, 1]), np.array([-0.1, -0.2], np.float32), 2)
    assert ds.seq_lens[:2].tolist() == [4, 2] and not ds.finished.any() and ds.num_queued_tokens == 2
    assert ds.tqueue.queued_pos_ids[:2].tolist() == [3, 1]
    ds = ds.update_tokens(np.array([8, 6]), np.array([0, 1]), np.array([-0.3, -0.4], np.float32), 2)
    assert ds.finished[:2].tolist() == [True, True]  # slot 0 hit its stop sequence, slot 1 its length limit
    assert ds.num_queued_tokens == 2  # finished sequences are not fed back
    assert ds.tokens[0, :5].tolist() == [1, 2, 3, 7, 8] and np.isnan(ds.logprobs[0, 2]) and abs(ds.logprobs[0, 4] + 0.3) < 1e-6
    a = ds.prng_keys_for(np.array([0, 0, 1]), np.array([3, 4, 3]))
    assert len(set(a.tolist())) == 3 and (a == ds.prng_keys_for(np.array([0, 0, 1]), np.array([3, 4, 3]))).all()
    ds = ds.invalidate_finished()
    assert ds.seq_lens[0] == INVALID and not ds.finished.any()


def test_outside_references_keep_pages_alive_and_lengths_round_up_to_a_page(backend):
    pt = _make_table(pages=8, seqs=4, page_size=4, pages_per_seq=3)
    assert pt.current_num_seqs == 0
    pt, a = pt.assign_seq_id_to_seq()
    pt, b = pt.assign_seq_id_to_seq()
    assert pt.current_num_seqs == 2 and (a, b) == (0, 1)
    pt, _ = pt.allocate_for_seq(np.zeros(6, np.int32), np.arange(6, dtype=np.int32))
    pages = pt.page_indices[0, :2].copy()
    held = pt.increment_ref_counts_for_pages(pages)  # e.g. a prefix cache that keeps the pages after the sequence is gone
    assert held.page_ref_counts[pages].tolist() == [2, 2] and pt.page_ref_counts[pages].tolist() == [1, 1]  # tables are values
    freed = held.free_pages(0)
    assert freed.page_ref_counts[pages].tolist() == [1, 1] and freed.num_free_pages == 8 - 2 and freed.current_num_seqs == 1
    assert pt.free_pages(0).num_free_pages == 8
    assert held.increment_ref_counts_for_pages([INVALID, int(pages[0])], count=2).page_ref_counts[pages].tolist() == [4, 2]  # holes are skipped
    # 6 tokens on pages of 4: rounding up makes the next token start a fresh page
    bumped = pt.bump_seq_len_to_next_page(0)
    assert bumped.seq_lens[0] == 8 and pt.seq_lens[0] == 6
    assert bumped.bump_seq_len_to_next_page(0).seq_lens[0] == 8  # already on a boundary
    grown, info = bumped.allocate_for_seq(np.zeros(1, np.int32), np.array([8], np.int32))
    assert grown.seq_lens[0] == 9 and is_valid_page(grown.page_indices[0, 2]) and grown.page_indices[0, 2] not in pages.tolist()


def is_valid_page(p) -> bool:
    return int(p) != INVALID and int(p) >= 0


def test_relative_positions_restart_with_every_run_of_equal_ids():
    assert PT._relative_positions(np.array([3, 3, 3, 1, 1, 3, 0, 0, 0, 0])).tolist() == [0, 1, 2, 0, 1, 0, 0, 1, 2, 3]
    assert PT._relative_positions(np.array([7])).tolist() == [0]


def test_decode_output_buffer_keeps_what_fits_and_accumulates_finished_flags():
    from levanter_b200.inference.jit_scheduler import _DecodeOutputs

    out = _DecodeOutputs.init(max_tokens=5, max_seqs=3, with_logprobs=True)
    assert out.max_queued_tokens == 5 and out.empty_queue_space == 5 and out.num_tokens == 0
    out = out.append(np.array([10, 11, 12, 99]), np.array([0, 1, 0, 2]), np.array([-0.1, -0.2, -0.3, -9.0]), 3, np.array([False, True, False]))
    assert out.num_tokens == 3 and out.tokens[:3].tolist() == [10, 11, 12] and out.tokens[3] == INVALID  # only the first three count
    out = out.append(np.array([13, 14, 15]), np.array([2, 2, 2]), None, 3, np.array([False, False, True]))  # room for two more
    assert out.num_tokens == 5 and out.empty_queue_space == 0 and out.tokens.tolist() == [10, 11, 12, 13, 14]
    assert out.slot_ids.tolist() == [0, 1, 0, 2, 2] and out.finished.tolist() == [False, True, True]
    assert out.logprobs[:3].tolist() == pytest.approx([-0.1, -0.2, -0.3]) and np.isnan(out.logprobs[3:]).all()
    assert _DecodeOutputs.init(4, 2, with_logprobs=False).append([1], [0], [-1.0], 1, [False, False]).logprobs is None


def test_queue_clearing_clone_discharge_and_finished_lookup():
    q = TokenQueue.init(6).enqueue_tokens(np.array([5, 6, 7]), np.array([0, 1, 0]), np.array([0, 0, 1]), 3)
    assert q.num_queued_tokens == 3
    empty = q.cleared()
    assert empty.num_queued_tokens == 0 and empty.max_queued_tokens == 6 and q.num_queued_tokens == 3
    st = DecodeState.init(_make_table(pages=8, seqs=4, page_size=2, pages_per_seq=2))
    st.clone_sources[:] = [INVALID, 0, 0, 1]
    st = st.discharge_clone(np.array([2, INVALID, 3]), 2)  # the first two entries only: slot 2 and a hole
    assert st.clone_sources.tolist() == [INVALID, 0, INVALID, 1]
    st.finished[:] = [True, False, False, True]
    assert st.is_finished(3).tolist() == [True] and st.is_finished(np.array([0, 1])).tolist() == [True, False]
