"""Stand-alone gradient accumulation, shape specifications, process / tensor helpers, and small helpers of the inference engine
(levanter_b200/grad_accum.py, shapes.py, utils/torch_utils.py, inference/utils.py, inference/jit_scheduler.py)."""
import numpy as np
import pytest
import torch

from levanter_b200.grad_accum import ReductionType, microbatch_slices, microbatched
from levanter_b200.inference.jit_scheduler import DecodeState, SeqDecodingParams
from levanter_b200.inference.utils import INVALID, get_unique_in_order, is_invalid, is_valid, masked_set, pad_to_standard_length, purge
from levanter_b200.shapes import NamedShapeSpec, ShapeSpec, conforms, shape_spec_of, to_raw_shape
from levanter_b200.utils import torch_utils as TU


def test_microbatched_gradients_equal_the_full_batch():
    torch.manual_seed(0)
    model = torch.nn.Linear(6, 3)
    x, y = torch.randn(8, 6), torch.randn(8, 3)

    def loss_and_grads(batch):
        model.zero_grad()
        loss = ((model(batch["x"]) - batch["y"]) ** 2).mean()
        loss.backward()
        return loss, {n: p.grad.clone() for n, p in model.named_parameters()}

    full_loss, full = loss_and_grads({"x": x, "y": y})
    for mb in (2, 4, 8, None, 100):
        loss, grads = microbatched(loss_and_grads, mb)({"x": x, "y": y})
        assert float(loss) == pytest.approx(float(full_loss.detach()), rel=1e-6)
        for n in full:
            assert torch.allclose(grads[n], full[n], atol=1e-6) and grads[n].dtype == torch.float32
    total_loss, total = microbatched(loss_and_grads, 2, reduce=ReductionType.SUM)({"x": x, "y": y})
    assert float(total_loss) == pytest.approx(4 * float(full_loss.detach()), rel=1e-5)
    assert torch.allclose(total["weight"], 4 * full["weight"], atol=1e-5)
    with pytest.raises(ValueError):
        microbatched(loss_and_grads, 3)({"x": x, "y": y})
    assert microbatch_slices(8, 4) == [(0, 4), (4, 8)] and microbatch_slices(8, None) == [(0, 8)] and microbatch_slices(8, 16) == [(0, 8)]
    # tuples, lists and extra arguments pass through
    seen = []

    def fn(batch, scale, *, tag):
        seen.append((batch[0].shape[0], batch[1][0].shape[0], scale, tag))
        return torch.tensor(1.0), {"g": torch.ones(1), "none": None}

    loss, grads = microbatched(fn, 2)((x, [y]), 3.0, tag="t")
    assert seen == [(2, 2, 3.0, "t")] * 4 and float(loss) == 1.0 and set(grads) == {"g"}


def test_shape_specifications():
    spec = ShapeSpec((None, 16), torch.int32)
    named = NamedShapeSpec((("batch", None), ("position", 16)), torch.int32)
    assert to_raw_shape(spec) == (None, 16) == to_raw_shape(named) and named.names == ("batch", "position")
    assert conforms(spec, torch.zeros(4, 16)) and conforms(named, np.zeros((9, 16))) and not conforms(spec, torch.zeros(4, 8))
    assert not conforms(spec, torch.zeros(16)) and conforms(ShapeSpec(None, None), "anything at all")
    assert shape_spec_of(torch.zeros(2, 3, dtype=torch.bfloat16)) == ShapeSpec((2, 3), torch.bfloat16)
    assert shape_spec_of([[1, 2], [3, 4]]).shape == (2, 2)


def test_tensor_and_process_helpers_on_one_process():
    assert TU.to_python(torch.tensor(3)) == 3 and TU.to_python(torch.tensor([1.5, 2.5])) == [1.5, 2.5] and TU.to_python("x") == "x"
    with TU.use_cpu_device():
        assert torch.zeros(1).device.type == "cpu"
    shared = torch.nn.Parameter(torch.zeros(5))
    m = torch.nn.Module()
    m.a, m.b = shared, shared
    m.c = torch.nn.Parameter(torch.zeros(2), requires_grad=False)
    assert TU.parameter_count(m) == 7 and TU.parameter_count(m, need_grad_only=True) == 5
    assert TU.parameter_count({"x": torch.zeros(3), "y": {"z": torch.zeros(2, 2)}}) == 7
    assert TU.multihost_broadcast_sync({"k": 1}) == {"k": 1}
    tree = {"a": torch.arange(4), "b": [torch.ones(2), (torch.zeros(1),)], "n": 3}
    assert TU.broadcast_shard(tree) is tree  # one process: nothing to send
    leaves, _ = TU._flatten_tensors(tree)
    rebuilt = TU._rebuild(TU._structure_of(tree), leaves)
    assert rebuilt["n"] == 3 and torch.equal(rebuilt["b"][1][0], torch.zeros(1)) and isinstance(rebuilt["b"][1], tuple)
    keys = TU.key_iterator(7)
    first = [next(keys) for _ in range(3)]
    again = TU.key_iterator(7)
    assert first == [next(again) for _ in range(3)] and len(set(first)) == 3
    assert TU.is_inexact_arrayish(torch.zeros(1)) and not TU.is_inexact_arrayish(torch.zeros(1, dtype=torch.int32)) and not TU.is_inexact_arrayish(1.0)
    free = TU.estimated_free_device_memory()
    assert free is None or free > 0
    z = TU.zeros_like_tree({"a": torch.ones(2), "b": None}, dtype=torch.float64) if hasattr(TU, "zeros_like_tree") else None
    assert z is None or (z["a"].dtype == torch.float64 and float(z["a"].sum()) == 0)


def test_inference_index_helpers():
    x = np.array([0, 5, -1, INVALID])
    assert is_invalid(x).tolist() == [False, False, True, True] and is_valid(x).tolist() == [True, True, False, False]
    dest = np.zeros((2, 5), dtype=np.int32)
    masked_set(dest, 1, 3, np.array([[1, 2, 3], [4, 5, 6]]), 3)  # clipped to the destination
    assert dest.tolist() == [[0, 0, 0, 1, 2], [0, 0, 0, 4, 5]]
    assert masked_set(dest.copy(), 1, 9, np.ones((2, 2), dtype=np.int32), 2).tolist() == dest.tolist()  # starts past the end: nothing copied
    assert purge(np.array([1, 2, 3, 4]), np.array([False, True, False, True])).tolist() == [1, 3, INVALID, INVALID]
    with pytest.raises(ValueError):
        purge(np.zeros((2, 2)), np.zeros((2, 2), dtype=bool))
    assert pad_to_standard_length(np.array([1, 2, 3]), [2, 4, 8], 0).tolist() == [1, 2, 3, 0]
    assert pad_to_standard_length(np.array([1, 2]), [2, 4], 0).tolist() == [1, 2]
    with pytest.raises(ValueError):
        pad_to_standard_length(np.arange(9), [2, 4, 8], 0)
    uniq, inverse = get_unique_in_order(np.array([7, 3, 7, 9, 3]), size=4)
    assert uniq.tolist() == [7, 3, 9, INVALID] and inverse.tolist() == [0, 1, 0, 2, 1]


def test_per_sequence_sampling_seeds_and_default_decoding_parameters():
    d = SeqDecodingParams.default()
    assert d.temperature == 0.0 and d.stop_tokens is None and d.max_num_tokens > 2 ** 30
    from levanter_b200.inference.page_table import PageTable

    table = PageTable.init(max_pages=8, max_seqs=4, page_size=4, max_pages_per_seq=4)
    state = DecodeState.init(table, pad_token_id=0, max_stop_seqs=2, max_stop_tokens=3, max_queued_tokens=8)
    state.prng_keys[:] = np.array([11, 22, 33, 44])
    a = state.prng_key_for(1, 5)
    assert a == state.prng_key_for(1, 5) and a != state.prng_key_for(1, 6) and a != state.prng_key_for(2, 5) and 0 <= a < 2 ** 63
    many = state.prng_keys_for(np.array([0, 1, 2, 3]), np.array([5, 5, 5, 5]))
    assert many[1] == a and len(set(many.tolist())) == 4
    assert state.max_queued_tokens == 8 and state.empty_queue_space == 8 and state.num_queued_tokens == 0 and state.max_stop_seq_len == 3
    state = state.enqueue_tokens(np.array([9, 8]), np.array([1, 0]), np.array([0, 0]), 2)
    assert state.num_queued_tokens == 2 and state.empty_queue_space == 6
    state, packed = state.pack_next_sequence(4)
    assert packed.num_tokens == 2 and packed.slot_ids[:2].tolist() == [0, 1] and packed.tokens[:2].tolist() == [8, 9]  # sorted by slot
    assert packed.token_counts_per_slot(4).tolist() == [1, 1, 0, 0]
