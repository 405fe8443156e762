"""Data loader: which rows a rank loads for every mesh position, batch-size schedules, resume by step, padding of a short last
batch, error propagation from the producer thread (modelled on the reference's tests/test_new_loader.py)."""
import pytest
import torch

from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.data.loader import DataLoader
from levanter_b200.parallel.mesh import DeviceMesh
from levanter_b200.schedule import BatchSchedule, ScheduleStep


def _ds(n):
    return ListAsyncDataset([torch.tensor([i, 10 * i]) for i in range(n)], is_complete=True)


def _mesh(replica, data, model, rank):
    return DeviceMesh(replica, data, model, world_size=replica * data * model, rank=rank, create_groups=False)


@pytest.mark.parametrize("replica,data,model", [(1, 4, 1), (1, 2, 2), (2, 2, 1), (2, 1, 2)])
def test_every_data_shard_loads_its_rows_and_model_ranks_share_them(replica, data, model):
    world = replica * data * model
    seen = {}
    for rank in range(world):
        mesh = _mesh(replica, data, model, rank)
        dl = DataLoader(_ds(64), 8, mesh=mesh, max_buffered_batches=0, pin_memory=False)
        rows, pad = dl.local_indices_at_step(3)
        assert pad == 0
        seen.setdefault(mesh.batch_index, []).append(rows)
    shards = replica * data
    assert sorted(seen) == list(range(shards))
    for idx, lists in seen.items():
        assert len(lists) == model and all(l == lists[0] for l in lists)  # ranks along the model axis load the same rows
    union = sorted(i for lists in seen.values() for i in lists[0])
    assert union == list(range(24, 32))  # batch 3 of size 8, each row exactly once


def test_batch_schedule_and_resume_by_step():
    sched = BatchSchedule([ScheduleStep(0, 4), ScheduleStep(3, 8)])
    dl = DataLoader(_ds(100), sched, max_buffered_batches=0, pin_memory=False)
    it = iter(dl)
    sizes = [next(it).shape[0] for _ in range(5)]
    assert sizes == [4, 4, 4, 8, 8]
    resumed = dl.iter_from_step(4)
    b = next(resumed)
    assert b[:, 0].tolist() == list(range(20, 28))  # 3 * 4 + 8 rows precede step 4


def test_short_last_batch_is_padded_and_then_the_loader_stops():
    dl = DataLoader(_ds(10), 4, max_buffered_batches=0, pin_memory=False)
    batches = list(dl)
    assert [b.shape[0] for b in batches] == [4, 4, 4]
    assert batches[2][:2, 0].tolist() == [8, 9] and batches[2][2:].abs().sum() == 0


def test_nondivisible_batch_size_needs_the_flag():
    mesh = _mesh(1, 4, 1, 0)
    with pytest.raises(ValueError):
        DataLoader(_ds(64), 6, mesh=mesh, pin_memory=False)
    dl = DataLoader(_ds(64), 6, mesh=mesh, allow_nondivisible_batch_size=True, max_buffered_batches=0, pin_memory=False)
    rows, pad = dl.local_indices_at_step(0)
    assert rows == [0, 1] and pad == 0
    rows3, pad3 = DataLoader(_ds(64), 6, mesh=_mesh(1, 4, 1, 3), allow_nondivisible_batch_size=True, max_buffered_batches=0,
                             pin_memory=False).local_indices_at_step(0)
    assert rows3 == [] and pad3 == 2  # 6 rows over 4 shards of 2: the last shard is all padding


def test_background_prefetch_gives_the_same_batches_and_surfaces_errors():
    a = [b[:, 0].tolist() for b in DataLoader(_ds(40), 8, max_buffered_batches=0, pin_memory=False)]
    b = [b[:, 0].tolist() for b in DataLoader(_ds(40), 8, max_buffered_batches=4, prefetch_size=2, pin_memory=False)]
    assert a == b and len(a) == 5

    class Broken(ListAsyncDataset):
        async def get_batch(self, indices):
            if any(i >= 16 for i in indices):
                raise RuntimeError("shard went away")
            return await super().get_batch(indices)

    dl = DataLoader(Broken([torch.tensor([i]) for i in range(40)], is_complete=True), 8, max_buffered_batches=4, pin_memory=False)
    it = iter(dl)
    with pytest.raises(RuntimeError, match="shard went away"):  # batches are fetched ahead in groups, so it may surface early
        for _ in range(3):
            next(it)


# ---------------------------------------------------------------- more scenarios after the reference's tests/test_new_loader.py
SCHEDULE = [ScheduleStep(start=0, value=8), ScheduleStep(start=10, value=16), ScheduleStep(start=20, value=32)]


def _token_rows(n, seq_len=16):
    return ListAsyncDataset([torch.full((seq_len,), i + 1, dtype=torch.int32) for i in range(n)], is_complete=True)


@pytest.mark.parametrize("model_axis", [1, 2])
def test_batch_size_schedule_without_padding_drops_the_short_last_batch(model_axis):
    mesh = _mesh(1, 2, model_axis, 0)
    dl = DataLoader(_token_rows(1000), BatchSchedule(SCHEDULE), mesh=mesh, max_buffered_batches=10, pad_final_batch=False, pin_memory=False)
    sizes = [b.shape[0] for b in dl]
    # this rank loads half of every batch; 10 * 8 + 10 * 16 = 240 rows in the first 20 steps, (1000 - 240) // 32 = 23 whole batches after
    assert sizes == [4] * 10 + [8] * 10 + [16] * 23


@pytest.mark.parametrize("model_axis", [1, 2])
def test_batch_size_schedule_with_a_padded_last_batch(model_axis):
    world = 2 * model_axis
    last = []
    for rank in range(world):
        mesh = _mesh(1, 2, model_axis, rank)
        dl = DataLoader(_token_rows(1007), BatchSchedule(SCHEDULE), mesh=mesh, max_buffered_batches=10, pad_final_batch=True, pin_memory=False)
        batches = list(dl)
        assert [b.shape[0] for b in batches] == [4] * 10 + [8] * 10 + [16] * 24
        last.append((mesh.batch_index, batches[-1]))
    # the 24th large batch holds the last (1007 - 240) % 32 = 31 rows and one row of zeros, at the end of the last shard
    by_shard = dict(last)
    whole = torch.cat([by_shard[0], by_shard[1]])
    assert whole.shape[0] == 32 and (whole[:31, 0] == torch.arange(1007 - 30, 1008)).all() and whole[31].abs().sum() == 0


def test_examples_that_are_trees_are_stacked_leaf_by_leaf():
    def example(i):
        image = torch.arange(16 * 16, dtype=torch.int32).reshape(16, 16) + i * 1000
        return {"input_ids": image, "labels": image.clone(), "extra": {"input_ids": image.clone(), "mask": torch.arange(16) + i * 1000}}

    ds = ListAsyncDataset([example(i) for i in range(40)], is_complete=True)
    per_rank = {}
    for rank in range(4):
        mesh = _mesh(1, 4, 1, rank)
        batches = list(DataLoader(ds, 8, mesh=mesh, max_buffered_batches=0, pin_memory=False))
        assert len(batches) == 5
        per_rank[rank] = batches
        for b in batches:
            assert b["input_ids"].shape == (2, 16, 16) and b["extra"]["mask"].shape == (2, 16)
            assert torch.equal(b["input_ids"], b["labels"]) and torch.equal(b["input_ids"], b["extra"]["input_ids"])
            assert torch.equal(b["extra"]["mask"][:, 0], b["input_ids"][:, 0, 0])  # leaves of one example stay together
    # ranks hold different rows of a batch, and together every row once
    step2 = torch.cat([per_rank[r][2]["input_ids"][:, 0, 0] for r in range(4)])
    assert sorted((step2 // 1000).tolist()) == list(range(16, 24))


def test_a_dataclass_example_keeps_its_type():
    from levanter_b200.models.lm_model import LmExample

    ds = ListAsyncDataset([LmExample.causal(torch.full((8,), i, dtype=torch.int32)) for i in range(12)], is_complete=True)
    (first, *_rest) = list(DataLoader(ds, 4, max_buffered_batches=0, pin_memory=False))
    assert isinstance(first, LmExample) and first.tokens.shape == (4, 8) and first.loss_mask.shape == (4, 8)
    assert first.tokens[:, 0].tolist() == [0, 1, 2, 3] and first.attn_mask.is_causal
