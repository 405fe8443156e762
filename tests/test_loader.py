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
