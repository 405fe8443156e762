"""Dataset combinators, stateless permutations and mixtures (levanter_b200/data/{dataset,_prp,permutation,mixture}.py; scenarios
after the reference's tests/test_newdataset.py, tests/test_prp.py, tests/test_mixture.py and tests/test_varying_mixture.py)."""
import asyncio

import numpy as np
import pytest

from levanter_b200.data._prp import FeistelPermutation, LcgPermutation, Permutation
from levanter_b200.data.dataset import EpochDataset, ListAsyncDataset
from levanter_b200.data.mixture import MixtureDataset, StopStrategy, rescale_mixture_schedule_for_batch_schedule
from levanter_b200.data.permutation import EraShufflingDataset, PermutationDataset
from levanter_b200.schedule import BatchSchedule, ScheduleStep

run = asyncio.run
KINDS = [LcgPermutation, FeistelPermutation]


# ---------------------------------------------------------------- permutations

@pytest.mark.parametrize("cls", KINDS)
def test_permutation_of_one_index_and_of_arrays(cls):
    p = cls(100, 0)
    assert p.length == 100
    one = p(5)
    assert isinstance(one, (int, np.integer)) and 0 <= one < 100
    idx = np.array([0, 1, 2, 3, 50, 99])
    img = p(idx)
    assert img.shape == idx.shape and ((img >= 0) & (img < 100)).all()
    assert img[4] == p(50) and p(idx.reshape(2, 3)).shape == (2, 3)


@pytest.mark.parametrize("cls", KINDS)
@pytest.mark.parametrize("n", [1, 2, 10, 97, 1000, 4096])
def test_permutation_is_a_bijection(cls, n):
    img = cls(n, 7)(np.arange(n))
    assert sorted(np.asarray(img).tolist()) == list(range(n))


@pytest.mark.parametrize("cls", KINDS)
def test_permutation_of_length_one(cls):
    p = cls(1, 0)
    assert p(0) == 0 and p(np.array([0])).tolist() == [0]


@pytest.mark.parametrize("cls", KINDS)
def test_permutation_rejects_indices_outside_the_range(cls):
    p = cls(10, 0)
    for bad in (-1, 10, np.array([0, 10]), np.array([-1, 3])):
        with pytest.raises(IndexError):
            p(bad)


@pytest.mark.parametrize("cls", KINDS)
def test_permutation_is_a_function_of_the_key(cls):
    idx = np.arange(50)
    a, b, c = cls(50, 12)(idx), cls(50, 12)(idx), cls(50, 13)(idx)
    assert (a == b).all() and not (a == c).all()
    assert (cls(50, np.array([0, 12], dtype=np.uint32))(idx) == cls(50, np.array([0, 12], dtype=np.uint32))(idx)).all()


@pytest.mark.parametrize("cls", KINDS)
def test_permutation_of_a_very_long_range_does_not_overflow(cls):
    n = 2 ** 34
    p = cls(n, 3)
    idx = np.array([0, 1, n // 2, n - 2, n - 1], dtype=np.int64)
    img = np.asarray(p(idx))
    assert ((img >= 0) & (img < n)).all() and len(set(img.tolist())) == 5
    assert 0 <= p(n - 1) < n


@pytest.mark.parametrize("cls", KINDS)
@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.uint32, np.uint64])
def test_permutation_takes_the_usual_index_types(cls, dtype):
    p = cls(100, 0)
    assert (np.asarray(p(np.arange(10, dtype=dtype))) == np.asarray(p(np.arange(10)))).all()


def test_permutation_factory():
    assert isinstance(Permutation.make("feistel", 10, 0), FeistelPermutation)
    assert isinstance(Permutation.make("linear", 10, 0), LcgPermutation)
    with pytest.raises(ValueError):
        Permutation.make("sorted", 10, 0)


# ---------------------------------------------------------------- list, permuted and era-shuffled datasets

def test_list_dataset_length_items_and_growth():
    ds = ListAsyncDataset([1, 2, 3], is_complete=True)
    assert run(ds.async_len()) == 3 and run(ds.getitem_async(1)) == 2 and run(ds.get_batch([2, 0])) == [3, 1]
    assert run(ds.final_length_is_known()) and ds.is_finite()

    growing = ListAsyncDataset()
    growing.append(4)
    growing.append(5)
    assert run(growing.current_len()) == 2 and not run(growing.final_length_is_known())
    growing.finalize()
    assert run(growing.async_len()) == 2 and run(growing.get_batch([0, 1])) == [4, 5]
    with pytest.raises(Exception):
        growing.append(6)


def test_a_reader_waits_for_rows_that_are_appended_later():
    ds = ListAsyncDataset()

    async def scenario():
        async def produce():
            for i in range(5):
                await asyncio.sleep(0.01)
                ds.append(i * i)
            ds.finalize()

        task = asyncio.create_task(produce())
        n = await asyncio.wait_for(ds.wait_until_len_at_least(3), 5)
        got = await asyncio.wait_for(ds.get_batch([4]), 5)
        await task
        return n, got, await ds.async_len()

    n, got, total = run(scenario())
    assert n >= 3 and got == [16] and total == 5


def test_permutation_dataset_permutes_and_keeps_every_item():
    ds = ListAsyncDataset(list(range(50)), is_complete=True)
    p = PermutationDataset(ds, key=1)
    got = run(p.get_batch(list(range(50))))
    assert got != list(range(50)) and sorted(got) == list(range(50)) and run(p.async_len()) == 50
    assert run(p.getitem_async(7)) == got[7]
    assert run(ds.shuffle(1).get_batch(list(range(50)))) == got
    assert run(PermutationDataset(ds, key=2).get_batch(list(range(50)))) != got


def test_era_shuffle_shuffles_inside_eras_only():
    ds = ListAsyncDataset(list(range(23)), is_complete=True)
    e = EraShufflingDataset(ds, 5, key=0)
    assert run(e.async_len()) == 23
    got = run(e.get_batch(list(range(23))))
    for era in range(5):
        lo, hi = era * 5, min(23, era * 5 + 5)
        assert sorted(got[lo:hi]) == list(range(lo, hi))
    assert got != list(range(23))
    assert run(ds.era_shuffle(5, key=0).get_batch(list(range(23)))) == got


def test_era_shuffle_over_a_dataset_that_still_grows():
    ds = ListAsyncDataset(list(range(7)))
    e = EraShufflingDataset(ds, 5, key=0)

    async def scenario():
        first = await asyncio.wait_for(e.get_batch(list(range(5))), 5)  # the first era is complete
        assert sorted(first) == list(range(5))
        with pytest.raises(asyncio.TimeoutError):
            await asyncio.wait_for(e.getitem_async(6), 0.1)  # the second era is not: its permutation is not fixed yet
        for i in range(7, 10):
            ds.append(i)
        second = await asyncio.wait_for(e.get_batch(list(range(5, 10))), 5)
        assert sorted(second) == list(range(5, 10))
        ds.append(10)
        ds.finalize()
        assert await asyncio.wait_for(e.getitem_async(10), 5) == 10 and await e.async_len() == 11

    run(scenario())


def test_epochs_repeat_the_dataset():
    ds = ListAsyncDataset([1, 2, 3], is_complete=True)
    assert run(EpochDataset(ds).get_batch([0, 3, 7])) == [1, 1, 2] and not EpochDataset(ds).is_finite()
    two = EpochDataset(ds, max_epochs=2)
    assert run(two.async_len()) == 6 and two.is_finite()


# ---------------------------------------------------------------- mixtures

def _datasets():
    return {"ds1": ListAsyncDataset([1, 2, 3, 4, 5], is_complete=True), "ds2": ListAsyncDataset([10, 20, 30, 40, 50], is_complete=True),
            "ds3": ListAsyncDataset([100, 200, 300, 400, 500], is_complete=True)}


W = {"ds1": 0.5, "ds2": 0.3, "ds3": 0.2}


def test_mixture_in_source_order_when_blocks_are_not_randomized():
    m = MixtureDataset(_datasets(), W, 10, key=42, randomize_blocks=False)
    assert run(m.getitem_async(0)) == 1
    assert run(m.get_batch(list(range(10)))) == [1, 2, 3, 4, 5, 10, 20, 30, 100, 200]
    # the second block continues every source where the first left it (and wraps the short ones)
    assert run(m.get_batch(list(range(10, 20)))) == [1, 2, 3, 4, 5, 40, 50, 10, 300, 400]


def test_mixture_length_is_not_defined_for_the_restart_strategy():
    m = MixtureDataset(_datasets(), W, 10, key=42, stop_strategy=StopStrategy.RESTART_STRATEGY)
    with pytest.raises(ValueError):
        run(m.async_len())
    assert not m.is_finite()
    with pytest.raises(ValueError):
        MixtureDataset(_datasets(), W, 10, key=42, stop_strategy="whenever")


def test_mixture_over_sliced_sources_repeats_their_few_items():
    third = {k: 1 / 3 for k in W}
    for n, allowed in ((1, {1, 10, 100}), (2, {1, 2, 10, 20, 100, 200})):
        m = MixtureDataset({k: d.slice_dataset(end_index=n) for k, d in _datasets().items()}, third, 10, key=42, randomize_blocks=False)
        for _ in range(3):
            got = run(m.get_batch([0, 1, 2, 25, 77]))
            assert len(got) == 5 and set(got) <= allowed


def test_mixture_weights_are_normalised_and_zero_means_never():
    m = MixtureDataset(_datasets(), {"ds1": 0, "ds2": 2.0, "ds3": 2.0}, 10, key=42)
    got = run(m.get_batch(list(range(200))))
    assert all(x >= 10 for x in got) and sum(x >= 100 for x in got) == 100


def test_mixture_remaps_indices_past_the_end_of_a_source():
    d = _datasets()
    m = MixtureDataset(d, W, 10, key=42)
    assert list(run(m._remap_indices(d["ds1"], [0, 1, 2]))) == [0, 1, 2]
    assert list(run(m._remap_indices(d["ds1"], [4, 5, 6]))) == [4, 0, 1]


def test_mixture_follows_the_weights_and_reaches_every_item():
    m = MixtureDataset(_datasets(), W, 10, key=42)
    got = run(m.get_batch(list(range(1000))))
    share = {"ds1": sum(x < 10 for x in got) / 1000, "ds2": sum(10 <= x < 100 for x in got) / 1000, "ds3": sum(x >= 100 for x in got) / 1000}
    for k in W:
        assert abs(share[k] - W[k]) < 0.01
    assert set(got) == {1, 2, 3, 4, 5, 10, 20, 30, 40, 50, 100, 200, 300, 400, 500}


def test_mixture_blocks_are_shuffled_differently_but_reproducibly():
    m = MixtureDataset(_datasets(), W, 10, key=42)
    a, a2, b = m._block_assignments(0), m._block_assignments(0), m._block_assignments(1)
    assert len(a) == 10 and (a == a2).all() and not (a == b).all()
    assert sorted((a >> 32).tolist()) == [0] * 5 + [1] * 3 + [2] * 2
    other = MixtureDataset(_datasets(), W, 10, key=43)
    assert not all((other._block_assignments(i) == m._block_assignments(i)).all() for i in range(4))


def test_mixture_schedule_in_steps_becomes_a_schedule_in_sequences():
    stages = [(0, {"ds1": 0.5, "ds2": 0.5}), (10, {"ds1": 0.2, "ds2": 0.8})]
    sched = BatchSchedule([ScheduleStep(start=0, value=10), ScheduleStep(start=5, value=20)])
    assert rescale_mixture_schedule_for_batch_schedule(stages, sched) == [(0, stages[0][1]), (150, stages[1][1])]
    sched = BatchSchedule([ScheduleStep(start=0, value=10), ScheduleStep(start=10, value=20)])
    assert rescale_mixture_schedule_for_batch_schedule(stages, sched) == [(0, stages[0][1]), (100, stages[1][1])]


def test_mixture_stages_change_the_proportions_gradually():
    big = {"ds1": ListAsyncDataset(list(range(1000)), is_complete=True), "ds2": ListAsyncDataset(list(range(10000, 11000)), is_complete=True)}
    stages = [(0, {"ds1": 0.8, "ds2": 0.2}), (20, {"ds1": 0.5, "ds2": 0.5}), (40, {"ds1": 0.2, "ds2": 0.8})]
    m = MixtureDataset(big, stages, 10, key=0)
    got = run(m.get_batch(list(range(60))))
    shares = [sum(x < 10000 for x in got[i:i + 20]) / 20 for i in (0, 20, 40)]
    assert shares == [0.8, 0.5, 0.2]
    # no item of a source is read twice across the stage changes
    firsts = [x for x in got if x < 10000]
    assert sorted(firsts) == list(range(len(firsts)))
    # a block never straddles two stages
    for blk in range(6):
        chunk = got[blk * 10:blk * 10 + 10]
        assert sum(x < 10000 for x in chunk) == [8, 8, 5, 5, 2, 2][blk]


def test_mixture_stage_lists_are_checked():
    d = _datasets()
    with pytest.raises(ValueError):
        MixtureDataset(d, [(10, W)], 10, key=0)  # does not start at 0
    with pytest.raises(ValueError):
        MixtureDataset(d, [(0, W), (20, W), (10, W)], 10, key=0)  # not increasing
    with pytest.raises(ValueError):
        MixtureDataset(d, [(0, W), (15, W)], 10, key=0)  # not a block boundary
    with pytest.raises(ValueError):
        MixtureDataset(d, {"ds1": 0.5, "nope": 0.5}, 10, key=0)
    with pytest.raises(ValueError):
        MixtureDataset(d, {"ds1": 0.0, "ds2": 0.0, "ds3": 0.0}, 10, key=0)
