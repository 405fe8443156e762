"""The jagged-array store, the tree store and the cache builder (levanter_b200/store/; scenarios after the reference's
tests/test_jagged_array.py, tests/test_tree_store.py and tests/test_new_cache.py)."""
import asyncio
import threading
from typing import Iterator, Sequence

import numpy as np
import pytest

from levanter_b200.data._preprocessor import BatchProcessor
from levanter_b200.data.sharded_datasource import ShardedDataSource, UrlDataSource
from levanter_b200.store.cache import CacheOptions, SerialCacheWriter, TreeCache, build_or_load_cache
from levanter_b200.store.jagged_array import JaggedArrayStore, PreparedBatch
from levanter_b200.store.tree_store import TreeStore


# ---------------------------------------------------------------- jagged arrays

@pytest.mark.parametrize("cache_metadata", [True, False])
def test_append_and_get(tmp_path, cache_metadata):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=1, dtype=np.float32, cache_metadata=cache_metadata)
    d1, d2 = np.array([1.0, 2.0, 3.0], np.float32), np.array([4.0, 5.0], np.float32)
    b.append(d1)
    b.append(d2)
    assert len(b) == 2 and b.data_size == 5
    np.testing.assert_array_equal(b[0], d1)
    np.testing.assert_array_equal(b[1], d2)
    np.testing.assert_array_equal(b[-1], d2)
    r = JaggedArrayStore.open(str(tmp_path), mode="r", item_rank=1, dtype=np.float32, cache_metadata=cache_metadata)
    np.testing.assert_array_equal(r[1], d2)
    a, c = r[0:2]
    np.testing.assert_array_equal(a, d1)
    np.testing.assert_array_equal(c, d2)


def test_extend_with_many_rows_and_with_a_prepared_batch(tmp_path):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=1, dtype=np.int64)
    rows = [np.arange(n, dtype=np.int64) + 10 * n for n in (3, 1, 4, 1, 5)]
    b.extend(rows[:2])
    prepared = PreparedBatch.from_batch(rows[2:])
    assert prepared.num_rows == 3 and prepared.offsets.tolist() == [4, 5, 10] and prepared.shapes is None
    b.extend(prepared)
    assert len(b) == 5
    for got, want in zip(list(b), rows):
        np.testing.assert_array_equal(got, want)

    async def more():
        await b.extend_async(PreparedBatch.from_batch(rows[:1]))
        await b.append_async(rows[4])
        return await b.get_item_async(6), await b.num_rows_async(), await b.data_size_async()

    last, n, size = asyncio.run(more())
    np.testing.assert_array_equal(last, rows[4])
    assert n == 7 and size == sum(len(r) for r in rows) + 3 + 5


def test_prepared_batches_concatenate():
    a = PreparedBatch.from_batch([np.ones((2, 3)), np.ones((1, 3))])
    b = PreparedBatch.from_batch([np.zeros((4, 3))])
    c = PreparedBatch.concat([a, b])
    assert c.offsets.tolist() == [6, 9, 21] and c.shapes.tolist() == [[2], [1], [4]] and c.data.shape == (21,)
    assert c.astype(np.float32).data.dtype == np.float32 and c.byte_size() == 21 * 8


def test_a_row_of_the_wrong_rank_is_refused(tmp_path):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=1, dtype=np.float32)
    with pytest.raises(ValueError, match="rank"):
        b.append(np.array([[1.0, 2.0]], np.float32))


@pytest.mark.parametrize("cache_metadata", [True, False])
def test_rows_of_rank_two_keep_their_shapes(tmp_path, cache_metadata):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=2, dtype=np.float32)
    d1 = np.array([[1.0, 2.0], [3.0, 4.0]], np.float32)
    d2 = np.array([[5.0], [6.0], [7.0]], np.float32)
    b.append(d1)
    b.extend([d2, d1.T.copy()])
    r = JaggedArrayStore.open(str(tmp_path), mode="r", item_rank=2, dtype=np.float32, cache_metadata=cache_metadata)
    assert len(r) == 3
    np.testing.assert_array_equal(r[0], d1)
    np.testing.assert_array_equal(r[1], d2)
    assert r[1].shape == (3, 1)
    got = asyncio.run(r.get_batch([2, 0]))
    np.testing.assert_array_equal(got[0], d1.T)
    np.testing.assert_array_equal(got[1], d1)


def test_out_of_range_rows_raise(tmp_path):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=1, dtype=np.int32)
    b.append(np.array([1, 2], np.int32))
    with pytest.raises(IndexError):
        b[2]
    with pytest.raises(IndexError):
        b[-2]
    with pytest.raises(IndexError):
        b.get_batch_sync([0, 5])


def test_slices_with_steps(tmp_path):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=1, dtype=np.int32)
    rows = [np.full(i + 1, i, np.int32) for i in range(10)]
    b.extend(rows)
    assert [r[0] for r in b[::3]] == [0, 3, 6, 9]
    assert [r[0] for r in b[8:2:-2]] == [8, 6, 4]
    assert b[4:4] == [] and [len(r) for r in b[7:]] == [8, 9, 10]


def test_trim_to_size(tmp_path):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=1, dtype=np.int64)
    rows = [np.arange(i + 2, dtype=np.int64) for i in range(10)]
    b.extend(rows)
    asyncio.run(b.trim_to_size_async(5))
    assert len(b) == 5 and b.data_size == sum(len(r) for r in rows[:5])
    np.testing.assert_array_equal(b[4], rows[4])
    with pytest.raises(IndexError):
        b[5]
    b.trim_to_size(20)  # larger than the store: nothing happens
    assert len(b) == 5
    # appends continue where the trim left the store, for a fresh reader too
    b.append(np.array([7, 7, 7], np.int64))
    r = JaggedArrayStore.open(str(tmp_path), mode="r", item_rank=1, dtype=np.int64)
    assert len(r) == 6 and r[5].tolist() == [7, 7, 7] and r.data_size == b.data_size
    b.trim_to_size(0)
    assert len(b) == 0 and b.data_size == 0 and list(b) == []


@pytest.mark.parametrize("cache_metadata", [True, False])
def test_trim_to_size_with_shapes(tmp_path, cache_metadata):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=2, dtype=np.int64, cache_metadata=cache_metadata)
    rows = [np.arange((i + 1) * 3, dtype=np.int64).reshape(i + 1, 3) for i in range(6)]
    b.extend(rows)
    b.trim_to_size(2)
    assert len(b) == 2 and b.shapes.shape[0] == 2
    b.append(rows[5])
    np.testing.assert_array_equal(b[2], rows[5])
    np.testing.assert_array_equal(b[1], rows[1])


def test_get_batch_forms(tmp_path):
    b = JaggedArrayStore.open(str(tmp_path), item_rank=1, dtype=np.int64)
    rng = np.random.default_rng(0)
    rows = [rng.integers(0, 100, size=rng.integers(1, 9)) for _ in range(50)]
    b.extend(rows)
    assert asyncio.run(b.get_batch([])) == []
    (one,) = asyncio.run(b.get_batch([17]))
    np.testing.assert_array_equal(one, rows[17])
    idx = [40, 3, 41, 3, 0, 49, 25]  # out of order, repeated, far apart
    for got, i in zip(asyncio.run(b.get_batch(idx)), idx):
        np.testing.assert_array_equal(got, rows[i])


# ---------------------------------------------------------------- tree stores

class _PairProcessor(BatchProcessor):
    """Raw rows are lists of ints; the output has two leaves."""

    def __call__(self, batch):
        return [{"data": np.asarray(x, np.int64), "length": np.array([len(x)], np.int64)} for x in batch]

    @property
    def output_exemplar(self):
        return {"data": np.zeros(0, np.int64), "length": np.zeros(0, np.int64)}

    @property
    def metadata(self):
        return {"kind": "pair"}

    @property
    def num_cpus(self):
        return 1


def test_tree_store_from_a_processor(tmp_path):
    proc = _PairProcessor()
    t = TreeStore.open(proc.output_exemplar, str(tmp_path), mode="w")
    t.extend(proc([[1, 2, 3], [4, 5, 6, 7]]))
    t.extend(proc([[8]]))
    assert len(t) == 3
    assert t[1]["data"].tolist() == [4, 5, 6, 7] and t[1]["length"].tolist() == [4]
    assert t[-1]["data"].tolist() == [8]


def test_tree_store_rows_of_different_shapes_and_nested_leaves(tmp_path):
    ex = {"a": np.zeros((0, 2), np.float64), "n": {"b": np.zeros(0, np.float32)}}
    t = TreeStore.open(ex, str(tmp_path), mode="w")
    batch = [{"a": np.ones((2, 2)), "n": {"b": np.array([3.0], np.float32)}}, {"a": np.full((3, 2), 5.0), "n": {"b": np.array([7.0, 8.0], np.float32)}}]
    t.append(batch[0])
    t.extend(batch[1:])
    assert len(t) == 2
    assert t[1]["a"].shape == (3, 2) and (t[1]["a"] == 5).all() and t[1]["n"]["b"].tolist() == [7.0, 8.0]
    assert t[0]["n"]["b"].dtype == np.float32
    got = t[0:2]
    assert [g["a"].shape for g in got] == [(2, 2), (3, 2)]
    assert [g["n"]["b"].tolist() for g in t] == [[3.0], [7.0, 8.0]]
    with pytest.raises(IndexError):
        t[2]


def test_tree_store_prepared_batches_and_a_reader_that_follows(tmp_path):
    ex = {"a": np.zeros(0, np.float64), "b": np.zeros(0, np.float64)}
    writer = TreeStore.open(ex, str(tmp_path), mode="w")
    batch = [{"a": np.array([1.0, 2.0]), "b": np.array([3.0, 4.0])}, {"a": np.array([5.0, 6.0]), "b": np.array([7.0, 8.0])}]
    follower = TreeStore.open(ex, str(tmp_path), mode="r")
    assert len(follower) == 0
    writer.extend_with_batch(writer.batch_preparer(batch))
    assert len(follower.reload()) == 2 and len(TreeStore.open(ex, str(tmp_path), mode="r")) == 2
    asyncio.run(writer.extend_with_batch_async(writer.batch_preparer(batch)))
    follower = follower.reload()
    assert len(follower) == 4 and asyncio.run(follower.async_len()) == 4
    assert follower[3]["b"].tolist() == [7.0, 8.0]
    got = asyncio.run(follower.get_batch([3, 0]))
    assert got[0]["a"].tolist() == [5.0, 6.0] and got[1]["a"].tolist() == [1.0, 2.0]
    assert asyncio.run(follower.get_batch([])) == []
    asyncio.run(writer.trim_to_size_async(1))
    assert len(writer) == 1 and len(follower.reload()) == 1


# ---------------------------------------------------------------- the cache builder

class _Processor(BatchProcessor):
    def __call__(self, batch):
        return [{"test": np.asarray(x, np.int64)} for x in batch]

    @property
    def output_exemplar(self):
        return {"test": np.zeros(0, np.int64)}

    @property
    def metadata(self):
        return {}

    @property
    def num_cpus(self):
        return 1


class _Shards(ShardedDataSource):
    def __init__(self, num_shards=4, rows=10):
        self._n, self._rows = num_shards, rows

    @property
    def shard_names(self) -> Sequence[str]:
        return [f"shard_{i}" for i in range(self._n)]

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[list]:
        k = int(shard_name.split("_")[1])
        return ([k * 10 + i] * 10 for i in range(row, self._rows))


def _expected(source):
    return [np.asarray(x, np.int64) for s in source.shard_names for x in source.open_shard(s)]


def _check(cache, expected):
    got = list(cache)
    assert len(got) == len(expected)
    for g, e in zip(got, expected):
        np.testing.assert_array_equal(g["test"], e)


@pytest.mark.parametrize("options", [CacheOptions.default(), CacheOptions.no_fanciness(8), CacheOptions.one_group(),
                                     CacheOptions(num_shard_groups=2, batch_size=3, target_size_per_flush=1)])
def test_cache_end_to_end_in_shard_order(tmp_path, options):
    cache = build_or_load_cache(str(tmp_path), _Shards(5), _Processor(), options=options)
    assert cache.is_finished and len(cache) == 50
    _check(cache, _expected(_Shards(5)))
    # a fresh reader over the finished directory
    again = TreeCache.load(str(tmp_path), _Processor().output_exemplar)
    _check(again, _expected(_Shards(5)))
    assert again[7]["test"].tolist() == [7] * 10 and [r["test"][0] for r in again[48:50]] == [48, 49]


def test_a_finished_cache_is_not_rebuilt(tmp_path):
    first = build_or_load_cache(str(tmp_path), _Shards(), _Processor())

    class Throws(_Processor):
        def __call__(self, batch):
            raise RuntimeError("the processor must not run again")

    second = build_or_load_cache(str(tmp_path), _Shards(), Throws())
    _check(second, [r["test"] for r in first])


class _Boom(Exception):
    pass


class _CrashingShards(_Shards):
    def __init__(self, crash_point):
        super().__init__(4, 10)
        self.crash_point = crash_point

    def open_shard_at_row(self, shard_name, row):
        k = int(shard_name.split("_")[1])
        for i in range(10):
            if i == self.crash_point:
                raise _Boom(f"crash in {shard_name} at {i}")
            if i >= row:
                yield [k * 10 + i] * 10


def test_a_build_that_crashed_twice_resumes_to_the_same_cache(tmp_path):
    d = str(tmp_path / "a")
    with pytest.raises(_Boom):
        build_or_load_cache(d, _CrashingShards(4), _Processor(), options=CacheOptions(target_size_per_flush=1, batch_size=2))
    with pytest.raises(_Boom):
        build_or_load_cache(d, _CrashingShards(5), _Processor(), options=CacheOptions(batch_size=3))
    resumed = build_or_load_cache(d, _CrashingShards(10 ** 6), _Processor())
    straight = build_or_load_cache(str(tmp_path / "b"), _Shards(4), _Processor())
    assert len(resumed) == 40
    _check(resumed, [r["test"] for r in straight])


def test_a_source_without_shards_gives_an_empty_finished_cache(tmp_path):
    class Empty(ShardedDataSource):
        @property
        def shard_names(self):
            return []

        def open_shard_at_row(self, shard_name, row):
            raise RuntimeError("there is no shard to open")

    cache = build_or_load_cache(str(tmp_path), Empty(), _Processor())
    assert cache.is_finished and len(cache) == 0 and list(cache) == []


def test_shards_of_unequal_length_keep_their_order(tmp_path):
    class Uneven(ShardedDataSource):
        @property
        def shard_names(self):
            return ["shard_0", "shard_1"]

        def open_shard_at_row(self, shard_name, row):
            k = int(shard_name.split("_")[1])
            return ([i * 10 + k] * 10 for i in range(row, 40 if k == 1 else 20))

    cache = build_or_load_cache(str(tmp_path), Uneven(), _Processor(), await_finished=False, options=CacheOptions.no_fanciness(16))
    cache.await_finished(timeout=30)
    _check(cache, _expected(Uneven()))


def test_rows_are_readable_before_the_build_is_finished(tmp_path):
    gate = threading.Event()

    class Gated(ShardedDataSource):
        @property
        def shard_names(self):
            return ["shard_0"]

        def open_shard_at_row(self, shard_name, row):
            for i in range(row, 20):
                if i == 10:
                    assert gate.wait(30)
                yield [i] * 10

    cache = build_or_load_cache(str(tmp_path), Gated(), _Processor(), await_finished=False,
                                options=CacheOptions(target_size_per_flush=1, batch_size=1))

    async def scenario():
        first = await asyncio.wait_for(cache.get_batch(range(0, 10)), timeout=30)
        for i, x in enumerate(first):
            np.testing.assert_array_equal(x["test"], [i] * 10)
        assert not cache.is_finished and await cache.current_len() >= 10 and not await cache.final_length_is_known()
        with pytest.raises(asyncio.TimeoutError):
            await asyncio.wait_for(cache.get_batch(range(10, 20)), timeout=0.3)
        gate.set()
        rest = await asyncio.wait_for(cache.get_batch(range(10, 20)), timeout=30)
        for i, x in enumerate(rest, 10):
            np.testing.assert_array_equal(x["test"], [i] * 10)

    try:
        asyncio.run(scenario())
    finally:
        gate.set()
    cache.await_finished(timeout=30)
    assert cache.is_finished and len(cache) == 20


def test_a_processor_that_throws_fails_the_build_for_every_reader(tmp_path):
    class Throws(_Processor):
        def __call__(self, batch):
            raise RuntimeError("exc")

    with pytest.raises(RuntimeError, match="exc"):
        build_or_load_cache(str(tmp_path / "a"), _Shards(), Throws())
    cache = build_or_load_cache(str(tmp_path / "b"), _Shards(), Throws(), await_finished=False)
    with pytest.raises(RuntimeError, match="exc"):
        cache.get_batch_sync([0])
    with pytest.raises(RuntimeError, match="exc"):
        cache.await_finished(timeout=10)


def test_url_sources_refuse_duplicate_names_and_unknown_file_types(tmp_path):
    d = str(tmp_path)
    for name in ("data.txt", "data.txt.1", "data.not_a_real_extension"):
        open(f"{d}/{name}", "w").close()
    with pytest.raises(ValueError):
        UrlDataSource([f"{d}/data.txt", f"{d}/data.txt"]).shard_names
    with pytest.raises(ValueError):
        build_or_load_cache(f"{d}/c1", UrlDataSource([f"{d}/data.not_a_real_extension"]), _Processor())
    cache = build_or_load_cache(f"{d}/c2", UrlDataSource([f"{d}/data.not_a_real_extension"]), _Processor(), await_finished=False)
    with pytest.raises(ValueError):
        asyncio.run(cache.get_batch([0]))
    with pytest.raises(ValueError):
        cache.await_finished(timeout=10)


def test_serial_writer_drops_an_unfinished_cache_on_error(tmp_path):
    ex = {"test": np.zeros(0, np.int64)}
    with pytest.raises(_Boom):
        with SerialCacheWriter(str(tmp_path / "c"), ex) as w:
            w.write_batch([{"test": np.arange(3)}])
            raise _Boom()
    with pytest.raises(FileNotFoundError):
        TreeCache.load(str(tmp_path / "c"), ex)


def test_two_requests_for_a_cache_that_is_being_built_share_one_builder(tmp_path):
    gate = threading.Event()
    opened = []

    class Gated(ShardedDataSource):
        @property
        def shard_names(self):
            return ["shard_0"]

        def open_shard_at_row(self, shard_name, row):
            opened.append(row)
            for i in range(row, 12):
                if i == 6:
                    assert gate.wait(30)
                yield [i] * 4

    opts = CacheOptions(target_size_per_flush=1, batch_size=2)
    first = build_or_load_cache(str(tmp_path), Gated(), _Processor(), await_finished=False, options=opts)
    first.get_batch_sync([0])
    second = build_or_load_cache(str(tmp_path), Gated(), _Processor(), await_finished=False, options=opts)
    assert second._builder is first._builder and opened == [0]  # the source was opened once
    gate.set()
    first.await_finished(timeout=30)
    second.await_finished(timeout=30)
    _check(second, [np.asarray([i] * 4, np.int64) for i in range(12)])
    third = build_or_load_cache(str(tmp_path), Gated(), _Processor(), options=opts)  # finished: no builder at all
    assert third._builder is None and len(third) == 12
