"""Preprocessed-dataset cache: a :class:`TreeStore` plus a ledger, built from a sharded source by a batch processor
(src/levanter/store/cache.py:109-172 ``build_or_load_cache``, :174-476 ``TreeCache``, :479-523 ``CacheLedger``).

The reference fans the build out over Ray actors that write temporary per-group caches and copies them into the final
one.  Here one process builds: reader/processor threads (Hugging Face fast tokenizers release the GIL) work on several
shards at once and hand prepared batches to a single writer through bounded per-shard queues; the writer appends shards
in the source's order, so the cache contents depend only on (source, processor) and never on thread timing.  The ledger
(``shard_ledger.json``, the reference's name and fields) is re-committed after every flush with the rows consumed per
shard, so an interrupted build resumes mid-shard through ``open_shard_at_row`` and a reader can train on the rows that
exist while the build is still running.  In a multi-process job rank 0 builds and the others follow the ledger.
"""
from __future__ import annotations

import asyncio
import copy
import dataclasses
import json
import logging as pylogging
import os
import queue
import threading
import time
from contextlib import AbstractContextManager
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Generic, List, Optional, Sequence, TypeVar, Union

import numpy as np

from ..data._preprocessor import BatchProcessor, _canonicalize_batch
from ..data.dataset import AsyncDataset
from ..data.metrics_monitor import InProgressCacheMetrics, LoggerMetricsMonitor, MetricsMonitor
from ..data.utils import batched
from ..utils import fsspec_utils
from .tree_store import TreeBatchPreparer, TreeStore

T = TypeVar("T")
T_co = TypeVar("T_co", covariant=True)
logger = pylogging.getLogger(__name__)

LEDGER_FILE_NAME = "shard_ledger.json"
DEFAULT_LOG_LEVEL = pylogging.INFO
LEVEL_TO_LOG = pylogging.INFO


def _parse_size(s: Union[int, str]) -> int:
    if isinstance(s, int):
        return s
    s = s.strip().upper()
    units = [("KIB", 1 << 10), ("MIB", 1 << 20), ("GIB", 1 << 30), ("TIB", 1 << 40), ("KB", 10**3), ("MB", 10**6), ("GB", 10**9),
             ("TB", 10**12), ("K", 10**3), ("M", 10**6), ("G", 10**9), ("B", 1)]
    for suf, mul in units:
        if s.endswith(suf):
            return int(float(s[: -len(suf)]) * mul)
    return int(s)


@dataclass(frozen=True)
class CacheOptions:
    """Build-time knobs.  ``num_shard_groups`` bounds how many shards are processed concurrently; the two others only change
    memory use and flush cadence, never the result."""
    num_shard_groups: Optional[int] = 128
    target_size_per_flush: Union[int, str] = "512MB"
    batch_size: int = 128

    @property
    def target_bytes_per_flush(self) -> int:
        return _parse_size(self.target_size_per_flush)

    @staticmethod
    def default() -> "CacheOptions":
        return CacheOptions()

    @staticmethod
    def no_fanciness(batch_size: Optional[int] = None) -> "CacheOptions":
        return CacheOptions(num_shard_groups=None, batch_size=batch_size or 128)

    @staticmethod
    def one_group() -> "CacheOptions":
        return CacheOptions(num_shard_groups=1, batch_size=128)


@dataclass(frozen=True)
class CacheMetadata:
    preprocessor_metadata: Optional[Dict[str, Any]] = None

    def compare_to(self, other: "CacheMetadata") -> Dict[str, Any]:
        """Differences against ``other`` ({} when compatible).  ``other.preprocessor_metadata is None`` matches anything."""
        if other.preprocessor_metadata is None or self.preprocessor_metadata == other.preprocessor_metadata:
            return {}
        a, b = self.preprocessor_metadata or {}, other.preprocessor_metadata or {}
        return {k: (a.get(k), b.get(k)) for k in sorted(set(a) | set(b)) if a.get(k) != b.get(k)}

    @staticmethod
    def empty() -> "CacheMetadata":
        return CacheMetadata()


@dataclass
class CacheLedger:
    """What has been written so far.  The existence of a ledger does not mean the cache is finished: check ``is_finished``."""
    total_num_rows: int
    shard_rows: Dict[str, int]
    is_finished: bool = False
    finished_shards: List[str] = field(default_factory=list)
    field_counts: Dict[str, int] = field(default_factory=dict)
    metadata: CacheMetadata = field(default_factory=lambda: CacheMetadata({}))

    def to_json(self) -> str:
        d = dataclasses.asdict(self)
        return json.dumps(d)

    @staticmethod
    def from_json(s: Union[str, bytes]) -> "CacheLedger":
        d = json.loads(s)
        md = d.get("metadata") or {}
        return CacheLedger(total_num_rows=d["total_num_rows"], shard_rows=d.get("shard_rows", {}), is_finished=d.get("is_finished", False),
                           finished_shards=d.get("finished_shards", []), field_counts=d.get("field_counts", {}),
                           metadata=CacheMetadata(md.get("preprocessor_metadata")))

    @staticmethod
    def load_or_initialize(cache_dir: str, source, processor: BatchProcessor) -> "CacheLedger":
        metadata = CacheMetadata(preprocessor_metadata=processor.metadata)
        try:
            return CacheLedger.load(cache_dir, metadata)
        except FileNotFoundError:
            return CacheLedger(total_num_rows=0, shard_rows={s: 0 for s in source.shard_names}, is_finished=False, metadata=metadata)

    @staticmethod
    def load(cache_dir: str, metadata: Optional[CacheMetadata] = None) -> "CacheLedger":
        path = os.path.join(cache_dir, LEDGER_FILE_NAME)
        import fsspec

        try:
            with fsspec.open(path, "r") as f:
                ledger = CacheLedger.from_json(f.read())
        except FileNotFoundError:
            raise FileNotFoundError(f"Cache ledger not found at {path}")
        if metadata is not None:
            diff = ledger.metadata.compare_to(metadata)
            if diff:
                logger.warning(f"Cache metadata mismatch at {cache_dir}: {diff}")
        return ledger

    def _serialize_and_commit(self, cache_dir: str) -> None:
        _serialize_json_and_commit(os.path.join(cache_dir, LEDGER_FILE_NAME), self)


def _serialize_json_and_commit(path: str, obj) -> None:
    """Write ``path`` atomically where the filesystem allows: write a sibling then rename over the target."""
    import fsspec

    fs, p = fsspec.core.url_to_fs(path)
    fs.makedirs(os.path.dirname(p), exist_ok=True)
    tmp = f"{p}.tmp"
    with fs.open(tmp, "w") as f:
        f.write(obj.to_json())
    try:
        fs.mv(tmp, p)
    except Exception:
        if fs.exists(p):
            fs.copy(p, f"{p}.bak")
        fs.mv(tmp, p)


def _ledger_to_metrics(ledger: CacheLedger) -> InProgressCacheMetrics:
    return InProgressCacheMetrics(rows_finished=ledger.total_num_rows, is_finished=ledger.is_finished,
                                  shards_finished=len(ledger.finished_shards), field_counts=dict(ledger.field_counts))


def _count_fields(ledger: CacheLedger, rows: List[dict]) -> None:
    for r in rows:
        if not isinstance(r, dict):
            continue
        for k, v in r.items():
            try:
                ledger.field_counts[k] = ledger.field_counts.get(k, 0) + int(np.size(v))
            except Exception:
                pass


class SerialCacheWriter(AbstractContextManager):
    """Write a cache from the calling thread: ``with SerialCacheWriter(dir, exemplar) as w: w.write_batch(rows)``
    (src/levanter/store/cache.py:548-603).  Leaving the block without an exception marks the cache finished."""

    def __init__(self, cache_dir: str, exemplar, metadata: Optional[CacheMetadata] = None, shard_name: str = ""):
        self.cache_dir = cache_dir
        self.metadata = metadata or CacheMetadata.empty()
        self._exemplar = exemplar
        self._shard_name = shard_name
        self._tree_store = TreeStore.open(exemplar, cache_dir, mode="w", cache_metadata=False)
        self._is_closed = False
        self._ledger = CacheLedger(0, {}, metadata=self.metadata)

    def __enter__(self) -> "SerialCacheWriter":
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        if exc_type is None:
            self._ledger.is_finished = True
        self._ledger.total_num_rows = len(self._tree_store)
        self._ledger._serialize_and_commit(self.cache_dir)
        self._is_closed = True
        return False

    def result(self) -> "TreeCache":
        if not self._is_closed:
            raise RuntimeError("Cannot get result until the writer is closed")
        return TreeCache.load(self.cache_dir, self._exemplar, self.metadata)

    def write_batch(self, batch) -> None:
        rows = _canonicalize_batch(batch)
        if not rows:
            return
        self._tree_store.extend(rows)
        _count_fields(self._ledger, rows)
        self._ledger.total_num_rows = len(self._tree_store)
        if self._shard_name:
            self._ledger.shard_rows[self._shard_name] = self._ledger.shard_rows.get(self._shard_name, 0) + len(rows)


class TreeCache(AsyncDataset[T_co]):
    """Random-access dataset over a cache directory.  While a build is running (``_builder`` set) reads wait until the rows
    they need exist; when built by another process the ledger is polled instead."""

    def __init__(self, cache_dir: str, exemplar, ledger: Optional[CacheLedger], _builder: Optional["_CacheBuilder"] = None):
        super().__init__()
        self.cache_dir = cache_dir
        self.ledger = ledger
        self._exemplar = exemplar
        self._builder = _builder
        self._store: Optional[TreeStore] = None
        self._metrics_monitors: List[MetricsMonitor] = []
        name = os.path.join(*cache_dir.rstrip("/").split("/")[-2:])
        self.logger = pylogging.getLogger(f"TreeCache.{name}")
        if _builder is not None:
            _builder.add_listener(self._on_ledger)
        if ledger is not None and ledger.is_finished:
            self._attempt_to_load_store(cache_metadata=True)

    # -- construction -------------------------------------------------------------------------------------------
    @staticmethod
    def load(cache_dir: str, exemplar, options: Optional[CacheMetadata] = None) -> "TreeCache":
        """Open a finished cache; raises FileNotFoundError if there is no finished cache at ``cache_dir``."""
        ledger = CacheLedger.load(cache_dir, options)
        if not ledger.is_finished:
            raise FileNotFoundError(f"Cache at {cache_dir} is not finished. Use build_or_load to build it.")
        return TreeCache(cache_dir, exemplar, ledger, None)

    @staticmethod
    def build_or_load(cache_dir: str, shard_source, processor: BatchProcessor, options: Optional[CacheOptions] = None) -> "TreeCache":
        return build_or_load_cache(cache_dir, shard_source, processor, await_finished=False, options=options or CacheOptions.default())

    def _attempt_to_load_store(self, cache_metadata: bool = False) -> bool:
        try:
            self._store = TreeStore.open(self._exemplar, self.cache_dir, mode="r", cache_metadata=cache_metadata)
            return True
        except FileNotFoundError:
            return False

    @property
    def store(self) -> TreeStore:
        if self._store is None:
            self.await_finished() if self._builder is None else self._wait_for_rows(1)
            if self._store is None and not self._attempt_to_load_store(cache_metadata=self.is_finished):
                raise FileNotFoundError(f"no cache data under {self.cache_dir}")
        return self._store  # type: ignore

    async def store_async(self) -> TreeStore:
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.store)

    @property
    def is_finished(self) -> bool:
        return self.ledger is not None and self.ledger.is_finished

    def _on_ledger(self, ledger: CacheLedger) -> None:
        self.ledger = ledger
        metrics = _ledger_to_metrics(ledger)
        for m in self._metrics_monitors:
            try:
                m(metrics)
            except Exception:
                self.logger.exception("metrics monitor failed")
        if ledger.is_finished:
            self._store = None  # reopen with cached metadata

    def attach_metrics_monitor(self, monitor: MetricsMonitor) -> None:
        self._metrics_monitors.append(monitor)
        if self.ledger is not None:
            monitor(_ledger_to_metrics(self.ledger))

    # -- waiting ------------------------------------------------------------------------------------------------
    def _refresh_ledger(self) -> None:
        if self._builder is not None:
            self._builder.raise_if_failed()
            self.ledger = self._builder.ledger_snapshot()
        else:
            try:
                self.ledger = CacheLedger.load(self.cache_dir)
            except FileNotFoundError:
                pass

    def _wait_for_rows(self, needed: int, timeout: Optional[float] = None) -> int:
        t0 = time.time()
        while True:
            if self.ledger is not None and (self.ledger.total_num_rows >= needed or self.ledger.is_finished):
                return self.ledger.total_num_rows
            self._refresh_ledger()
            if self.ledger is not None and (self.ledger.total_num_rows >= needed or self.ledger.is_finished):
                return self.ledger.total_num_rows
            if timeout is not None and time.time() - t0 > timeout:
                raise TimeoutError(f"cache at {self.cache_dir} did not reach {needed} rows in {timeout} s")
            time.sleep(0.05 if self._builder is not None else 1.0)

    def await_finished(self, timeout: Optional[float] = None) -> None:
        if self.is_finished:
            return
        if self._builder is not None:
            self._builder.join(timeout)
            self._builder.raise_if_failed()
            self.ledger = self._builder.ledger_snapshot()
        else:
            self._wait_for_rows(1 << 62, timeout)
        if self.is_finished:
            self._store = None
            self._attempt_to_load_store(cache_metadata=True)

    async def finished(self) -> None:
        await asyncio.get_event_loop().run_in_executor(None, self.await_finished)

    # -- AsyncDataset -------------------------------------------------------------------------------------------
    async def async_len(self) -> int:
        await self.finished()
        return len(self.store)

    def __len__(self) -> int:
        self.await_finished()
        return len(self.store)

    async def final_length_is_known(self) -> bool:
        return self.is_finished

    def is_finite(self) -> bool:
        return True

    async def current_len(self) -> int:
        if not self.is_finished:
            self._refresh_ledger()
        return 0 if self.ledger is None else self.ledger.total_num_rows

    async def wait_until_len_at_least(self, length: int) -> int:
        return await asyncio.get_event_loop().run_in_executor(None, self._wait_for_rows, length)

    def _store_for_read(self) -> TreeStore:
        if self.is_finished:
            return self.store
        # rows are still being appended: reopen so array shapes are current
        if not self._attempt_to_load_store(cache_metadata=False):
            raise FileNotFoundError(f"no cache data under {self.cache_dir}")
        return self._store  # type: ignore

    def get_batch_sync(self, indices) -> List[T_co]:
        if isinstance(indices, slice):
            start, stop, step = indices.start or 0, indices.stop, indices.step or 1
            if stop is None or stop < 0 or start < 0:
                start, stop, step = indices.indices(len(self))
            indices = range(start, stop, step)
        indices = list(indices)
        if not indices:
            return []
        n = self._wait_for_rows(max(indices) + 1)
        if max(indices) >= n:
            raise IndexError(f"index {max(indices)} out of bounds for cache of {n} rows")
        return self._store_for_read().get_batch_sync(indices)

    async def get_batch(self, indices) -> List[T_co]:
        return await asyncio.get_event_loop().run_in_executor(None, self.get_batch_sync, indices)

    def __getitem__(self, item):
        if isinstance(item, slice):
            return self.get_batch_sync(item)
        if item < 0:
            item += len(self)
        return self.get_batch_sync([item])[0]

    def __iter__(self):
        n = len(self)
        for s in range(0, n, 256):
            yield from self.get_batch_sync(range(s, min(n, s + 256)))


_SENTINEL = object()
_BUILDERS: Dict[str, "_CacheBuilder"] = {}  # running builds of this process by cache directory
_BUILDERS_LOCK = threading.Lock()


class _CacheBuilder:
    """Background build.  ``workers`` reader threads each take the next unfinished shard, run the processor on batches of raw
    rows and push ``(n_input_rows, processed rows, prepared leaves)`` into that shard's bounded queue; the writer thread drains
    the queues in shard order and commits the ledger every ``target_bytes_per_flush`` bytes."""

    def __init__(self, cache_dir: str, source, processor: BatchProcessor, options: CacheOptions, ledger: CacheLedger):
        self.cache_dir, self.source, self.processor, self.options = cache_dir, source, processor, options
        self._ledger = ledger
        self._lock = threading.Lock()
        self._listeners: List[Callable[[CacheLedger], None]] = []
        self._error: Optional[BaseException] = None
        self._stop = threading.Event()
        self._shards = [s for s in source.shard_names if s not in set(ledger.finished_shards)]
        n_workers = options.num_shard_groups or len(self._shards) or 1
        self._n_workers = max(1, min(n_workers, len(self._shards) or 1, (os.cpu_count() or 4), 16))
        self._queues: Dict[str, "queue.Queue"] = {s: queue.Queue(maxsize=4) for s in self._shards}
        self._next_shard = 0
        self._thread = threading.Thread(target=self._run, name=f"cache-writer:{cache_dir}", daemon=True)
        self._thread.start()

    # -- public -------------------------------------------------------------------------------------------------
    def add_listener(self, fn) -> None:
        self._listeners.append(fn)

    def ledger_snapshot(self) -> CacheLedger:
        with self._lock:
            return copy.deepcopy(self._ledger)

    def join(self, timeout: Optional[float] = None) -> None:
        self._thread.join(timeout)

    def raise_if_failed(self) -> None:
        if self._error is not None:
            # the builder's own exception, so that callers can catch what the source or the processor raised
            err = self._error
            note = f"raised by the cache build at {self.cache_dir}"
            if isinstance(err, Exception) and note not in getattr(err, "__notes__", ()):
                err.add_note(note)
            raise err

    # -- threads ------------------------------------------------------------------------------------------------
    def _take_shard(self) -> Optional[str]:
        with self._lock:
            if self._next_shard >= len(self._shards):
                return None
            s = self._shards[self._next_shard]
            self._next_shard += 1
            return s

    def _reader(self, preparer: TreeBatchPreparer) -> None:
        try:
            while not self._stop.is_set():
                shard = self._take_shard()
                if shard is None:
                    return
                q = self._queues[shard]
                start_row = self._ledger.shard_rows.get(shard, 0)
                it = self.source.open_shard_at_row(shard, start_row)
                for raw in batched(it, self.options.batch_size):
                    if self._stop.is_set():
                        return
                    rows = _canonicalize_batch(self.processor(raw))
                    prepared = preparer(rows) if rows else None
                    self._put(q, (len(raw), rows, prepared))
                self._put(q, _SENTINEL)
        except BaseException as e:  # noqa: BLE001 - forwarded to the waiting reader of the cache
            self._error = e
            self._stop.set()

    def _put(self, q, item) -> None:
        while not self._stop.is_set():
            try:
                q.put(item, timeout=0.2)
                return
            except queue.Full:
                continue

    def _commit(self, finished: bool = False) -> None:
        with self._lock:
            self._ledger.is_finished = finished
            snap = copy.deepcopy(self._ledger)
        snap._serialize_and_commit(self.cache_dir)
        for fn in self._listeners:
            fn(snap)

    def _run(self) -> None:
        try:
            exemplar = self.processor.output_exemplar
            mode = "a" if self._ledger.total_num_rows > 0 else "w"
            store = TreeStore.open(exemplar, self.cache_dir, mode=mode)
            if len(store) != self._ledger.total_num_rows:
                # an append after the last ledger commit was interrupted: drop the rows the ledger does not know about
                store.trim_to_size(self._ledger.total_num_rows)
            preparer = TreeBatchPreparer(exemplar)
            readers = [threading.Thread(target=self._reader, args=(preparer,), daemon=True) for _ in range(self._n_workers)]
            for r in readers:
                r.start()
            unflushed = 0
            for shard in self._shards:
                q = self._queues[shard]
                while True:
                    try:
                        item = q.get(timeout=0.2)
                    except queue.Empty:
                        if self._stop.is_set():
                            raise self._error or RuntimeError("cache build stopped")
                        continue
                    if item is _SENTINEL:
                        break
                    n_in, rows, prepared = item
                    if prepared is not None:
                        store.extend_with_batch(prepared)
                        unflushed += sum(p.byte_size() for p in prepared.values())
                    with self._lock:
                        self._ledger.total_num_rows += len(rows)
                        self._ledger.shard_rows[shard] = self._ledger.shard_rows.get(shard, 0) + n_in
                        _count_fields(self._ledger, rows)
                    if unflushed >= self.options.target_bytes_per_flush:
                        self._commit()
                        unflushed = 0
                with self._lock:
                    self._ledger.finished_shards.append(shard)
                self._commit()
                unflushed = 0
            self._commit(finished=True)
        except BaseException as e:  # noqa: BLE001
            if self._error is None:
                self._error = e
            self._stop.set()
            logger.exception(f"cache build at {self.cache_dir} failed")
        finally:
            with _BUILDERS_LOCK:  # finished or failed: the next request starts from the ledger on disk
                for k, b in list(_BUILDERS.items()):
                    if b is self:
                        del _BUILDERS[k]


def build_or_load_cache(cache_dir: str, source, processor: BatchProcessor, await_finished: bool = True,
                        monitors: Optional[Sequence[MetricsMonitor]] = None, options: CacheOptions = CacheOptions.default(),
                        force_flush: bool = False) -> TreeCache:
    """Open the cache at ``cache_dir``, building (or resuming the build of) it from ``source`` through ``processor`` when it is
    not finished.  With ``await_finished=False`` the returned cache can be read while rows are still being added."""
    if options is None:
        options = CacheOptions.default()
    metadata = CacheMetadata(preprocessor_metadata=processor.metadata)
    try:
        return TreeCache.load(cache_dir, processor.output_exemplar, metadata)
    except FileNotFoundError:
        pass
    from ..distributed import process_index

    if process_index() != 0:
        cache = TreeCache(cache_dir, processor.output_exemplar, None, None)  # follows the ledger rank 0 writes
    else:
        # one builder per directory and process: a second request while a build is running reads along with it (the
        # reference gets this from a named actor per cache directory)
        key = os.path.abspath(cache_dir) if "://" not in cache_dir else cache_dir
        with _BUILDERS_LOCK:
            builder = _BUILDERS.get(key)
            if builder is not None and (not builder._thread.is_alive() or builder._error is not None):
                builder = None
            if builder is None:
                ledger = CacheLedger.load_or_initialize(cache_dir, source, processor)
                for s in source.shard_names:
                    ledger.shard_rows.setdefault(s, 0)
                builder = _BUILDERS[key] = _CacheBuilder(cache_dir, source, processor, options, ledger)
        cache = TreeCache(cache_dir, processor.output_exemplar, builder.ledger_snapshot(), builder)
    for m in monitors or []:
        cache.attach_metrics_monitor(m)
    if await_finished:
        cache.await_finished()
    return cache
