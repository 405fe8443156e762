"""Jagged (ragged) array store: many variable-length rows in one flat array plus an offsets array
(src/levanter/store/jagged_array.py:85-131).

Layout under ``path`` (three zarr-v2 arrays, the reference's names): ``offsets`` int64 with ``offsets[0]`` = number of
rows and ``offsets[i + 1]`` = end of row ``i`` in ``data``; ``data`` flat, of the store's dtype; ``shapes`` int64
``[rows, item_rank - 1]`` with the leading dimensions of each row when rows are not 1-D.  Reads are batched: one decode of
the offset range plus one decode of the covering data range (row reads inside a batch are sliced from it), because a
chunk decode costs far more than a slice."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from .zarr_array import ZarrArray

# chunk lengths chosen so a chunk of int32 tokens is 1 MiB uncompressed: a cold random read of one 4k-token
# sequence decodes at most 2 chunks, while sequential cache builds still write few objects.
DEFAULT_CHUNK_SIZE = 256 * 1024
DEFAULT_WRITE_CHUNK_SIZE = DEFAULT_CHUNK_SIZE * 512


@dataclass
class PreparedBatch:
    """Rows already flattened for appending: ``data`` flat, ``offsets`` the exclusive end of each row *within the batch*,
    ``shapes`` the leading dims per row (or None)."""
    data: np.ndarray
    offsets: np.ndarray
    shapes: Optional[np.ndarray]

    def byte_size(self) -> int:
        return self.data.nbytes

    def astype(self, dtype) -> "PreparedBatch":
        return PreparedBatch(self.data.astype(dtype), self.offsets, self.shapes)

    @property
    def num_rows(self) -> int:
        return len(self.offsets)

    @staticmethod
    def from_batch(items: Sequence[np.ndarray], item_rank: Optional[int] = None) -> "PreparedBatch":
        if item_rank is None:
            item_rank = np.asarray(items[0]).ndim if len(items) else 1
        arrays = [np.asarray(x) for x in items]
        for a in arrays:
            if a.ndim != item_rank:
                raise ValueError(f"Expected rank {item_rank}, got {a.ndim}")
        shapes = np.array([a.shape[:-1] for a in arrays], dtype=np.int64).reshape(len(arrays), item_rank - 1) if item_rank > 1 else None
        sizes = np.array([a.size for a in arrays], dtype=np.int64)
        data = np.concatenate([a.reshape(-1) for a in arrays]) if arrays else np.zeros((0,), dtype=np.int32)
        return PreparedBatch(data, np.cumsum(sizes), shapes)

    @staticmethod
    def concat(batches: Sequence["PreparedBatch"]) -> "PreparedBatch":
        data = np.concatenate([b.data for b in batches])
        shapes = np.concatenate([b.shapes for b in batches]) if batches and batches[0].shapes is not None else None
        offs, base = [], 0
        for b in batches:
            offs.append(b.offsets + base)
            base += int(b.offsets[-1]) if len(b.offsets) else 0
        return PreparedBatch(data, np.concatenate(offs) if offs else np.zeros(0, np.int64), shapes)


class JaggedArrayStore:
    def __init__(self, offsets: ZarrArray, data: ZarrArray, shapes: Optional[ZarrArray], item_rank: int = 1, cache_metadata: bool = False):
        self.offsets, self.data, self.shapes = offsets, data, shapes
        self.item_rank = item_rank
        self._cache_metadata = cache_metadata
        self._cached_num_rows: Optional[int] = None
        self._cached_data_size: Optional[int] = None
        self._offset_cache: Optional[np.ndarray] = None

    @staticmethod
    def open(path: str, *, mode: str = "a", item_rank: int = 1, dtype, cache_metadata: bool = False) -> "JaggedArrayStore":
        def _open(sub, shape, chunks, dt):
            p = f"{path.rstrip('/')}/{sub}"
            if mode == "r" or (mode == "a" and ZarrArray.exists(p)):
                return ZarrArray.open(p)
            arr = ZarrArray.create(p, shape, chunks, dt, overwrite=(mode == "w"))
            return arr

        offsets = _open("offsets", [1], [DEFAULT_CHUNK_SIZE], np.int64)
        if offsets.shape == (1,) and mode != "r":
            try:
                offsets.read([0], [1])
            except Exception:
                pass
        data = _open("data", [0], [DEFAULT_CHUNK_SIZE], np.dtype(dtype))
        shapes = _open("shapes", [0, item_rank - 1], [DEFAULT_CHUNK_SIZE, item_rank - 1], np.int64) if item_rank > 1 else None
        return JaggedArrayStore(offsets, data, shapes, item_rank, cache_metadata and mode == "r")

    @staticmethod
    async def open_async(path: str, *, mode: str = "a", item_rank: int = 1, dtype, cache_metadata: bool = False) -> "JaggedArrayStore":
        return JaggedArrayStore.open(path, mode=mode, item_rank=item_rank, dtype=dtype, cache_metadata=cache_metadata)

    # -- sizes ---------------------------------------------------------------------------------------------------
    @property
    def num_rows(self) -> int:
        if self._cached_num_rows is not None:
            return self._cached_num_rows
        n = int(self.offsets.read([0], [1])[0])
        if self._cache_metadata:
            self._cached_num_rows = n
        return n

    async def num_rows_async(self) -> int:
        return self.num_rows

    @property
    def data_size(self) -> int:
        if self._cached_data_size is not None:
            return self._cached_data_size
        n = self.num_rows
        size = 0 if n == 0 else int(self.offsets.read([n], [n + 1])[0])
        if self._cache_metadata:
            self._cached_data_size = size
        return size

    async def data_size_async(self) -> int:
        return self.data_size

    def __len__(self) -> int:
        return self.num_rows

    # -- writing -------------------------------------------------------------------------------------------------
    def append(self, data: np.ndarray) -> None:
        self.extend([data])

    def extend(self, arrays) -> None:
        prepared = arrays if isinstance(arrays, PreparedBatch) else PreparedBatch.from_batch(arrays, self.item_rank)
        if prepared.num_rows == 0:
            return
        n, size = self.num_rows, self.data_size
        new_n = n + prepared.num_rows
        new_size = size + len(prepared.data)
        # data and shapes first, row count (offsets[0]) last: a reader that sees the new count sees complete rows
        if self.data.shape[0] < new_size:
            self.data.resize([new_size])
        self.data.write(prepared.data.astype(self.data.np_dtype, copy=False), [size])
        if self.shapes is not None:
            if self.shapes.shape[0] < new_n:
                self.shapes.resize([new_n, self.item_rank - 1])
            self.shapes.write(prepared.shapes, [n, 0])
        if self.offsets.shape[0] < new_n + 1:
            self.offsets.resize([new_n + 1])
        self.offsets.write(prepared.offsets + size, [n + 1])
        self.offsets.write(np.array([new_n], dtype=np.int64), [0])
        self._cached_num_rows = self._cached_data_size = None
        self._offset_cache = None

    async def extend_async(self, arrays) -> None:
        self.extend(arrays)

    async def append_async(self, data) -> None:
        self.extend([data])

    def trim_to_size(self, size: int) -> None:
        """Drop rows beyond ``size`` (recovery after an interrupted cache build)."""
        n = self.num_rows
        if size >= n:
            return
        new_data = 0 if size == 0 else int(self.offsets.read([size], [size + 1])[0])
        self.offsets.write(np.array([size], dtype=np.int64), [0])
        self.offsets.resize([size + 1])
        self.data.resize([new_data])
        if self.shapes is not None:
            self.shapes.resize([size, self.item_rank - 1])
        self._cached_num_rows = self._cached_data_size = None
        self._offset_cache = None

    async def trim_to_size_async(self, size: int) -> None:
        self.trim_to_size(size)

    def reload(self) -> "JaggedArrayStore":
        return JaggedArrayStore(ZarrArray.open(self.offsets.path), ZarrArray.open(self.data.path),
                                ZarrArray.open(self.shapes.path) if self.shapes is not None else None, self.item_rank, self._cache_metadata)

    async def reload_async(self) -> "JaggedArrayStore":
        return self.reload()

    # -- reading -------------------------------------------------------------------------------------------------
    def _bounds(self, start: int, stop: int) -> np.ndarray:
        """``[stop - start + 1]`` int64: data offsets delimiting rows ``start..stop``."""
        if self._cache_metadata:
            if self._offset_cache is None:
                self._offset_cache = self.offsets.read([0], [self.num_rows + 1]).copy()
                self._offset_cache[0] = 0
            return self._offset_cache[start:stop + 1]
        offs = self.offsets.read([start], [stop + 1]).astype(np.int64)
        if start == 0:
            offs[0] = 0
        return offs

    def _rows_from(self, lo_row: int, hi_row: int) -> List[np.ndarray]:
        bounds = self._bounds(lo_row, hi_row)
        flat = self.data.read([int(bounds[0])], [int(bounds[-1])])
        shapes = self.shapes.read([lo_row, 0], [hi_row, self.item_rank - 1]) if self.shapes is not None else None
        out = []
        for i in range(hi_row - lo_row):
            row = flat[int(bounds[i] - bounds[0]):int(bounds[i + 1] - bounds[0])]
            if shapes is not None:
                row = row.reshape(*[int(s) for s in shapes[i]], -1)
            out.append(row)
        return out

    def get_batch_sync(self, indices: Sequence[int]) -> List[np.ndarray]:
        indices = [int(i) for i in indices]
        if not indices:
            return []
        n = self.num_rows
        for i in indices:
            if i < 0 or i >= n:
                raise IndexError(f"Index {i} out of bounds for {n} rows")
        # group runs of nearby rows into single range reads
        order = np.argsort(indices, kind="stable")
        out: List[Optional[np.ndarray]] = [None] * len(indices)
        run = [order[0]]
        for j in order[1:]:
            if indices[j] - indices[run[-1]] <= 8:
                run.append(j)
            else:
                self._fill_run(indices, run, out)
                run = [j]
        self._fill_run(indices, run, out)
        return out  # type: ignore

    def _fill_run(self, indices, run, out):
        lo, hi = indices[run[0]], indices[run[-1]] + 1
        rows = self._rows_from(lo, hi)
        for j in run:
            out[j] = rows[indices[j] - lo]

    async def get_batch(self, indices: Sequence[int]) -> List[np.ndarray]:
        return self.get_batch_sync(indices)

    async def get_item_async(self, item):
        return self[item]

    def __getitem__(self, item):
        if isinstance(item, slice):
            start, stop, step = item.indices(self.num_rows)
            if step != 1:
                return self.get_batch_sync(range(start, stop, step))
            return self._rows_from(start, stop) if stop > start else []
        n = self.num_rows
        if item < 0:
            item += n
        if item < 0 or item >= n:
            raise IndexError(f"Index {item} out of bounds for {n} rows")
        return self._rows_from(item, item + 1)[0]

    def __iter__(self):
        n = self.num_rows
        step = 1024
        for s in range(0, n, step):
            yield from self._rows_from(s, min(n, s + step))
