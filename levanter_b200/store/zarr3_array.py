"""Read-only zarr v3 arrays, as far as the reference's token caches need them.

The reference stores every cache field as TensorStore ``zarr3`` arrays (``offsets``, ``data``, ``shapes``) whose chunks are
shards: ``sharding_indexed`` with inner chunks compressed by blosc (src/levanter/store/jagged_array.py:605-635).  A shard
file is the concatenation of its encoded inner chunks plus an index of ``(offset, nbytes)`` uint64 pairs, one per inner
chunk in C order, little-endian, followed by a CRC-32C of the index; ``2^64 - 1`` twice marks a chunk that was never
written.  This class parses ``zarr.json``, finds the inner chunks that a requested region touches, reads only their byte
ranges, and decodes them with the native codec (``ops/csrc/chunk_codec.cpp``: blosc frames with lz4 or zstd, byte shuffle).
Supported codecs: ``bytes`` (little-endian), ``blosc``, ``zstd``, ``gzip``, ``crc32c``, and ``sharding_indexed`` around
them; ``transpose`` and big-endian data are refused.  New caches are written in this framework's zarr v2 layout
(:mod:`zarr_array`); an existing v3 cache opens through the same ``ZarrArray.open`` call and reads the same way."""
from __future__ import annotations

import ctypes
import itertools
import json
import struct
import zlib
from typing import List, Optional, Sequence, Tuple

import numpy as np
from fsspec.core import url_to_fs

_V3_DTYPES = {"bool": "bool", "int8": "int8", "int16": "int16", "int32": "int32", "int64": "int64", "uint8": "uint8",
              "uint16": "uint16", "uint32": "uint32", "uint64": "uint64", "float16": "float16", "float32": "float32",
              "float64": "float64", "bfloat16": "uint16"}
_MISSING = (1 << 64) - 1


def _native():
    from ..ops import lib as L

    l = L.load()
    l.lvb_blosc_nbytes.restype = ctypes.c_longlong
    l.lvb_blosc_nbytes.argtypes = [ctypes.c_char_p, ctypes.c_longlong]
    l.lvb_crc32c.restype = ctypes.c_uint
    l.lvb_crc32c.argtypes = [ctypes.c_char_p, ctypes.c_longlong]
    return l


def crc32c(data: bytes) -> int:
    return int(_native().lvb_crc32c(data, len(data)))


def blosc_decompress_many(blobs: List[bytes], threads: int = 8, expect: Optional[int] = None) -> List[np.ndarray]:
    """Decode blosc frames (lz4 / zstd / stored, byte shuffle) in parallel on the native thread pool.  ``expect``: the decoded
    size every frame must declare (a chunk's byte count), checked before any buffer is allocated from a frame's own header."""
    l = _native()
    n = len(blobs)
    sizes = [int(l.lvb_blosc_nbytes(b, len(b))) for b in blobs]
    if any(s < 0 for s in sizes):
        raise ValueError("not a blosc frame")
    if expect is not None and any(s != expect for s in sizes):
        raise ValueError(f"a blosc frame declares {[s for s in sizes if s != expect][0]} decoded bytes where the chunk has {expect}")
    outs = [np.empty(max(s, 1), dtype=np.uint8) for s in sizes]
    P, LL = ctypes.c_void_p, ctypes.c_longlong
    keep = [ctypes.create_string_buffer(b, len(b)) for b in blobs]
    src = (P * n)(*[ctypes.cast(k, P) for k in keep])
    dst = (P * n)(*[o.ctypes.data for o in outs])
    src_len = (LL * n)(*[len(b) for b in blobs])
    cap = (LL * n)(*sizes)
    out_len = (LL * n)()
    l.lvb_blosc_decompress_many.argtypes = [ctypes.c_int, ctypes.POINTER(P), ctypes.POINTER(LL), ctypes.POINTER(P), ctypes.POINTER(LL),
                                            ctypes.POINTER(LL), ctypes.c_int]
    rc = l.lvb_blosc_decompress_many(n, src, src_len, dst, cap, out_len, threads)
    if rc != 0:
        raise ValueError(f"blosc frame could not be decoded (code {rc}: -13 = malformed or a codec other than lz4 / zstd / stored, "
                         "or bit shuffle; -10 = zstd library missing)")
    return [o[:s] for o, s in zip(outs, sizes)]


class _Pipeline:
    """The bytes -> bytes part of a codec chain plus the array -> bytes ``bytes`` codec."""

    def __init__(self, codecs: List[dict], where: str):
        self.steps: List[Tuple[str, dict]] = []
        seen_bytes = False
        for c in codecs:
            name, conf = c["name"], c.get("configuration", {}) or {}
            if name == "bytes":
                if conf.get("endian", "little") != "little":
                    raise NotImplementedError(f"{where}: big-endian data is not supported")
                seen_bytes = True
            elif name in ("blosc", "zstd", "gzip", "crc32c"):
                self.steps.append((name, conf))
            else:
                raise NotImplementedError(f"{where}: codec {name!r} is not supported")
        del seen_bytes

    def decode_many(self, blobs: List[bytes], expect: Optional[int] = None) -> List[np.ndarray]:
        """``expect``: byte count of a decoded chunk (known from the chunk shape), enforced on the innermost compressor."""
        cur: List = list(blobs)
        for pos in range(len(self.steps) - 1, -1, -1):
            name = self.steps[pos][0]
            innermost = pos == 0
            if name == "crc32c":
                nxt = []
                for b in cur:
                    b = bytes(b)
                    body, (want,) = b[:-4], struct.unpack("<I", b[-4:])
                    if crc32c(body) != want:
                        raise ValueError("CRC-32C mismatch in a zarr v3 chunk")
                    nxt.append(body)
                cur = nxt
            elif name == "blosc":
                cur = blosc_decompress_many([bytes(b) for b in cur], expect=expect if innermost else None)
            elif name == "gzip":
                cur = [zlib.decompress(bytes(b), 15 + 32) for b in cur]
            elif name == "zstd":
                from .zarr_array import CODEC

                if not CODEC.has_zstd:
                    raise RuntimeError("this array is zstd-compressed but libzstd could not be loaded")
                lib = CODEC.lib()
                sizes = [int(lib.lvb_zstd_frame_size(bytes(b), len(b))) for b in cur]
                cur = CODEC.decompress_many([bytes(b) for b in cur], sizes)
        return [np.frombuffer(bytes(b), dtype=np.uint8) if not isinstance(b, np.ndarray) else b for b in cur]


class Zarr3Array:
    """One zarr v3 array, read-only.  ``read(lo, hi)`` has the semantics of :meth:`ZarrArray.read`."""

    zarr_format = 3

    def __init__(self, path: str, meta: dict):
        self.path = path.rstrip("/")
        self.fs, self.root = url_to_fs(self.path)
        if meta.get("node_type", "array") != "array":
            raise ValueError(f"{path}: a zarr v3 group, not an array")
        self.meta = meta
        self.shape: List[int] = [int(s) for s in meta["shape"]]
        dt = meta["data_type"]
        if not isinstance(dt, str) or dt not in _V3_DTYPES:
            raise NotImplementedError(f"{path}: data type {dt!r} is not supported")
        self.dtype_str = dt
        self.np_dtype = np.dtype(_V3_DTYPES[dt])
        grid = meta["chunk_grid"]
        if grid.get("name") != "regular":
            raise NotImplementedError(f"{path}: chunk grid {grid.get('name')!r}")
        self.chunks: List[int] = [int(c) for c in grid["configuration"]["chunk_shape"]]
        enc = meta.get("chunk_key_encoding", {"name": "default"})
        self._key_style = enc.get("name", "default")
        self._sep = (enc.get("configuration") or {}).get("separator", "/" if self._key_style == "default" else ".")
        fv = meta.get("fill_value", 0)
        if isinstance(fv, str):
            fv = {"NaN": np.nan, "Infinity": np.inf, "-Infinity": -np.inf}.get(fv, 0)
        self.fill = 0 if dt == "bfloat16" else (fv if fv is not None else 0)
        codecs = meta.get("codecs", [])
        self.inner: Optional[List[int]] = None
        if codecs and codecs[0]["name"] == "sharding_indexed":
            if len(codecs) != 1:
                raise NotImplementedError(f"{path}: codecs after sharding_indexed")
            conf = codecs[0]["configuration"]
            self.inner = [int(c) for c in conf["chunk_shape"]]
            if any(o % i for o, i in zip(self.chunks, self.inner)):
                raise ValueError(f"{path}: the shard shape is not a multiple of the inner chunk shape")
            self.pipe = _Pipeline(conf.get("codecs", []), path)
            idx = conf.get("index_codecs", [{"name": "bytes"}, {"name": "crc32c"}])
            self._index_crc = any(c["name"] == "crc32c" for c in idx)
            if any(c["name"] not in ("bytes", "crc32c") for c in idx):
                raise NotImplementedError(f"{path}: index codecs {idx}")
            self._index_at_end = conf.get("index_location", "end") == "end"
        else:
            self.pipe = _Pipeline(codecs, path)

    # ------------------------------------------------------------------------------------------------------------------
    @staticmethod
    def exists(path: str) -> bool:
        fs, root = url_to_fs(path.rstrip("/"))
        return fs.exists(f"{root}/zarr.json")

    @staticmethod
    def open(path: str) -> "Zarr3Array":
        fs, root = url_to_fs(path.rstrip("/"))
        with fs.open(f"{root}/zarr.json", "r") as f:
            meta = json.load(f)
        if meta.get("zarr_format") != 3:
            raise NotImplementedError(f"zarr_format {meta.get('zarr_format')}")
        return Zarr3Array(path, meta)

    def _key(self, idx: Tuple[int, ...]) -> str:
        if self._key_style == "default":
            return f"{self.root}/" + self._sep.join(["c"] + [str(i) for i in idx])
        return f"{self.root}/" + (self._sep.join(str(i) for i in idx) if idx else "0")

    def _chunk_elems(self, shape: Sequence[int]) -> int:
        return int(np.prod(shape, dtype=np.int64)) if len(shape) else 1

    def _read_shard_parts(self, key: str, wanted: List[int]) -> List[Optional[bytes]]:
        """Encoded bytes of the inner chunks ``wanted`` (linear C-order indices within the shard); ``None`` where unwritten."""
        per = [o // i for o, i in zip(self.chunks, self.inner)]
        n_inner = self._chunk_elems(per)
        index_bytes = 16 * n_inner + (4 if self._index_crc else 0)
        try:
            f = self.fs.open(key, "rb")
        except FileNotFoundError:
            return [None] * len(wanted)
        with f:
            size = self.fs.size(key)
            f.seek(size - index_bytes if self._index_at_end else 0)
            raw = f.read(index_bytes)
            if self._index_crc:
                body, (want,) = raw[:-4], struct.unpack("<I", raw[-4:])
                if crc32c(body) != want:
                    raise ValueError(f"{key}: CRC-32C mismatch in the shard index")
                raw = body
            index = np.frombuffer(raw, dtype="<u8").reshape(n_inner, 2)
            out: List[Optional[bytes]] = []
            for w in wanted:
                off, nb = int(index[w, 0]), int(index[w, 1])
                if off == _MISSING and nb == _MISSING:
                    out.append(None)
                    continue
                f.seek(off)
                out.append(f.read(nb))
        return out

    def read(self, lo: Optional[Sequence[int]] = None, hi: Optional[Sequence[int]] = None) -> np.ndarray:
        nd = len(self.shape)
        lo = [0] * nd if lo is None else [int(x) for x in lo]
        hi = list(self.shape) if hi is None else [int(x) for x in hi]
        out = np.full([h - l for l, h in zip(lo, hi)], self.fill, dtype=self.np_dtype)
        if nd == 0 or any(h <= l for l, h in zip(lo, hi)):
            if nd == 0:
                parts = self._collect([()], lo, hi)
                for _, _, arr in parts:
                    return arr.reshape(()).copy()
            return out
        shard_idxs = list(itertools.product(*[range(l // c, (h - 1) // c + 1) for l, h, c in zip(lo, hi, self.chunks)]))
        for origin, shape, arr in self._collect(shard_idxs, lo, hi):
            src = tuple(slice(max(l, o) - o, min(h, o + s) - o) for l, h, o, s in zip(lo, hi, origin, shape))
            dst = tuple(slice(max(l, o) - l, min(h, o + s) - l) for l, h, o, s in zip(lo, hi, origin, shape))
            out[dst] = arr[src]
        return out

    def _collect(self, shard_idxs, lo, hi):
        """Yield ``(origin, shape, array)`` for every stored (inner) chunk that overlaps ``[lo, hi)``."""
        todo: List[Tuple[Tuple[int, ...], List[int]]] = []  # (origin, shape) per blob
        blobs: List[bytes] = []
        for sidx in shard_idxs:
            key = self._key(tuple(sidx))
            s_origin = [i * c for i, c in zip(sidx, self.chunks)]
            if self.inner is None:
                try:
                    with self.fs.open(key, "rb") as f:
                        blobs.append(f.read())
                    todo.append((tuple(s_origin), list(self.chunks)))
                except FileNotFoundError:
                    pass
                continue
            per = [o // i for o, i in zip(self.chunks, self.inner)]
            ranges = []
            for l, h, so, ic, p in zip(lo, hi, s_origin, self.inner, per):
                a = max(l, so) - so
                b = min(h, so + ic * p) - so
                ranges.append(range(a // ic, (b - 1) // ic + 1))
            inner_idxs = list(itertools.product(*ranges))
            linear = [int(np.ravel_multi_index(ii, per)) for ii in inner_idxs]
            for ii, blob in zip(inner_idxs, self._read_shard_parts(key, linear)):
                if blob is None:
                    continue
                blobs.append(blob)
                todo.append((tuple(so + i * ic for so, i, ic in zip(s_origin, ii, self.inner)), list(self.inner)))
        if not blobs:
            return
        same = {self._chunk_elems(shape) for _, shape in todo}
        decoded = self.pipe.decode_many(blobs, expect=same.pop() * self.np_dtype.itemsize if len(same) == 1 else None)
        for (origin, shape), d in zip(todo, decoded):
            n = self._chunk_elems(shape) * self.np_dtype.itemsize
            if d.nbytes != n:
                raise ValueError(f"{self.path}: a chunk decoded to {d.nbytes} bytes, expected {n}")
            yield origin, shape, d.view(self.np_dtype).reshape(shape)

    def read_tensor(self, lo=None, hi=None):
        from .zarr_array import _numpy_to_torch

        return _numpy_to_torch(self.read(lo, hi), self.dtype_str)

    # -- this class does not write --------------------------------------------------------------------------------------
    def write(self, *a, **k):
        raise NotImplementedError("zarr v3 arrays are read-only here; new caches are written as zarr v2")

    write_tensor = resize = write
