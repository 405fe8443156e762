"""Minimal zarr-v2 array over fsspec: the on-disk array format of checkpoints and of the token cache.

A checkpoint leaf written by the reference is one TensorStore ``zarr`` array: a directory with a ``.zarray`` JSON
(``zarr_format: 2``, C order, ``dimension_separator: "."``, ``compressor: {"id": "zstd"}``, chunk shape = the writer's
per-device shard shape) and one file per chunk named by its dot-separated chunk index
(src/levanter/tensorstore_serialization.py:36-112 through JAX's array serialisation).  This class reads arrays with any
chunk grid and the ``zstd`` / ``gzip`` / ``null`` compressors, and writes zstd (or uncompressed when libzstd is
absent) chunks through the parallel C++ codec in ``ops/csrc/chunk_codec.cpp``.  ``bfloat16`` uses TensorStore's dtype name.
"""
from __future__ import annotations

import ctypes
import itertools
import json
import os
import threading
import time
import math
import zlib
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import fsspec
import numpy as np
import torch
from fsspec.core import url_to_fs

_NP_TO_ZARR = {
    np.dtype("float32"): "<f4", np.dtype("float64"): "<f8", np.dtype("float16"): "<f2",
    np.dtype("int64"): "<i8", np.dtype("int32"): "<i4", np.dtype("int16"): "<i2", np.dtype("int8"): "|i1",
    np.dtype("uint64"): "<u8", np.dtype("uint32"): "<u4", np.dtype("uint16"): "<u2", np.dtype("uint8"): "|u1",
    np.dtype("bool"): "|b1",
}
_ZARR_TO_NP = {v: k for k, v in _NP_TO_ZARR.items()}
_ZARR_TO_NP.update({"float32": np.dtype("float32"), "float64": np.dtype("float64"), "float16": np.dtype("float16"),
                    "int64": np.dtype("int64"), "int32": np.dtype("int32"), "int16": np.dtype("int16"), "int8": np.dtype("int8"),
                    "uint64": np.dtype("uint64"), "uint32": np.dtype("uint32"), "uint16": np.dtype("uint16"),
                    "uint8": np.dtype("uint8"), "bool": np.dtype("bool")})
BF16 = "bfloat16"


# ------------------------------------------------------------------------------------------------ codec
class _Codec:
    def __init__(self):
        self._lib = None
        self._tried = False

    def lib(self):
        if not self._tried:
            self._tried = True
            try:
                from ..ops import lib as L

                l = L.load()
                l.lvb_zstd_available.restype = ctypes.c_int
                if l.lvb_zstd_available():
                    l.lvb_zstd_bound.restype = ctypes.c_longlong
                    l.lvb_zstd_bound.argtypes = [ctypes.c_longlong]
                    l.lvb_zstd_frame_size.restype = ctypes.c_longlong
                    l.lvb_zstd_frame_size.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
                    self._lib = l
            except Exception:
                self._lib = None
        return self._lib

    @property
    def has_zstd(self) -> bool:
        return self.lib() is not None

    def compress_many(self, bufs: List[np.ndarray], level: int = 1, threads: int = 8) -> List[bytes]:
        l = self.lib()
        n = len(bufs)
        if n == 0:
            return []
        srcs = [np.ascontiguousarray(b).view(np.uint8).reshape(-1) for b in bufs]
        caps = [int(l.lvb_zstd_bound(s.nbytes)) for s in srcs]
        dsts = [np.empty(c, dtype=np.uint8) for c in caps]
        P = ctypes.c_void_p * n
        LL = ctypes.c_longlong * n
        out_len = LL()
        rc = l.lvb_zstd_compress_many(n, P(*[s.ctypes.data for s in srcs]), LL(*[s.nbytes for s in srcs]),
                                      P(*[d.ctypes.data for d in dsts]), LL(*caps), out_len, level, threads)
        if rc != 0:
            raise RuntimeError(f"zstd compression failed ({rc})")
        return [d[:out_len[i]].tobytes() for i, d in enumerate(dsts)]

    def decompress_many(self, blobs: List[bytes], sizes: List[int], threads: int = 8) -> List[np.ndarray]:
        l = self.lib()
        n = len(blobs)
        if n == 0:
            return []
        srcs = [np.frombuffer(b, dtype=np.uint8) for b in blobs]
        dsts = [np.empty(s, dtype=np.uint8) for s in sizes]
        P = ctypes.c_void_p * n
        LL = ctypes.c_longlong * n
        out_len = LL()
        rc = l.lvb_zstd_decompress_many(n, P(*[s.ctypes.data for s in srcs]), LL(*[s.nbytes for s in srcs]),
                                        P(*[d.ctypes.data for d in dsts]), LL(*sizes), out_len, threads)
        if rc != 0:
            raise RuntimeError(f"zstd decompression failed ({rc})")
        return dsts


CODEC = _Codec()


def _torch_to_numpy(t: torch.Tensor) -> Tuple[np.ndarray, str]:
    t = t.detach()
    if t.device.type != "cpu":
        t = t.cpu()
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), BF16
    a = t.numpy()
    return a, _NP_TO_ZARR[a.dtype]


def _numpy_to_torch(a: np.ndarray, dtype_str: str) -> torch.Tensor:
    if dtype_str == BF16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(a))


def _write_json_atomically(fs, path: str, obj) -> None:
    """Readers (a trainer reading a cache that is still being built) must never see a half-written metadata file: write a
    sibling and rename it over the target; file systems without rename fall back to a plain write."""
    tmp = f"{path}.tmp{os.getpid()}"
    with fs.open(tmp, "w") as f:
        json.dump(obj, f, indent=1)
    try:
        fs.mv(tmp, path)
    except Exception:  # noqa: BLE001
        with fs.open(path, "w") as f:
            json.dump(obj, f, indent=1)
        try:
            fs.rm(tmp)
        except Exception:  # noqa: BLE001
            pass


class ZarrArray:
    """One zarr-v2 array stored under ``path`` (any fsspec URL)."""

    def __init__(self, path: str, meta: dict):
        self.path = path.rstrip("/")
        self.fs, self.root = url_to_fs(self.path)
        self.meta = meta
        self.shape: Tuple[int, ...] = tuple(meta["shape"])
        self.chunks: Tuple[int, ...] = tuple(meta["chunks"])
        self.dtype_str: str = meta["dtype"]
        self.np_dtype = np.dtype("uint16") if self.dtype_str == BF16 else _ZARR_TO_NP[self.dtype_str]
        comp = meta.get("compressor")
        self.compressor = None if comp is None else comp.get("id")
        self.level = 1 if comp is None else int(comp.get("level", 1))
        self.sep = meta.get("dimension_separator", ".")
        self.fill = meta.get("fill_value", 0) or 0
        if meta.get("order", "C") != "C":
            raise NotImplementedError("only C-order zarr arrays are supported")
        if meta.get("filters"):
            raise NotImplementedError("zarr filters are not supported")

    # -- construction ------------------------------------------------------------------------------------------
    @staticmethod
    def create(path: str, shape: Sequence[int], chunks: Sequence[int], dtype: Union[str, np.dtype, torch.dtype],
               compressor: Optional[str] = "zstd", level: int = 1, overwrite: bool = True) -> "ZarrArray":
        if isinstance(dtype, torch.dtype):
            dtype_str = BF16 if dtype == torch.bfloat16 else _NP_TO_ZARR[np.dtype(str(dtype).replace("torch.", ""))]
        elif isinstance(dtype, str) and (dtype == BF16 or dtype in _ZARR_TO_NP):
            dtype_str = dtype if dtype == BF16 or dtype.startswith(("<", "|", ">")) else _NP_TO_ZARR[_ZARR_TO_NP[dtype]]
        else:
            dtype_str = _NP_TO_ZARR[np.dtype(dtype)]
        if compressor == "zstd" and not CODEC.has_zstd:
            compressor = None
        shape = [int(s) for s in shape]
        chunks = [max(1, int(c)) for c in chunks] if len(shape) else []
        meta = {
            "chunks": chunks, "compressor": None if compressor is None else {"id": compressor, "level": level},
            "dimension_separator": ".", "dtype": dtype_str, "fill_value": None, "filters": None, "order": "C",
            "shape": shape, "zarr_format": 2,
        }
        fs, root = url_to_fs(path.rstrip("/"))
        if overwrite and fs.exists(root):
            fs.rm(root, recursive=True)
        fs.makedirs(root, exist_ok=True)
        _write_json_atomically(fs, f"{root}/.zarray", meta)
        return ZarrArray(path, meta)

    @staticmethod
    def open(path: str) -> "ZarrArray":
        fs, root = url_to_fs(path.rstrip("/"))
        if not fs.exists(f"{root}/.zarray") and fs.exists(f"{root}/zarr.json"):
            from .zarr3_array import Zarr3Array  # an array written by the reference (zarr v3, sharded, blosc): read-only

            return Zarr3Array.open(path)
        meta = None
        for attempt in range(50):  # a writer on a file system without atomic rename may be in the middle of rewriting the file
            try:
                with fs.open(f"{root}/.zarray", "r") as f:
                    meta = json.load(f)
                break
            except json.JSONDecodeError:
                if attempt == 49:
                    raise
                time.sleep(0.01)
        if meta.get("zarr_format") != 2:
            raise NotImplementedError(f"zarr_format {meta.get('zarr_format')} is not supported")
        return ZarrArray(path, meta)

    @staticmethod
    def exists(path: str) -> bool:
        fs, root = url_to_fs(path.rstrip("/"))
        return fs.exists(f"{root}/.zarray") or fs.exists(f"{root}/zarr.json")

    def _write_chunk(self, key: str, blob: bytes) -> None:
        """Chunk files are replaced, never rewritten in place: a concurrent reader sees the old chunk or the new one."""
        tmp = f"{key}.tmp{os.getpid()}_{threading.get_ident()}"
        with self.fs.open(tmp, "wb") as f:
            f.write(blob)
        try:
            self.fs.mv(tmp, key)
        except Exception:  # noqa: BLE001  (no rename on this file system)
            with self.fs.open(key, "wb") as f:
                f.write(blob)
            try:
                self.fs.rm(tmp)
            except Exception:  # noqa: BLE001
                pass

    def _write_meta(self):
        self.meta["shape"] = list(self.shape)
        _write_json_atomically(self.fs, f"{self.root}/.zarray", self.meta)

    # -- chunk helpers -----------------------------------------------------------------------------------------
    def _chunk_key(self, idx: Tuple[int, ...]) -> str:
        return f"{self.root}/" + (self.sep.join(str(i) for i in idx) if idx else "0")

    def _grid(self, lo: Sequence[int], hi: Sequence[int]) -> Iterable[Tuple[int, ...]]:
        ranges = [range(l // c, (h - 1) // c + 1) if h > l else range(0) for l, h, c in zip(lo, hi, self.chunks)]
        return itertools.product(*ranges)

    def _chunk_nbytes(self) -> int:
        return int(np.prod(self.chunks, dtype=np.int64)) * self.np_dtype.itemsize if self.chunks else self.np_dtype.itemsize

    def _decode(self, blobs: List[Optional[bytes]]) -> List[Optional[np.ndarray]]:
        n = self._chunk_nbytes()
        present = [(i, b) for i, b in enumerate(blobs) if b is not None]
        out: List[Optional[np.ndarray]] = [None] * len(blobs)
        if not present:
            return out
        if self.compressor is None:
            for i, b in present:
                out[i] = np.frombuffer(b, dtype=np.uint8)
        elif self.compressor == "zstd":
            if not CODEC.has_zstd:
                raise RuntimeError("this array is zstd-compressed but libzstd could not be loaded")
            dec = CODEC.decompress_many([b for _, b in present], [n] * len(present))
            for (i, _), d in zip(present, dec):
                out[i] = d
        elif self.compressor in ("gzip", "zlib"):
            for i, b in present:
                out[i] = np.frombuffer(zlib.decompress(b, 15 + 32), dtype=np.uint8)
        else:
            raise NotImplementedError(f"compressor {self.compressor!r} is not supported")
        return out

    def _encode(self, arrays: List[np.ndarray]) -> List[bytes]:
        if self.compressor is None:
            return [np.ascontiguousarray(a).tobytes() for a in arrays]
        if self.compressor == "zstd":
            return CODEC.compress_many(arrays, self.level)
        if self.compressor in ("gzip", "zlib"):
            return [zlib.compress(np.ascontiguousarray(a).tobytes(), self.level) for a in arrays]
        raise NotImplementedError(self.compressor)

    def _read_blob(self, key: str) -> Optional[bytes]:
        try:
            with self.fs.open(key, "rb") as f:
                return f.read()
        except FileNotFoundError:
            return None

    # -- public I/O --------------------------------------------------------------------------------------------
    def read(self, lo: Optional[Sequence[int]] = None, hi: Optional[Sequence[int]] = None) -> np.ndarray:
        """Region ``[lo, hi)`` as a numpy array (bf16 comes back as uint16 bit patterns)."""
        nd = len(self.shape)
        if nd == 0:
            blob = self._read_blob(self._chunk_key(()))
            dec = self._decode([blob])[0]
            if dec is None:
                return np.full((), self.fill, dtype=self.np_dtype)
            return dec.view(self.np_dtype)[:1].reshape(()).copy()
        lo = [0] * nd if lo is None else list(lo)
        hi = list(self.shape) if hi is None else list(hi)
        out = np.full([h - l for l, h in zip(lo, hi)], self.fill, dtype=self.np_dtype)
        idxs = list(self._grid(lo, hi))
        blobs = [self._read_blob(self._chunk_key(i)) for i in idxs]
        decoded = self._decode(blobs)
        for idx, d in zip(idxs, decoded):
            if d is None:
                continue
            chunk = d.view(self.np_dtype).reshape(self.chunks)
            c_lo = [i * c for i, c in zip(idx, self.chunks)]
            src = tuple(slice(max(l, cl) - cl, min(h, cl + c) - cl) for l, h, cl, c in zip(lo, hi, c_lo, self.chunks))
            dst = tuple(slice(max(l, cl) - l, min(h, cl + c) - l) for l, h, cl, c in zip(lo, hi, c_lo, self.chunks))
            out[dst] = chunk[src]
        return out

    def write(self, data: np.ndarray, lo: Optional[Sequence[int]] = None) -> None:
        """Write ``data`` at offset ``lo``.  Chunks only partly covered are read, patched and rewritten."""
        nd = len(self.shape)
        data = np.asarray(data)
        if data.dtype != self.np_dtype:
            data = data.astype(self.np_dtype)
        if nd == 0:
            blob = self._encode([data.reshape(1)])[0]
            self._write_chunk(self._chunk_key(()), blob)
            return
        lo = [0] * nd if lo is None else list(lo)
        hi = [l + s for l, s in zip(lo, data.shape)]
        if any(h > s for h, s in zip(hi, self.shape)):
            raise ValueError(f"write region {lo}..{hi} exceeds array shape {self.shape}")
        idxs = list(self._grid(lo, hi))
        chunks_out: List[np.ndarray] = []
        for idx in idxs:
            c_lo = [i * c for i, c in zip(idx, self.chunks)]
            full = all(l <= cl and h >= min(cl + c, s) for l, h, cl, c, s in zip(lo, hi, c_lo, self.chunks, self.shape))
            if full and all(cl + c <= s for cl, c, s in zip(c_lo, self.chunks, self.shape)):
                src = tuple(slice(cl - l, cl - l + c) for l, cl, c in zip(lo, c_lo, self.chunks))
                chunk = np.ascontiguousarray(data[src])
            else:
                blob = None if full else self._read_blob(self._chunk_key(idx))
                dec = self._decode([blob])[0]
                chunk = (dec.view(self.np_dtype).reshape(self.chunks).copy() if dec is not None
                         else np.full(self.chunks, self.fill, dtype=self.np_dtype))
                src = tuple(slice(max(l, cl) - l, min(h, cl + c) - l) for l, h, cl, c in zip(lo, hi, c_lo, self.chunks))
                dst = tuple(slice(max(l, cl) - cl, min(h, cl + c) - cl) for l, h, cl, c in zip(lo, hi, c_lo, self.chunks))
                chunk[dst] = data[src]
            chunks_out.append(chunk)
        blobs = self._encode(chunks_out)
        for idx, blob in zip(idxs, blobs):
            self._write_chunk(self._chunk_key(idx), blob)

    def resize(self, new_shape: Sequence[int]) -> None:
        self.shape = tuple(int(s) for s in new_shape)
        self._write_meta()

    # -- torch convenience -------------------------------------------------------------------------------------
    def read_tensor(self, lo=None, hi=None) -> torch.Tensor:
        return _numpy_to_torch(self.read(lo, hi), self.dtype_str)

    def write_tensor(self, t: torch.Tensor, lo=None) -> None:
        a, ds = _torch_to_numpy(t)
        if ds != self.dtype_str and not (ds == BF16 and self.dtype_str == BF16):
            # dtype conversion on write (e.g. python scalars saved as 0-d arrays)
            if self.dtype_str == BF16:
                a, _ = _torch_to_numpy(t.to(torch.bfloat16))
            else:
                a = (t.float().numpy() if ds == BF16 else a).astype(self.np_dtype)
        self.write(a, lo)


def default_chunks(shape: Sequence[int], itemsize: int, target_bytes: int = 64 << 20) -> List[int]:
    """Chunk shape that cuts the leading dimension so a chunk is at most about ``target_bytes``."""
    shape = list(shape)
    if not shape:
        return []
    row = int(np.prod(shape[1:], dtype=np.int64)) * itemsize if len(shape) > 1 else itemsize
    rows = max(1, min(shape[0], target_bytes // max(row, 1)))
    return [rows] + shape[1:]
