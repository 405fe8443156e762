"""Write a finished token cache in the layout the reference reads: zarr v3 arrays, ``sharding_indexed`` shards of
blosc-compressed inner chunks (src/levanter/store/jagged_array.py:605-635), beside a copy of the ledger.

This framework builds and reads caches as zarr v2 + zstd (appends touch one small chunk file); the reference's layout packs
512 inner chunks of 256 Ki elements into every shard file, which suits a one-pass export of a finished cache, not appends.
Each array is streamed shard by shard: inner chunks are encoded as blosc frames (byte shuffle; the payload compressed as one
LZ4 block through pyarrow's codec, or a zstd frame through the native codec when pyarrow is absent; incompressible chunks are
stored), appended to the shard file as they are produced, and the ``(offset, nbytes)`` index with its CRC-32C closes the
file.  Memory stays at one inner chunk.  ``zarr.json`` carries the reference's metadata: nominal first dimension ``2^54``,
chunk grid = shard shape, little-endian ``bytes`` + ``blosc`` inside ``sharding_indexed``, index at the end.

The writer follows the zarr v3, sharding and blosc specifications and is checked by reading its output back with
:mod:`zarr3_array` (whose decoders are checked against independent encoders); it has not been read by TensorStore here.

``python -m levanter_b200.store.zarr3_export <cache_dir> <out_dir>`` exports every field of a cache."""
from __future__ import annotations

import json
import os
import shutil
import struct
import sys
from typing import List, Optional, Sequence

import numpy as np

from .jagged_array import DEFAULT_CHUNK_SIZE, DEFAULT_WRITE_CHUNK_SIZE
from .zarr3_array import crc32c
from .zarr_array import CODEC, ZarrArray

NOMINAL_ROWS = 2 ** 54
_MISSING = struct.pack("<QQ", 2 ** 64 - 1, 2 ** 64 - 1)
_V3_NAMES = {"uint16": "uint16", "bfloat16": "bfloat16"}


def _compress(raw: bytes, cname: str, level: int) -> bytes:
    if cname == "lz4":
        import pyarrow as pa

        return pa.compress(raw, codec="lz4_raw", asbytes=True)
    return CODEC.compress_many([np.frombuffer(raw, dtype=np.uint8)], level)[0]


def blosc_frame(chunk: np.ndarray, cname: str = "lz4", level: int = 5) -> bytes:
    """One blosc (version 1) frame holding ``chunk``: a single block, byte-shuffled by the element size, not split."""
    raw = np.ascontiguousarray(chunk)
    typesize, nbytes = raw.dtype.itemsize, raw.nbytes
    body = raw.view(np.uint8).reshape(-1, typesize).T.copy().tobytes() if typesize > 1 else raw.tobytes()
    flags = (1 if typesize > 1 else 0) | 0x10 | ({"lz4": 1, "zstd": 4}[cname] << 5)
    comp = _compress(body, cname, level)
    if len(comp) >= nbytes:
        comp = body  # a stream whose stored size equals its raw size is read back as is
    total = 16 + 4 + 4 + len(comp)
    return struct.pack("<BBBBIII", 2, 1, flags, typesize, nbytes, nbytes, total) + struct.pack("<II", 20, len(comp)) + comp


def _metadata(shape_tail: Sequence[int], dtype_name: str, shard_rows: int, inner_rows: int, cname: str, level: int, typesize: int) -> dict:
    return {
        "zarr_format": 3, "node_type": "array", "shape": [NOMINAL_ROWS, *shape_tail], "data_type": dtype_name,
        "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": [shard_rows, *shape_tail]}},
        "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
        "fill_value": 0, "attributes": {},
        "codecs": [{"name": "sharding_indexed", "configuration": {
            "chunk_shape": [inner_rows, *shape_tail],
            "codecs": [{"name": "bytes", "configuration": {"endian": "little"}},
                       {"name": "blosc", "configuration": {"cname": cname, "clevel": level, "shuffle": "shuffle" if typesize > 1 else "noshuffle",
                                                           "typesize": typesize, "blocksize": 0}}],
            "index_codecs": [{"name": "bytes", "configuration": {"endian": "little"}}, {"name": "crc32c"}],
            "index_location": "end"}}],
    }


def export_array(src, dst_path: str, rows: int, *, shard_rows: int = DEFAULT_WRITE_CHUNK_SIZE, inner_rows: int = DEFAULT_CHUNK_SIZE,
                 cname: Optional[str] = None, level: int = 5) -> None:
    """Rows ``[0, rows)`` of ``src`` (anything with ``read(lo, hi)``, ``shape``, ``np_dtype``) as a sharded zarr v3 array."""
    if shard_rows % inner_rows:
        raise ValueError("the shard must hold a whole number of inner chunks")
    if cname is None:
        try:
            import pyarrow  # noqa: F401

            cname = "lz4"
        except ImportError:
            cname = "zstd"
    tail = [int(s) for s in src.shape[1:]]
    dt = np.dtype(src.np_dtype)
    name = getattr(src, "dtype_str", None)
    dtype_name = "bfloat16" if name == "bfloat16" else dt.name
    os.makedirs(dst_path, exist_ok=True)
    per = shard_rows // inner_rows
    key_tail = ["0"] * len(tail)
    for s0 in range(0, max(rows, 0), shard_rows):
        key = os.path.join(dst_path, "c", str(s0 // shard_rows), *key_tail)
        os.makedirs(os.path.dirname(key), exist_ok=True)
        index: List[bytes] = []
        pos = 0
        with open(key + ".tmp", "wb") as f:
            for i in range(per):
                lo = s0 + i * inner_rows
                if lo >= rows:
                    index.append(_MISSING)
                    continue
                hi = min(lo + inner_rows, rows)
                chunk = np.zeros([inner_rows, *tail], dtype=dt)
                chunk[: hi - lo] = src.read([lo] + [0] * len(tail), [hi] + tail)
                frame = blosc_frame(chunk, cname, level)
                f.write(frame)
                index.append(struct.pack("<QQ", pos, len(frame)))
                pos += len(frame)
            raw = b"".join(index)
            f.write(raw + struct.pack("<I", crc32c(raw)))
        os.replace(key + ".tmp", key)
    with open(os.path.join(dst_path, "zarr.json"), "w") as f:
        json.dump(_metadata(tail, dtype_name, shard_rows, inner_rows, cname, level, dt.itemsize), f)


def export_cache(cache_dir: str, out_dir: str, **kw) -> List[str]:
    """Every jagged field under ``cache_dir`` (directories holding ``offsets`` and ``data``) plus the ledger; returns the
    fields written."""
    done = []
    for root, dirs, _ in os.walk(cache_dir):
        if "offsets" in dirs and "data" in dirs:
            rel = os.path.relpath(root, cache_dir)
            offsets = ZarrArray.open(os.path.join(root, "offsets"))
            n = int(offsets.read([0], [1])[0])
            size = 0 if n == 0 else int(offsets.read([n], [n + 1])[0])
            dst = os.path.join(out_dir, rel) if rel != "." else out_dir
            export_array(offsets, os.path.join(dst, "offsets"), n + 1, **kw)
            export_array(ZarrArray.open(os.path.join(root, "data")), os.path.join(dst, "data"), size, **kw)
            if "shapes" in dirs:
                export_array(ZarrArray.open(os.path.join(root, "shapes")), os.path.join(dst, "shapes"), n, **kw)
            done.append(rel)
            dirs[:] = [d for d in dirs if d not in ("offsets", "data", "shapes")]
    for name in ("shard_ledger.json",):
        p = os.path.join(cache_dir, name)
        if os.path.exists(p):
            os.makedirs(out_dir, exist_ok=True)
            shutil.copyfile(p, os.path.join(out_dir, name))
    return done


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if len(args) != 2:
        print("usage: python -m levanter_b200.store.zarr3_export <cache_dir> <out_dir>", file=sys.stderr)
        return 2
    fields = export_cache(args[0], args[1])
    print(f"exported {len(fields)} field(s): {', '.join(fields)}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
