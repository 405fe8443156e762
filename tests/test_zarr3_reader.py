"""Reading the reference's cache arrays: zarr v3, ``sharding_indexed`` shards of blosc-compressed inner chunks.

No zarr / blosc / tensorstore library is installed, so the test writes the bytes itself from the formats' specifications:
blosc frames (header, block offsets, split streams, byte shuffle) around LZ4 blocks and zstd frames produced by pyarrow's
codecs (an encoder this framework does not share), shard files with their index and CRC-32C, and ``zarr.json``."""
import json
import math
import os
import struct

import numpy as np
import pyarrow as pa
import pytest

from levanter_b200.store.zarr3_array import Zarr3Array, blosc_decompress_many, crc32c
from levanter_b200.store.zarr_array import ZarrArray


def _blosc_frame(data: bytes, typesize: int, blocksize: int, *, shuffle=True, codec="lz4", split=True, stored=False) -> bytes:
    nbytes = len(data)
    flags = (1 if shuffle else 0) | ((0 if split else 1) << 4) | ({"lz4": 1, "zstd": 4}[codec] << 5)
    if stored:
        return struct.pack("<BBBBIII", 2, 1, flags | 2, typesize, nbytes, blocksize, 16 + nbytes) + data
    nblocks = math.ceil(nbytes / blocksize)
    bodies = []
    for i in range(nblocks):
        b = data[i * blocksize:(i + 1) * blocksize]
        leftover = len(b) != blocksize
        if shuffle and typesize > 1:
            nel = len(b) // typesize
            b = np.frombuffer(b[:nel * typesize], np.uint8).reshape(nel, typesize).T.copy().tobytes() + b[nel * typesize:]
        nsplits = typesize if (split and typesize <= 16 and blocksize // typesize >= 128 and not leftover) else 1
        ne = len(b) // nsplits
        out = b""
        for s in range(nsplits):
            stream = b[s * ne:(s + 1) * ne]
            c = pa.compress(stream, codec="lz4_raw" if codec == "lz4" else "zstd", asbytes=True)
            out += struct.pack("<I", ne) + stream if len(c) >= ne else struct.pack("<I", len(c)) + c
        bodies.append(out)
    starts, pos = [], 16 + 4 * nblocks
    for b in bodies:
        starts.append(pos)
        pos += len(b)
    return struct.pack("<BBBBIII", 2, 1, flags, typesize, nbytes, blocksize, pos) + struct.pack(f"<{nblocks}I", *starts) + b"".join(bodies)


def test_crc32c_known_vector():
    assert crc32c(b"123456789") == 0xE3069283
    assert crc32c(b"") == 0


@pytest.mark.parametrize("codec", ["lz4", "zstd"])
@pytest.mark.parametrize("typesize,blocksize,n", [(4, 4096, 10000), (8, 1024, 1024), (2, 512, 3001), (1, 256, 1000), (4, 64, 300)])
def test_blosc_frames_decode(codec, typesize, blocksize, n):
    rng = np.random.default_rng(n)
    data = (rng.integers(0, 50, n) * 3).astype({1: np.uint8, 2: np.uint16, 4: np.int32, 8: np.int64}[typesize]).tobytes()
    data = data[: len(data) - (len(data) % 3 if typesize > 1 and n == 3001 else 0)]  # a tail shorter than an element
    frames = [_blosc_frame(data, typesize, blocksize, codec=codec),
              _blosc_frame(data, typesize, blocksize, codec=codec, shuffle=False),
              _blosc_frame(data, typesize, blocksize, codec=codec, split=False),
              _blosc_frame(data, typesize, blocksize, codec=codec, stored=True)]
    for got in blosc_decompress_many(frames):
        assert got.tobytes() == data
    with pytest.raises(ValueError):
        blosc_decompress_many([frames[0][:40]])


def _write_sharded(path, arr: np.ndarray, nominal_shape, shard, inner, *, skip=(), codec="lz4"):
    os.makedirs(path, exist_ok=True)
    meta = {"zarr_format": 3, "node_type": "array", "shape": list(nominal_shape), "data_type": str(arr.dtype),
            "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": list(shard)}},
            "chunk_key_encoding": {"name": "default"}, "fill_value": 0, "attributes": {},
            "codecs": [{"name": "sharding_indexed", "configuration": {
                "chunk_shape": list(inner),
                "codecs": [{"name": "bytes", "configuration": {"endian": "little"}},
                           {"name": "blosc", "configuration": {"cname": codec, "clevel": 5, "shuffle": "shuffle",
                                                               "typesize": arr.dtype.itemsize, "blocksize": 0}}],
                "index_codecs": [{"name": "bytes", "configuration": {"endian": "little"}}, {"name": "crc32c"}],
                "index_location": "end"}}]}
    with open(os.path.join(path, "zarr.json"), "w") as f:
        json.dump(meta, f)
    per = [s // i for s, i in zip(shard, inner)]
    n_shards = [math.ceil(a / s) for a, s in zip(arr.shape, shard)]
    for sidx in np.ndindex(*n_shards):
        body, index = b"", []
        for iidx in np.ndindex(*per):
            lo = [si * s + ii * i for si, s, ii, i in zip(sidx, shard, iidx, inner)]
            if any(l >= a for l, a in zip(lo, arr.shape)) or (tuple(sidx), tuple(iidx)) in skip:
                index.append((2 ** 64 - 1, 2 ** 64 - 1))
                continue
            chunk = np.zeros(inner, dtype=arr.dtype)
            sl = tuple(slice(l, min(l + i, a)) for l, i, a in zip(lo, inner, arr.shape))
            part = arr[sl]
            chunk[tuple(slice(0, p) for p in part.shape)] = part
            frame = _blosc_frame(chunk.tobytes(), arr.dtype.itemsize, 2048, codec=codec)
            index.append((len(body), len(frame)))
            body += frame
        raw = b"".join(struct.pack("<QQ", o, n) for o, n in index)
        key = os.path.join(path, "c", *[str(i) for i in sidx])
        os.makedirs(os.path.dirname(key), exist_ok=True)
        with open(key, "wb") as f:
            f.write(body + raw + struct.pack("<I", crc32c(raw)))


def test_sharded_blosc_array_reads_regions_and_missing_chunks(tmp_path):
    rng = np.random.default_rng(0)
    arr = rng.integers(0, 1000, (5000, 3), dtype=np.int32)
    p = str(tmp_path / "a")
    _write_sharded(p, arr, (2 ** 54, 3), shard=(2048, 3), inner=(512, 3), skip={((1,  0), (2, 0))})
    z = ZarrArray.open(p)  # the common entry point recognises the v3 metadata
    assert isinstance(z, Zarr3Array) and z.shape == [2 ** 54, 3] and z.chunks == [2048, 3] and z.inner == [512, 3]
    want = arr.copy()
    want[2048 + 1024: 2048 + 1536] = 0  # the inner chunk that was never written reads as the fill value
    for lo, hi in [(0, 5000), (100, 700), (2040, 2060), (3000, 3700), (4999, 5000), (5000, 5600)]:
        got = z.read([lo, 0], [hi, 3])
        ref = np.zeros((hi - lo, 3), np.int32)
        n = max(0, min(hi, 5000) - lo)
        ref[:n] = want[lo:lo + n]
        assert np.array_equal(got, ref), (lo, hi)
    assert np.array_equal(z.read([10, 1], [20, 2]), want[10:20, 1:2])
    with pytest.raises(NotImplementedError):
        z.write(np.zeros((1, 3), np.int32), [0, 0])
    # a flipped byte in the index is caught by its checksum
    shard = os.path.join(p, "c", "0", "0")
    raw = bytearray(open(shard, "rb").read())
    raw[-10] ^= 1
    open(shard, "wb").write(bytes(raw))
    with pytest.raises(ValueError):
        z.read([0, 0], [10, 3])


def test_jagged_store_opens_a_cache_in_the_reference_layout(tmp_path):
    """``offsets`` (``offsets[0]`` = number of rows, then the end of every row) and ``data`` as sharded zarr v3 arrays."""
    from levanter_b200.store.jagged_array import JaggedArrayStore

    rng = np.random.default_rng(1)
    rows = [rng.integers(0, 50000, int(n), dtype=np.int32) for n in rng.integers(1, 400, 300)]
    data = np.concatenate(rows)
    offsets = np.concatenate([[len(rows)], np.cumsum([len(r) for r in rows])]).astype(np.int64)
    _write_sharded(str(tmp_path / "offsets"), offsets, (2 ** 54,), shard=(1024,), inner=(256,), codec="lz4")
    _write_sharded(str(tmp_path / "data"), data, (2 ** 54,), shard=(16384,), inner=(4096,), codec="zstd")
    store = JaggedArrayStore.open(str(tmp_path), mode="r", dtype=np.int32)
    assert store.num_rows == 300 and store.data_size == len(data)
    for i in (0, 1, 17, 299):
        assert np.array_equal(store[i], rows[i])
    batch = store.get_batch_sync([5, 250, 6]) if hasattr(store, "get_batch_sync") else [store[j] for j in (5, 250, 6)]
    for got, j in zip(batch, (5, 250, 6)):
        assert np.array_equal(got, rows[j])


def test_tree_cache_loads_a_finished_cache_in_the_reference_layout(tmp_path):
    """A whole cache directory as the reference leaves it: ``shard_ledger.json`` plus ``<field>/{offsets,data}`` in zarr v3."""
    from levanter_b200.store.cache import TreeCache

    rng = np.random.default_rng(2)
    rows = [rng.integers(0, 32000, int(n), dtype=np.int32) for n in rng.integers(5, 200, 64)]
    data = np.concatenate(rows)
    offsets = np.concatenate([[len(rows)], np.cumsum([len(r) for r in rows])]).astype(np.int64)
    cache_dir = tmp_path / "cache" / "train"
    _write_sharded(str(cache_dir / "input_ids" / "offsets"), offsets, (2 ** 54,), shard=(1024,), inner=(256,))
    _write_sharded(str(cache_dir / "input_ids" / "data"), data, (2 ** 54,), shard=(8192,), inner=(2048,))
    ledger = {"total_num_rows": len(rows), "shard_rows": {"shard_0": len(rows)}, "is_finished": True, "finished_shards": ["shard_0"],
              "field_counts": {"input_ids": len(data)}, "metadata": {"preprocessor_metadata": {"tokenizer": "x"}}}
    with open(cache_dir / "shard_ledger.json", "w") as f:
        json.dump(ledger, f)
    cache = TreeCache.load(str(cache_dir), {"input_ids": np.zeros((0,), dtype=np.int32)})
    assert len(cache) == len(rows)
    got = cache.get_batch_sync([0, 63, 31])
    for g, j in zip(got, (0, 63, 31)):
        assert np.array_equal(g["input_ids"], rows[j])


def test_mutated_frames_are_rejected_or_decoded_but_never_trusted_for_sizes():
    """Bytes from a file are not trusted: a damaged frame is refused (or decodes to the declared size), and a frame that
    declares another size than its chunk is refused before anything is allocated for it."""
    import random

    rng = np.random.default_rng(3)
    data = (rng.integers(0, 50, 3000) * 3).astype(np.int32).tobytes()
    frames = [_blosc_frame(data, 4, 2048, codec=c, split=sp) for c in ("lz4", "zstd") for sp in (True, False)]
    random.seed(0)
    for _ in range(400):
        f = bytearray(random.choice(frames))
        for _ in range(random.randint(1, 4)):
            f[random.randrange(len(f))] = random.randrange(256)
        try:
            out = blosc_decompress_many([bytes(f)], expect=len(data))
            assert out[0].nbytes == len(data)
        except ValueError:
            pass
    big = bytearray(frames[0])
    big[4:8] = struct.pack("<I", 1 << 31)
    with pytest.raises(ValueError):
        blosc_decompress_many([bytes(big)], expect=len(data))


@pytest.mark.parametrize("cname", ["lz4", "zstd"])
def test_exported_cache_reads_back_through_the_v3_reader(tmp_path, cname):
    """Build a cache in this framework's layout, export it to the reference's, and read the export through every entry point."""
    from levanter_b200.store.cache import TreeCache
    from levanter_b200.store.jagged_array import JaggedArrayStore
    from levanter_b200.store.zarr3_export import blosc_frame, export_cache

    rng = np.random.default_rng(5)
    rows = [rng.integers(0, 32000, int(n), dtype=np.int32) for n in rng.integers(1, 300, 200)]
    src = tmp_path / "v2" / "input_ids"
    store = JaggedArrayStore.open(str(src), mode="w", dtype=np.int32)
    store.extend(rows)
    ledger = {"total_num_rows": len(rows), "shard_rows": {"s": len(rows)}, "is_finished": True, "finished_shards": ["s"],
              "field_counts": {}, "metadata": {"preprocessor_metadata": {}}}
    (tmp_path / "v2" / "shard_ledger.json").write_text(json.dumps(ledger))
    fields = export_cache(str(tmp_path / "v2"), str(tmp_path / "v3"), shard_rows=4096, inner_rows=512, cname=cname)
    assert fields == ["input_ids"]
    meta = json.load(open(tmp_path / "v3" / "input_ids" / "data" / "zarr.json"))
    assert meta["shape"] == [2 ** 54] and meta["codecs"][0]["name"] == "sharding_indexed"
    assert meta["codecs"][0]["configuration"]["codecs"][1]["configuration"]["cname"] == cname
    z = ZarrArray.open(str(tmp_path / "v3" / "input_ids" / "data"))
    assert isinstance(z, Zarr3Array)
    data = np.concatenate(rows)
    assert np.array_equal(z.read([0], [len(data)]), data)
    cache = TreeCache.load(str(tmp_path / "v3"), {"input_ids": np.zeros((0,), dtype=np.int32)})
    assert len(cache) == len(rows)
    for got, j in zip(cache.get_batch_sync([0, 199, 77]), (0, 199, 77)):
        assert np.array_equal(got["input_ids"], rows[j])
    # the frames are plain blosc: a stored (incompressible) chunk and a compressible one both decode
    noise = rng.integers(0, 2 ** 31, 1000, dtype=np.int64)
    for arr in (noise, np.zeros(1000, np.int64)):
        assert blosc_decompress_many([blosc_frame(arr, cname)])[0].tobytes() == arr.tobytes()


@pytest.mark.parametrize("codec,key_style", [("zstd", "default"), ("gzip", "v2"), ("none", "default")])
def test_plain_chunked_v3_arrays_with_other_codecs_and_key_encodings(tmp_path, codec, key_style):
    """Arrays without the sharding codec (how array checkpoints may be stored): one file per chunk, ``bytes`` + a compressor,
    either chunk-key encoding, a fill value for chunks that were never written."""
    import gzip

    rng = np.random.default_rng(7)
    arr = rng.standard_normal((70, 50)).astype(np.float32)
    p = tmp_path / "a"
    p.mkdir()
    codecs = [{"name": "bytes", "configuration": {"endian": "little"}}]
    if codec != "none":
        codecs.append({"name": codec, "configuration": {"level": 3}})
    enc = {"name": "default", "configuration": {"separator": "/"}} if key_style == "default" else {"name": "v2", "configuration": {"separator": "."}}
    meta = {"zarr_format": 3, "node_type": "array", "shape": [70, 50], "data_type": "float32",
            "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": [32, 32]}}, "chunk_key_encoding": enc,
            "fill_value": 1.5, "codecs": codecs, "attributes": {}}
    (p / "zarr.json").write_text(json.dumps(meta))
    for i in range(3):
        for j in range(2):
            if (i, j) == (2, 1):
                continue  # never written: reads as the fill value
            chunk = np.full((32, 32), 1.5, np.float32)
            part = arr[i * 32:(i + 1) * 32, j * 32:(j + 1) * 32]
            chunk[:part.shape[0], :part.shape[1]] = part
            raw = chunk.tobytes()
            blob = {"zstd": lambda b: pa.compress(b, codec="zstd", asbytes=True), "gzip": gzip.compress, "none": lambda b: b}[codec](raw)
            key = p / "c" / str(i) / str(j) if key_style == "default" else p / f"{i}.{j}"
            key.parent.mkdir(parents=True, exist_ok=True)
            key.write_bytes(blob)
    z = ZarrArray.open(str(p))
    want = arr.copy()
    want[64:, 32:] = 1.5
    assert np.array_equal(z.read(), want)
    assert np.array_equal(z.read([10, 20], [66, 45]), want[10:66, 20:45])
    t = z.read_tensor([0, 0], [4, 4])
    assert t.dtype.is_floating_point and t.shape == (4, 4)


def test_checkpoint_leaf_stored_as_a_v3_array_loads(tmp_path):
    """The checkpoint loader opens leaves through the same entry point, so a leaf written as a zarr v3 array (here: a stacked
    per-layer weight, bf16) loads, including the one-layer slice the loader takes from stacked arrays."""
    import torch

    from levanter_b200.store.zarr3_export import export_array
    from levanter_b200.tensorstore_serialization import _fs_path, read_leaf

    w = torch.randn(4, 6, 8).bfloat16()

    class Src:
        shape, np_dtype, dtype_str = list(w.shape), np.dtype("uint16"), "bfloat16"

        def read(self, lo, hi):
            return w.view(torch.int16).numpy().view(np.uint16)[tuple(slice(a, b) for a, b in zip(lo, hi))]

    p = _fs_path(str(tmp_path), "model.transformer.layers.stacked.weight")
    export_array(Src(), p, 4, shard_rows=4, inner_rows=2)
    meta = json.load(open(os.path.join(p, "zarr.json")))
    meta["shape"] = [4, 6, 8]  # a checkpoint array has its true shape, not the caches' nominal one
    json.dump(meta, open(os.path.join(p, "zarr.json"), "w"))
    got = read_leaf(str(tmp_path), "model.transformer.layers.stacked.weight")
    assert got.dtype == torch.bfloat16 and torch.equal(got, w)
    z = ZarrArray.open(p)
    assert torch.equal(z.read_tensor([2, 0, 0], [3, 6, 8])[0], w[2])
