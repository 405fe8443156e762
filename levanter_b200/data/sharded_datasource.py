"""Sharded sources of raw rows (src/levanter/data/sharded_datasource.py:53-630): named shards that can be reopened at a row,
so an interrupted cache build resumes mid-shard.  URL-backed sources cover jsonl(.gz/.zst), json, parquet and plain text."""
from __future__ import annotations

import abc
import io
import json
import os
from typing import Any, Callable, Dict, Generic, Iterator, List, Optional, Sequence, TypeVar

import numpy as np

from ..utils import fsspec_utils
from ._preprocessor import BatchProcessor, _BatchMapTransform, _canonicalize_batch, _CompositeBatchProcessor, _MapTransform
from .utils import batched

T = TypeVar("T")
T_co = TypeVar("T_co", covariant=True)
U = TypeVar("U")


class ShardedDataSource(Generic[T_co]):
    @property
    def shard_names(self) -> Sequence[str]:
        raise NotImplementedError

    @property
    def num_shards(self) -> int:
        return len(self.shard_names)

    def open_shard(self, shard_name: str) -> Iterator[T_co]:
        return self.open_shard_at_row(shard_name, 0)

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[T_co]:
        raise NotImplementedError

    def __iter__(self):
        for shard in self.shard_names:
            yield from self.open_shard(shard)

    def build_or_load_cache(self, path: str, *, await_finished: bool = True, monitors=None, options=None):
        """Materialise this (possibly mapped) source as a :class:`TreeCache` at ``path``."""
        from ..store.cache import CacheOptions, build_or_load_cache

        source, processor = _construct_composite_batch_processor(self)
        return build_or_load_cache(path, source, processor, await_finished=await_finished, monitors=monitors,
                                   options=options or CacheOptions.default())

    def map(self, fn: Callable[[T_co], U]) -> "ShardedDataSource[U]":
        return _MappedShardedDataSource(self, fn)

    def map_batches(self, fn, batch_size: int, *, num_cpus: int = 1, num_gpus: int = 0, output_exemplar=None, **resources):
        return _BatchMappedShardedDataSource(self, fn, batch_size, num_cpus=num_cpus, num_gpus=num_gpus,
                                             output_exemplar=output_exemplar, **resources)


def _mk_shard_name_mapping(urls: Sequence[str]) -> Dict[str, str]:
    """{shard name: url}: names are the urls minus their common prefix with dots replaced, as in the reference (:534-571),
    so ledgers written for the same url list agree."""
    urls = list(urls)
    common = os.path.dirname(urls[0]) if len(urls) == 1 else os.path.commonprefix(urls)
    expanded = [g for u in urls for g in fsspec_utils.expand_glob(u)]
    if urls and not expanded:
        raise ValueError(f"Could not expand any of the urls: {urls}")
    mapping: Dict[str, str] = {}
    missing = []
    for url in expanded:
        if not fsspec_utils.exists(url):
            missing.append(url)
            continue
        name = url[len(common):].lstrip("/") if common and url.startswith(common) else url
        name = name.replace(".", "_")
        if name in mapping:
            raise ValueError(f"Duplicate shard name {name}")
        mapping[name] = url
    if missing:
        raise FileNotFoundError("Could not find the following urls:\n  - " + "\n  - ".join(missing))
    return mapping


class UrlBackedShardedDataSource(ShardedDataSource[T_co], abc.ABC):
    def __init__(self, urls):
        self.urls = list(urls)
        self._mapping: Optional[Dict[str, str]] = None

    @property
    def _shard_name_to_url_mapping(self) -> Dict[str, str]:
        if self._mapping is None:
            self._mapping = _mk_shard_name_mapping(self.urls)
        return self._mapping

    @property
    def shard_names(self) -> Sequence[str]:
        return list(self._shard_name_to_url_mapping.keys())


def _open_text(url: str):
    import fsspec

    return fsspec.open(url, "rt", compression="infer", encoding="utf-8").open()


def _sniff_format_for_dataset(url: str) -> str:
    base = url
    for comp in (".gz", ".zst", ".zstd", ".bz2", ".xz"):
        if base.endswith(comp):
            base = base[: -len(comp)]
    for ext, fmt in ((".jsonl", "jsonl"), (".ndjson", "jsonl"), (".txt", "txt"), (".parquet", "parquet")):
        if base.endswith(ext):
            return fmt
    # ".json" is used for both one JSON document and one object per line, and a file without a known extension may be
    # either: look at the content.  "[" or "{" + newline starts a (pretty-printed) document, "{" + anything else a line.
    with _open_text(url) as f:
        head = f.read(2048).lstrip(" \t")
    if head.startswith("[") or head.startswith("{\n") or head.startswith("{\r"):
        return "json"
    if head.startswith("{"):
        return "jsonl"
    if base.endswith(".json"):
        return "json"
    raise ValueError(f"Unknown format for {url}: expected .jsonl, .json, .txt or .parquet (optionally compressed)")


def _iter_rows(url: str, row: int, columns=None) -> Iterator[dict]:
    fmt = _sniff_format_for_dataset(url)
    if fmt == "jsonl":
        with _open_text(url) as f:
            for i, line in enumerate(f):
                if i < row or not line.strip():
                    continue
                yield json.loads(line)
    elif fmt == "json":
        with _open_text(url) as f:
            data = json.load(f)
        yield from data[row:]
    elif fmt == "txt":
        with _open_text(url) as f:
            for i, line in enumerate(f):
                if i >= row:
                    yield {"text": line.rstrip("\n")}
    elif fmt == "parquet":
        import fsspec
        import pyarrow.parquet as pq

        with fsspec.open(url, "rb") as f:
            pf = pq.ParquetFile(f)
            seen = 0
            for g in range(pf.num_row_groups):
                n = pf.metadata.row_group(g).num_rows
                if seen + n <= row:
                    seen += n
                    continue
                table = pf.read_row_group(g, columns=columns)
                rows = table.to_pylist()
                yield from rows[max(0, row - seen):]
                seen += n
    else:
        raise ValueError(f"Unknown format {fmt}")


class UrlDataSource(UrlBackedShardedDataSource[dict]):
    """Dict rows from jsonl / json / parquet / text files; ``columns`` restricts the keys."""

    def __init__(self, urls, columns=None):
        super().__init__(urls)
        self.columns = columns

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[dict]:
        url = self._shard_name_to_url_mapping[shard_name]
        for r in _iter_rows(url, row, self.columns):
            yield {k: r[k] for k in self.columns} if self.columns else r


class TextUrlDataSource(UrlBackedShardedDataSource[str]):
    """The ``text_key`` string of every row."""

    def __init__(self, urls, text_key: str = "text"):
        super().__init__(urls)
        self.text_key = text_key

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[str]:
        url = self._shard_name_to_url_mapping[shard_name]
        for r in _iter_rows(url, row, None):
            yield r[self.text_key]


class JsonlDataSource(UrlDataSource):
    pass


class JsonDataSource(UrlDataSource):
    pass


class ParquetDataSource(UrlDataSource):
    pass


def datasource_from_jsonl(urls_or_paths: Sequence[str]) -> ShardedDataSource[dict]:
    return JsonlDataSource(urls_or_paths)


def datasource_from_json(urls_or_paths: Sequence[str]) -> ShardedDataSource[dict]:
    return JsonDataSource(urls_or_paths)


def datasource_from_parquet(urls_or_paths: Sequence[str]) -> ShardedDataSource[dict]:
    return ParquetDataSource(urls_or_paths)


class WrappedHFDataSource(ShardedDataSource[dict]):
    """A Hugging Face ``datasets`` dataset (streaming or not); shards follow the dataset's own ``n_shards``."""

    def __init__(self, id, *, split, streaming: bool = True, **kwargs):
        self.id, self.split, self.streaming, self.kwargs = id, split, streaming, kwargs
        self._names: Optional[List[str]] = None

    def _load_dataset(self):
        try:
            import datasets
        except ImportError as e:
            raise ImportError("the `datasets` package is required for Hugging Face dataset sources") from e
        return datasets.load_dataset(self.id, split=self.split, streaming=self.streaming, **self.kwargs)

    @property
    def shard_names(self) -> Sequence[str]:
        if self._names is None:
            ds = self._load_dataset()
            n = getattr(ds, "n_shards", 1) or 1
            self._names = [f"shard_{i}" for i in range(n)] if n > 1 else ["data"]
        return self._names

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[dict]:
        ds = self._load_dataset()
        if shard_name != "data":
            ds = ds.shard(len(self.shard_names), int(shard_name.split("_")[1]))
        if row:
            ds = ds.skip(row) if hasattr(ds, "skip") else ds.select(range(row, len(ds)))
        yield from ds


def datasource_from_hf(id: str, *, split, **kwargs) -> ShardedDataSource[dict]:
    return WrappedHFDataSource(id, split=split, **kwargs)


class AudioTextUrlDataSource(UrlBackedShardedDataSource):
    """``(audio array, sampling rate, text)`` triples from jsonl/parquet rows whose audio column holds an array, a dict with
    ``array``/``sampling_rate``, raw bytes, or a path to an audio file."""

    def __init__(self, urls, text_key="sentence", audio_key="audio", sampling_rate=16000):
        super().__init__(urls)
        self.text_key, self.audio_key, self.sampling_rate = text_key, audio_key, sampling_rate

    @staticmethod
    def resolve_audio_pointer(audio_pointer, sampling_rate) -> Dict[str, Any]:
        if isinstance(audio_pointer, dict) and "array" in audio_pointer:
            return {"array": np.asarray(audio_pointer["array"], dtype=np.float32), "sampling_rate": audio_pointer.get("sampling_rate", sampling_rate)}
        if isinstance(audio_pointer, (list, np.ndarray)):
            return {"array": np.asarray(audio_pointer, dtype=np.float32), "sampling_rate": sampling_rate}
        raw = None
        if isinstance(audio_pointer, dict) and audio_pointer.get("bytes"):
            raw = audio_pointer["bytes"]
        elif isinstance(audio_pointer, (bytes, bytearray)):
            raw = bytes(audio_pointer)
        elif isinstance(audio_pointer, str) or (isinstance(audio_pointer, dict) and audio_pointer.get("path")):
            import fsspec

            path = audio_pointer if isinstance(audio_pointer, str) else audio_pointer["path"]
            with fsspec.open(path, "rb") as f:
                raw = f.read()
        if raw is None:
            raise ValueError(f"Unsupported audio pointer {type(audio_pointer)}")
        return _decode_wav(raw, sampling_rate)

    def open_shard_at_row(self, shard_name: str, row: int):
        url = self._shard_name_to_url_mapping[shard_name]
        for r in _iter_rows(url, row, None):
            audio = self.resolve_audio_pointer(r[self.audio_key], self.sampling_rate)
            yield (audio["array"], audio["sampling_rate"], r[self.text_key])


def _decode_wav(raw: bytes, sampling_rate: int) -> Dict[str, Any]:
    """PCM WAV bytes -> mono float32 in [-1, 1], linearly resampled to ``sampling_rate``."""
    import wave

    with wave.open(io.BytesIO(raw)) as w:
        sr, nch, width, n = w.getframerate(), w.getnchannels(), w.getsampwidth(), w.getnframes()
        frames = w.readframes(n)
    dt = {1: np.uint8, 2: np.int16, 4: np.int32}[width]
    a = np.frombuffer(frames, dtype=dt).astype(np.float32)
    a = (a - 128.0) / 128.0 if width == 1 else a / float(1 << (8 * width - 1))
    if nch > 1:
        a = a.reshape(-1, nch).mean(axis=1)
    if sr != sampling_rate and len(a):
        new_n = int(round(len(a) * sampling_rate / sr))
        a = np.interp(np.linspace(0, len(a) - 1, new_n), np.arange(len(a)), a).astype(np.float32)
    return {"array": a, "sampling_rate": sampling_rate}


class _TransformedDataset:
    source: ShardedDataSource
    _transform: Any


class _MappedShardedDataSource(ShardedDataSource[T], _TransformedDataset):
    def __init__(self, source: ShardedDataSource, fn: Callable):
        self.source, self.fn = source, fn
        self._transform = _MapTransform(fn)

    @property
    def shard_names(self) -> Sequence[str]:
        return self.source.shard_names

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[T]:
        return map(self.fn, self.source.open_shard_at_row(shard_name, row))


class _BatchMappedShardedDataSource(ShardedDataSource[T], _TransformedDataset):
    def __init__(self, source: ShardedDataSource, fn, batch_size, num_cpus=1, num_gpus=0, output_exemplar=None, **resources):
        self.source, self.fn, self.batch_size = source, fn, batch_size
        self._transform = _BatchMapTransform(fn, batch_size, num_cpus, num_gpus, resources, output_exemplar=output_exemplar)

    @property
    def shard_names(self) -> Sequence[str]:
        return self.source.shard_names

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[T]:
        # a batch transform may change the number of rows, so ``row`` counts *input* rows
        for batch in batched(self.source.open_shard_at_row(shard_name, row), self.batch_size):
            yield from _canonicalize_batch(self.fn(batch))


def _construct_composite_batch_processor(dataset: ShardedDataSource):
    """Peel mapped layers off ``dataset``: (innermost source, one processor running all transforms in order)."""
    transforms = []
    num_cpus, num_gpus, resources = 0, 0, {}
    src = dataset
    while isinstance(src, _TransformedDataset):
        t = src._transform
        transforms.append(t)
        if isinstance(t, _BatchMapTransform):
            num_cpus, num_gpus = max(num_cpus, t.num_cpus), max(num_gpus, t.num_gpus)
            for k, v in t.resources.items():
                resources[k] = max(resources.get(k, 0), v)
        src = src.source
    transforms.reverse()
    return src, _CompositeBatchProcessor(transforms, num_cpus, num_gpus, resources)
