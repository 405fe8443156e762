"""Row sources over files (levanter_b200/data/sharded_datasource.py; scenarios after the reference's tests/test_sharded_dataset.py)."""
import gzip
import json

import pytest

from levanter_b200.data.sharded_datasource import (JsonDataSource, JsonlDataSource, ParquetDataSource, TextUrlDataSource, UrlDataSource,
                                                   _sniff_format_for_dataset)


def test_json_extension_means_a_document_or_one_object_per_line(tmp_path):
    p = tmp_path / "a.json"
    p.write_text('[{"text": "hello world"}, {"text": "hello world!"}]')
    assert _sniff_format_for_dataset(str(p)) == "json"
    p.write_text('{"text": "hello world"}\n{"text": "hello world!"}\n')
    assert _sniff_format_for_dataset(str(p)) == "jsonl"
    assert [r["text"] for r in UrlDataSource([str(p)]).open_shard_at_row(UrlDataSource([str(p)]).shard_names[0], 1)] == ["hello world!"]
    p.write_text('{\n"ids": [1, 2, 3]\n}\n')
    assert _sniff_format_for_dataset(str(p)) == "json"


def test_known_extensions_compressed_or_not(tmp_path):
    for name, fmt in (("x.jsonl", "jsonl"), ("x.jsonl.gz", "jsonl"), ("x.txt", "txt"), ("x.parquet", "parquet"), ("x.txt.zst", "txt")):
        assert _sniff_format_for_dataset(str(tmp_path / name)) == fmt  # decided by the name alone: the files do not exist
    q = tmp_path / "rows.data"
    q.write_text('{"text": "a"}\n{"text": "b"}\n')
    assert _sniff_format_for_dataset(str(q)) == "jsonl"  # no known extension: by content
    q.write_text("plain words\n")
    with pytest.raises(ValueError, match="Unknown format"):
        _sniff_format_for_dataset(str(q))


def test_jsonl_rows_from_a_row_offset_plain_and_gzipped(tmp_path):
    rows = [{"text": f"doc {i}", "n": i} for i in range(7)]
    (tmp_path / "a.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
    with gzip.open(tmp_path / "b.jsonl.gz", "wt") as f:
        f.write("".join(json.dumps(r) + "\n\n" for r in rows))  # blank lines are skipped
    src = JsonlDataSource([str(tmp_path / "a.jsonl"), str(tmp_path / "b.jsonl.gz")])
    assert len(src.shard_names) == 2 and len(set(src.shard_names)) == 2
    assert list(src.open_shard_at_row(src.shard_names[0], 5)) == rows[5:]
    assert [r["n"] for r in src.open_shard(src.shard_names[1])] == list(range(7))
    assert len(list(src)) == 14
    texts = TextUrlDataSource([str(tmp_path / "a.jsonl")])
    assert list(texts.open_shard_at_row(texts.shard_names[0], 4)) == ["doc 4", "doc 5", "doc 6"]


def test_json_document_rows(tmp_path):
    rows = [{"text": f"doc {i}"} for i in range(4)]
    (tmp_path / "a.json").write_text(json.dumps(rows, indent=1))
    src = JsonDataSource([str(tmp_path / "a.json")])
    assert list(src.open_shard_at_row(src.shard_names[0], 2)) == rows[2:]


def test_parquet_rows_from_a_row_offset(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq

    p = str(tmp_path / "t.parquet")
    pq.write_table(pa.Table.from_pydict({"column1": ["value1", "value2", "value3"], "column2": [10, 20, 30]}), p)
    src = ParquetDataSource([p])
    assert len(src.shard_names) == 1
    rows = list(src.open_shard_at_row(src.shard_names[0], 1))
    assert rows == [{"column1": "value2", "column2": 20}, {"column1": "value3", "column2": 30}]

    # several row groups: the offset may fall inside a later group
    p2 = str(tmp_path / "g.parquet")
    pq.write_table(pa.Table.from_pydict({"text": [f"line{i}" for i in range(1, 11)], "column2": list(range(10))}), p2, row_group_size=3)
    texts = TextUrlDataSource([p2], text_key="text")
    assert list(texts.open_shard_at_row(texts.shard_names[0], 2)) == [f"line{i}" for i in range(3, 11)]
    assert list(texts.open_shard_at_row(texts.shard_names[0], 7)) == ["line8", "line9", "line10"]
    assert list(texts.open_shard_at_row(texts.shard_names[0], 10)) == []


def test_mapped_sources_keep_shards_and_row_offsets(tmp_path):
    (tmp_path / "a.jsonl").write_text("".join(json.dumps({"text": str(i)}) + "\n" for i in range(6)))
    src = TextUrlDataSource([str(tmp_path / "a.jsonl")]).map(int).map_batches(lambda b: [x * 2 for x in b], batch_size=4)
    name = src.shard_names[0]
    assert list(src.open_shard_at_row(name, 3)) == [6, 8, 10]
    assert list(src) == [0, 2, 4, 6, 8, 10]


def test_hugging_face_dataset_source_with_a_stand_in_datasets_package(monkeypatch):
    import sys
    import types

    from levanter_b200.data.sharded_datasource import datasource_from_hf

    class Fake:
        def __init__(self, rows, n_shards=1):
            self.rows, self.n_shards = rows, n_shards

        def shard(self, num_shards, index):
            return Fake(self.rows[index::num_shards])

        def skip(self, n):
            return Fake(self.rows[n:])

        def __iter__(self):
            return iter(self.rows)

    calls = []

    def load_dataset(id, split, streaming, **kw):
        calls.append((id, split, streaming, kw))
        return Fake([{"text": f"doc {i}"} for i in range(10)], n_shards=2 if id == "two" else 1)

    fake = types.ModuleType("datasets")
    fake.load_dataset = load_dataset
    monkeypatch.setitem(sys.modules, "datasets", fake)
    one = datasource_from_hf("one", split="train", name="cfg")
    assert one.shard_names == ["data"] and [r["text"] for r in one.open_shard_at_row("data", 7)] == ["doc 7", "doc 8", "doc 9"]
    assert calls[0] == ("one", "train", True, {"name": "cfg"})
    two = datasource_from_hf("two", split="validation", streaming=False)
    assert two.shard_names == ["shard_0", "shard_1"] and two.num_shards == 2
    assert [r["text"] for r in two.open_shard_at_row("shard_1", 3)] == ["doc 7", "doc 9"]
    assert len(list(two)) == 10 and calls[-1][:3] == ("two", "validation", False)
    monkeypatch.setitem(sys.modules, "datasets", None)
    with pytest.raises(ImportError, match="datasets"):
        datasource_from_hf("x", split="train").shard_names


def test_audio_pointers_arrays_mappings_bytes_and_paths(tmp_path):
    import io
    import wave

    import numpy as np

    from levanter_b200.data.sharded_datasource import AudioTextUrlDataSource

    R = AudioTextUrlDataSource.resolve_audio_pointer
    a = R([0.0, 0.5, -0.5], 16000)
    assert a["array"].dtype == np.float32 and a["sampling_rate"] == 16000 and a["array"].tolist() == [0.0, 0.5, -0.5]
    b = R({"array": np.ones(4), "sampling_rate": 8000}, 16000)
    assert b["sampling_rate"] == 8000 and b["array"].shape == (4,)

    def wav(rate, channels, samples):
        buf = io.BytesIO()
        with wave.open(buf, "wb") as w:
            w.setnchannels(channels), w.setsampwidth(2), w.setframerate(rate)
            w.writeframes((np.asarray(samples) * 32767).astype(np.int16).tobytes())
        return buf.getvalue()

    t = np.sin(np.linspace(0, 20, 800))
    mono = R(wav(16000, 1, t), 16000)
    assert mono["array"].shape == (800,) and np.abs(mono["array"] - t).max() < 1e-3
    stereo = R({"bytes": wav(16000, 2, np.stack([t, -t], axis=1).reshape(-1))}, 16000)
    assert stereo["array"].shape == (800,) and np.abs(stereo["array"]).max() < 1e-3  # the channels cancel
    half = R(wav(8000, 1, t), 16000)
    assert half["array"].shape == (1600,) and half["sampling_rate"] == 16000  # resampled
    (tmp_path / "clip.wav").write_bytes(wav(16000, 1, t))
    assert R(str(tmp_path / "clip.wav"), 16000)["array"].shape == (800,)
    assert R({"path": str(tmp_path / "clip.wav")}, 16000)["array"].shape == (800,)
    with pytest.raises(ValueError, match="Unsupported"):
        R(12345, 16000)

    (tmp_path / "speech.jsonl").write_text(json.dumps({"audio": {"path": str(tmp_path / "clip.wav")}, "sentence": "hello"}) + "\n"
                                           + json.dumps({"audio": [0.1, 0.2], "sentence": "again"}) + "\n")
    src = AudioTextUrlDataSource([str(tmp_path / "speech.jsonl")])
    rows = list(src)
    assert rows[0][0].shape == (800,) and rows[0][1:] == (16000, "hello") and rows[1][2] == "again"
