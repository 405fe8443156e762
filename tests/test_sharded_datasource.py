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
