"""Small operations tools: metric history per commit, profile download, bulk deletion, splitting shards by a field (the
reference keeps these as stand-alone scripts under scripts/)."""
import gzip
import json
import os
import uuid
from types import SimpleNamespace

from levanter_b200.data.split_by_field import split_by_field
from levanter_b200.infra.bulk_delete import bulk_delete
from levanter_b200.infra.fetch_profile import fetch_profile
from levanter_b200.infra.loss_history import fetch_metric_for_sha, git_log, history_lines


class _Run:
    def __init__(self, rows):
        self.rows = rows

    def scan_history(self, keys, min_step, max_step):
        return [r for r in self.rows if min_step <= r["_step"] < max_step]


class _Api:
    def __init__(self, by_sha):
        self.by_sha, self.queries = by_sha, []

    def runs(self, project, filters):
        self.queries.append((project, filters))
        return self.by_sha.get(filters["config.git_commit"], [])


def test_metric_history_per_commit():
    rows = [{"_step": s, "train/loss": 5.0 - 0.01 * s} for s in range(0, 120, 5)]
    api = _Api({"abc": [_Run(rows)], "def": []})
    got = fetch_metric_for_sha("abc", api=api, project="proj")
    assert sorted(got) == list(range(0, 101, 10)) and got[100] == 4.0 and api.queries[0] == ("proj", {"config.git_commit": "abc"})
    assert fetch_metric_for_sha("def", api=api) == {} and fetch_metric_for_sha("unknown", api=api) == {}
    lines = history_lines([("abc", "fix the loader"), ("def", "docs")], api=api, steps=[0, 50])
    assert lines == ["abc - fix the loader -> 0: 5, 50: 4.5", "def - docs -> "]
    commits = git_log(3, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert 1 <= len(commits) <= 3 and all(len(sha) == 40 for sha, _ in commits)


def test_profile_artifact_is_laid_out_for_tensorboard(tmp_path):
    src = tmp_path / "artifact"
    (src / "sub").mkdir(parents=True)
    (src / "trace.json").write_text("{}")
    (src / "sub" / "more.pb").write_bytes(b"\x01")
    arts = [SimpleNamespace(type="config", version="v0", download=lambda: str(src)),
            SimpleNamespace(type="profile", version="v0", download=lambda: str(tmp_path / "missing")),
            SimpleNamespace(type="profile", version="v1", download=lambda: str(src))]
    api = SimpleNamespace(run=lambda path: SimpleNamespace(id="run42", logged_artifacts=lambda: arts))
    dest = fetch_profile("me/proj/run42", str(tmp_path / "tb"), api=api)
    assert dest == str(tmp_path / "tb" / "run42" / "plugins" / "profile" / "v1")  # the newest profile artifact
    assert sorted(os.listdir(dest)) == ["sub", "trace.json"] and os.path.exists(os.path.join(dest, "sub", "more.pb"))
    none = SimpleNamespace(run=lambda path: SimpleNamespace(id="r", logged_artifacts=lambda: arts[:1]))
    assert fetch_profile("me/proj/r", str(tmp_path / "tb"), api=none) is None


def test_bulk_delete_on_local_and_memory_filesystems(tmp_path):
    import fsspec

    root = tmp_path / "old-run"
    for i in range(25):
        d = root / f"step-{i}" / "model"
        d.mkdir(parents=True)
        (d / "0.0").write_bytes(b"x")
    (tmp_path / "keep.txt").write_text("stay")
    assert bulk_delete(str(root), dry_run=True) == (25, []) and root.exists()
    assert bulk_delete(str(root), workers=4, batch=7) == (25, [])
    assert not root.exists() and (tmp_path / "keep.txt").exists()
    assert bulk_delete(str(root)) == (0, [])  # nothing there any more

    fs = fsspec.filesystem("memory")
    base = f"memory://lvb-del/{uuid.uuid4().hex}"
    for i in range(10):
        with fs.open(f"{base}/a/{i}.bin", "wb") as f:
            f.write(b"1")
    with fs.open(f"{base}-other/x", "wb") as f:
        f.write(b"1")
    assert bulk_delete(f"{base}/a") == (10, [])
    assert fs.find(base) == [] and fs.exists(f"{base}-other/x")


def test_split_jsonl_shards_by_a_nested_field(tmp_path):
    rows = [{"text": f"doc {i}", "meta": {"pile_set_name": ["ArXiv", "Pile-CC", "Wikipedia (en)"][i % 3]}} for i in range(10)]
    with gzip.open(tmp_path / "00.jsonl.gz", "wt") as f:
        f.write("".join(json.dumps(r) + "\n" for r in rows[:6]) + "\n")
    (tmp_path / "01.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows[6:]))
    counts = split_by_field([str(tmp_path / "00.jsonl.gz"), str(tmp_path / "01.jsonl")], str(tmp_path / "out"), "meta.pile_set_name",
                            names={"Wikipedia (en)": "wiki_en"}, compression="gzip")
    assert counts == {"arxiv": 4, "pile-cc": 3, "wiki_en": 3}
    assert sorted(os.listdir(tmp_path / "out" / "arxiv")) == ["00.jsonl.gz", "01.jsonl.gz"]
    with gzip.open(tmp_path / "out" / "wiki_en" / "00.jsonl.gz", "rt") as f:
        back = [json.loads(line) for line in f]
    assert [r["text"] for r in back] == ["doc 2", "doc 5"]

    # the outputs are ordinary shards of a data source
    from levanter_b200.data.sharded_datasource import TextUrlDataSource

    src = TextUrlDataSource([str(tmp_path / "out" / "arxiv" / "{00,01}.jsonl.gz")])
    assert [t for t in src] == ["doc 0", "doc 3", "doc 6", "doc 9"]
