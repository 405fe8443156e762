"""Split jsonl shards into one output file per value of a field (the reference's scripts/preproc/split-pile-shards.py splits The
Pile by ``meta.pile_set_name`` so that each domain can be a component of a mixture).  Inputs and outputs may be compressed and
may live on any fsspec filesystem; an input ``<name>.jsonl.zst`` contributes ``<out>/<value>/<name>.jsonl.zst`` for every value
it contains.

``python -m levanter_b200.data.split_by_field --field meta.pile_set_name --out gs://bucket/pile-domains 00.jsonl.zst 01.jsonl.zst``"""
from __future__ import annotations

import argparse
import json
import os
import re
from typing import Dict, Iterable, Mapping, Optional


def _get(row: dict, dotted: str):
    cur = row
    for part in dotted.split("."):
        cur = cur[part]
    return cur


def _slug(value) -> str:
    return re.sub(r"[^A-Za-z0-9_.-]+", "_", str(value)).strip("_").lower() or "none"


def split_file(input_path: str, out_dir: str, field: str, names: Optional[Mapping[str, str]] = None, compression: str = "zstd") -> Dict[str, int]:
    """Returns ``{output name of the value: rows written}`` for one input file.  ``names`` maps field values to directory
    names (values not in it are slugged)."""
    import fsspec

    base = os.path.basename(input_path)
    stem = re.sub(r"\.(jsonl|json|ndjson)(\.(zst|zstd|gz|bz2|xz))?$", "", base)
    ext = {"zstd": ".jsonl.zst", "gzip": ".jsonl.gz", None: ".jsonl"}[compression]
    outs: Dict[str, object] = {}
    counts: Dict[str, int] = {}
    try:
        with fsspec.open(input_path, "r", compression="infer") as src:
            for line in src:
                if not line.strip():
                    continue
                value = _get(json.loads(line), field)
                name = (names or {}).get(value) or _slug(value)
                if name not in outs:
                    path = f"{out_dir.rstrip('/')}/{name}/{stem}{ext}"
                    fs, plain = fsspec.core.url_to_fs(path)
                    fs.makedirs(os.path.dirname(plain), exist_ok=True)
                    outs[name] = fsspec.open(path, "w", compression=compression).open()
                    counts[name] = 0
                outs[name].write(line if line.endswith("\n") else line + "\n")  # type: ignore
                counts[name] += 1
    finally:
        for f in outs.values():
            f.close()  # type: ignore
    return counts


def split_by_field(inputs: Iterable[str], out_dir: str, field: str, names: Optional[Mapping[str, str]] = None,
                   compression: str = "zstd") -> Dict[str, int]:
    total: Dict[str, int] = {}
    for path in inputs:
        for k, v in split_file(path, out_dir, field, names, compression).items():
            total[k] = total.get(k, 0) + v
    return total


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("inputs", nargs="+")
    ap.add_argument("--field", required=True, help="dotted path of the field to split by, e.g. meta.pile_set_name")
    ap.add_argument("--out", required=True)
    ap.add_argument("--compression", default="zstd", choices=["zstd", "gzip", "none"])
    args = ap.parse_args(argv)
    from ..utils.fsspec_utils import expand_glob

    files = [f for pattern in args.inputs for f in expand_glob(pattern)]
    counts = split_by_field(files, args.out, args.field, compression=None if args.compression == "none" else args.compression)
    for k in sorted(counts):
        print(f"{k}: {counts[k]} rows")


if __name__ == "__main__":
    main()
