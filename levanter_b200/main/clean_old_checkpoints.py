"""Delete superseded training checkpoints (the reference's scripts/clean_old_checkpoints.py:25-75): per run directory keep the
newest complete checkpoint and the newest one whose step ends in ``000``; only checkpoints older than ``--min-age-days`` go.

``python -m levanter_b200.main.clean_old_checkpoints checkpoints/ [--dry-run]``"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import shutil
from typing import List, Tuple


def _complete_checkpoints(run_dir: str) -> List[Tuple[int, str, datetime.datetime]]:
    out = []
    for name in os.listdir(run_dir):
        meta = os.path.join(run_dir, name, "metadata.json")
        if not os.path.isfile(meta):
            continue
        try:
            with open(meta) as f:
                m = json.load(f)
            ts = datetime.datetime.fromisoformat(m["timestamp"]) if "timestamp" in m else datetime.datetime.fromtimestamp(os.path.getmtime(meta))
            out.append((int(m["step"]), os.path.join(run_dir, name), ts))
        except Exception:  # noqa: BLE001  (unreadable metadata: leave the directory alone)
            continue
    return sorted(out)


def checkpoints_to_delete(run_dir: str, min_age_days: float = 0.0, now=None) -> List[str]:
    cks = _complete_checkpoints(run_dir)
    if len(cks) <= 1:
        return []
    keep = {cks[-1][1]}
    thousands = [c for c in cks if c[0] % 1000 == 0]
    if thousands:
        keep.add(thousands[-1][1])
    now = now or datetime.datetime.now()
    return [p for _, p, ts in cks if p not in keep and (now - ts.replace(tzinfo=None)).total_seconds() >= min_age_days * 86400]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("base_path")
    ap.add_argument("--min-age-days", type=float, default=1.0)
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    for run in sorted(os.listdir(a.base_path)):
        run_dir = os.path.join(a.base_path, run)
        if not os.path.isdir(run_dir):
            continue
        for p in checkpoints_to_delete(run_dir, a.min_age_days):
            print(("would delete " if a.dry_run else "deleting ") + p)
            if not a.dry_run:
                shutil.rmtree(p)


if __name__ == "__main__":
    main()
