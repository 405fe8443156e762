"""Delete everything under a prefix of any fsspec filesystem, many objects at a time (stands in for the reference's
scripts/gcs_bulk_delete.py, which schedules a storage-transfer job for the same purpose on one cloud): old checkpoint trees and
caches hold millions of small chunk files, and removing them one by one from a laptop takes days.

``python -m levanter_b200.infra.bulk_delete gs://bucket/checkpoints/old-run [--workers 64] [--dry-run]``"""
from __future__ import annotations

import argparse
from concurrent.futures import ThreadPoolExecutor
from typing import List, Tuple


def bulk_delete(url: str, *, workers: int = 64, batch: int = 500, dry_run: bool = False) -> Tuple[int, List[str]]:
    """Remove every file under ``url`` and then the directories.  Returns ``(files removed, failures)``."""
    import fsspec

    fs, plain = fsspec.core.url_to_fs(url)
    if not fs.exists(plain):
        return 0, []
    files = [plain] if fs.isfile(plain) else fs.find(plain)
    if dry_run:
        return len(files), []
    failures: List[str] = []

    def rm(chunk: List[str]) -> int:
        try:
            fs.rm(chunk)
            return len(chunk)
        except Exception:  # noqa: BLE001  (one bad object must not stop the others: retry singly)
            done = 0
            for f in chunk:
                try:
                    fs.rm(f)
                    done += 1
                except FileNotFoundError:
                    done += 1
                except Exception as e:  # noqa: BLE001
                    failures.append(f"{f}: {e}")
            return done

    chunks = [files[i:i + batch] for i in range(0, len(files), batch)]
    with ThreadPoolExecutor(max_workers=max(1, workers)) as pool:
        removed = sum(pool.map(rm, chunks))
    if not failures and fs.exists(plain):
        try:
            fs.rm(plain, recursive=True)  # the now-empty directories (object stores have none)
        except Exception:  # noqa: BLE001
            pass
    return removed, failures


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("url")
    ap.add_argument("--workers", type=int, default=64)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    n, failures = bulk_delete(args.url, workers=args.workers, dry_run=args.dry_run)
    print(f"{'would remove' if args.dry_run else 'removed'} {n} files under {args.url}")
    for f in failures:
        print("FAILED", f)
    raise SystemExit(1 if failures else 0)


if __name__ == "__main__":
    main()
