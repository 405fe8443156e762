"""The value of a metric at a few steps for every commit of the current git history, from the Weights & Biases runs that
recorded ``config.git_commit`` (the reference's scripts/loss_history.py:12-51): a quick way to see which commit moved the
loss curve.

``python -m levanter_b200.infra.loss_history [--project levanter] [--metric train/loss] [--max-commits 50]``"""
from __future__ import annotations

import argparse
import subprocess
from typing import Dict, Iterable, List, Optional, Tuple

DEFAULT_METRIC = "train/loss"


def fetch_metric_for_sha(sha: str, metric_name: str = DEFAULT_METRIC, steps: Iterable[int] = range(0, 101, 10), *, project: str = "levanter",
                         api=None) -> Dict[int, float]:
    """``{step: value}`` of the first run whose config names commit ``sha``; empty when there is none."""
    if api is None:
        import wandb

        api = wandb.Api()
    steps = list(steps)
    runs = api.runs(project, {"config.git_commit": sha})
    out: Dict[int, float] = {}
    for run in runs:
        for row in run.scan_history(keys=["_step", metric_name], min_step=min(steps), max_step=max(steps) + 1):
            step = int(row["_step"])
            if step in steps and row.get(metric_name) is not None:
                out[step] = float(row[metric_name])
        break
    return out


def git_log(max_commits: Optional[int] = None, cwd: Optional[str] = None) -> List[Tuple[str, str]]:
    """``[(sha, subject)]``, newest first."""
    cmd = ["git", "log", "--pretty=format:%H %s"] + ([f"-{max_commits}"] if max_commits else [])
    text = subprocess.run(cmd, stdout=subprocess.PIPE, check=True, cwd=cwd).stdout.decode("utf-8").strip()
    return [tuple(line.split(" ", 1)) if " " in line else (line, "") for line in text.split("\n") if line]  # type: ignore


def history_lines(commits: Iterable[Tuple[str, str]], metric_name: str = DEFAULT_METRIC, *, project: str = "levanter", api=None,
                  steps: Iterable[int] = range(0, 101, 10)) -> List[str]:
    steps = list(steps)
    lines = []
    for sha, subject in commits:
        values = fetch_metric_for_sha(sha, metric_name, steps, project=project, api=api)
        shown = ", ".join(f"{s}: {v:.4g}" for s, v in sorted(values.items()))
        lines.append(f"{sha} - {subject} -> {shown}")
    return lines


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--project", default="levanter")
    ap.add_argument("--metric", default=DEFAULT_METRIC)
    ap.add_argument("--max-commits", type=int, default=None)
    args = ap.parse_args(argv)
    for line in history_lines(git_log(args.max_commits), args.metric, project=args.project):
        print(line)


if __name__ == "__main__":
    main()
