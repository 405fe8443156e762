"""Download the profiler trace that a run logged as an artifact and lay it out for TensorBoard's profile plugin (the
reference's scripts/wandb_tensorboard_profile.py:96-151).  The trainer's profiler hook logs its trace directory as an
artifact of type ``profile``; this fetches the newest one of a run.

``python -m levanter_b200.infra.fetch_profile <entity/project/run_id> [--out profiles_tb] [--type profile]``
then ``tensorboard --logdir profiles_tb``."""
from __future__ import annotations

import argparse
import os
import shutil
from typing import Optional


def fetch_profile(run_path: str, out_dir: str = "profiles_tb", artifact_type: str = "profile", *, api=None) -> Optional[str]:
    """Returns the directory the trace was written to (``<out_dir>/<run id>/plugins/profile/<artifact version>``), or None
    when the run logged no artifact of that type."""
    if api is None:
        import wandb

        api = wandb.Api()
    run = api.run(run_path)
    newest = None
    for art in run.logged_artifacts():
        if art.type == artifact_type:
            newest = art  # logged_artifacts lists in order of creation
    if newest is None:
        return None
    version = str(getattr(newest, "version", "v0"))
    dest = os.path.join(out_dir, str(getattr(run, "id", run_path.split("/")[-1])), "plugins", "profile", version)
    os.makedirs(dest, exist_ok=True)
    got = newest.download()
    for root, _, files in os.walk(got):
        for name in files:
            rel = os.path.relpath(os.path.join(root, name), got)
            os.makedirs(os.path.dirname(os.path.join(dest, rel)) or dest, exist_ok=True)
            shutil.copy2(os.path.join(root, name), os.path.join(dest, rel))
    return dest


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("run_path")
    ap.add_argument("--out", default="profiles_tb")
    ap.add_argument("--type", default="profile")
    args = ap.parse_args(argv)
    dest = fetch_profile(args.run_path, args.out, args.type)
    print(f"no artifact of type {args.type!r} in {args.run_path}" if dest is None else f"wrote {dest}; run: tensorboard --logdir {args.out}")


if __name__ == "__main__":
    main()
