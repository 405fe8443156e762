"""``python -m levanter_b200.infra.launch [--nproc-per-node N] [--docker IMAGE] -- levanter_b200.main.train_lm --config_path X``

Starts one process per GPU on this node through ``torch.distributed.run``.  Under SLURM (``SLURM_JOB_ID`` set) the node
count, node rank and the rendezvous address are taken from the job's environment the same way
:class:`levanter_b200.distributed.LevanterSlurmCluster` does, so the same line works inside ``srun``."""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

from ..distributed import LevanterSlurmCluster
from . import cli_helpers


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--nproc-per-node", type=int, default=None)
    ap.add_argument("--master-port", type=int, default=None)
    ap.add_argument("--docker", default=None, help="run inside this image instead of the current environment")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    rest = a.rest[1:] if a.rest and a.rest[0] == "--" else a.rest
    if not rest:
        ap.error("give the module to run after --")
    cfg = cli_helpers.load_config()
    launch_cfg = cfg.get("launch", {})
    nproc = a.nproc_per_node or launch_cfg.get("nproc_per_node")
    if nproc is None:
        import torch

        nproc = max(torch.cuda.device_count(), 1)
    nnodes, node_rank, addr, port = 1, 0, "127.0.0.1", a.master_port or int(launch_cfg.get("master_port", 29500))
    if LevanterSlurmCluster.is_env_present():
        nnodes = int(os.environ.get("SLURM_JOB_NUM_NODES", os.environ.get("SLURM_NNODES", "1")))
        node_rank = int(os.environ.get("SLURM_NODEID", "0"))
        if nnodes > 1:
            addr = LevanterSlurmCluster.get_coordinator_address().rsplit(":", 1)[0]
            port = a.master_port or int(LevanterSlurmCluster.get_coordinator_address().rsplit(":", 1)[1])
    cmd = cli_helpers.make_torchrun_command(rest[0], rest[1:], nproc_per_node=nproc, nnodes=nnodes, node_rank=node_rank,
                                            master_addr=addr, master_port=port)
    env = dict(os.environ)
    env.update({str(k): str(v) for k, v in cfg.get("env", {}).items()})
    env.setdefault("RUN_ID", cli_helpers.default_run_id())
    if a.docker:
        cmd = cli_helpers.make_docker_run_command(a.docker, cmd, env={k: env[k] for k in list(cfg.get("env", {})) + ["RUN_ID"]},
                                                  mounts={os.getcwd(): "/workspace"})
    print(cli_helpers.format_command(cmd), file=sys.stderr)
    if a.dry_run:
        return 0
    return subprocess.call(cmd, env=env)


if __name__ == "__main__":
    raise SystemExit(main())
