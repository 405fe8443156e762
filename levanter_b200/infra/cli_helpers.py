"""Launcher defaults and command construction (src/levanter/infra/cli_helpers.py).

``.levanter.yaml`` (searched from the working directory upwards, then in the home directory) supplies default values for
launcher options and environment variables: ``{env: {WANDB_API_KEY: ...}, launch: {nproc_per_node: 8}}``."""
from __future__ import annotations

import os
import shlex
import subprocess
from typing import Dict, List, Optional

import yaml


def load_config(start: Optional[str] = None) -> dict:
    d = os.path.abspath(start or os.getcwd())
    candidates = []
    while True:
        candidates.append(os.path.join(d, ".levanter.yaml"))
        parent = os.path.dirname(d)
        if parent == d:
            break
        d = parent
    candidates.append(os.path.expanduser("~/.levanter.yaml"))
    for c in candidates:
        if os.path.isfile(c):
            with open(c) as f:
                return yaml.safe_load(f) or {}
    return {}


def get_git_commit() -> Optional[str]:
    try:
        return subprocess.check_output(["git", "rev-parse", "HEAD"], stderr=subprocess.DEVNULL).decode().strip()
    except Exception:  # noqa: BLE001
        return None


def default_run_id() -> str:
    """A short random run id, the same on every rank only if the launcher exports it (``RUN_ID``)."""
    import random
    import string

    return os.environ.get("RUN_ID") or "".join(random.choice(string.ascii_lowercase + string.digits) for _ in range(8))


def make_torchrun_command(module: str, args: List[str], *, nproc_per_node: int, nnodes: int = 1, node_rank: int = 0,
                          master_addr: str = "127.0.0.1", master_port: int = 29500) -> List[str]:
    cmd = ["python", "-m", "torch.distributed.run", f"--nnodes={nnodes}", f"--nproc-per-node={nproc_per_node}",
           f"--node-rank={node_rank}", "--master-addr", master_addr, "--master-port", str(master_port), "-m", module]
    return cmd + list(args)


def make_docker_run_command(image: str, command: List[str], *, env: Optional[Dict[str, str]] = None, gpus: str = "all",
                            mounts: Optional[Dict[str, str]] = None, foreground: bool = True) -> List[str]:
    out = ["docker", "run", "--rm" if foreground else "-d", "--gpus", gpus, "--ipc=host", "--ulimit", "memlock=-1", "--net=host"]
    for k, v in (env or {}).items():
        out += ["-e", f"{k}={v}"]
    for host, cont in (mounts or {}).items():
        out += ["-v", f"{host}:{cont}"]
    return out + [image] + list(command)


def format_command(cmd: List[str]) -> str:
    return " ".join(shlex.quote(c) for c in cmd)
