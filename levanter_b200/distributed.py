"""Process bootstrap: cluster discovery (torchrun or SLURM environment), ``torch.distributed`` initialisation, and the
local-leader election (src/levanter/distributed.py).

The reference calls ``jax.distributed.initialize`` with a 30-minute timeout after deriving the coordinator address
from SLURM variables (:315-373) and can auto-start a Ray cluster for data preprocessing (:200-312).  Here the data plane
is ``torch.distributed`` (NCCL on GPUs, gloo on CPU) and preprocessing uses local worker processes, so ``RayConfig`` is
accepted for config compatibility only."""
from __future__ import annotations

import logging
import os
import re
import socket
from dataclasses import dataclass
from datetime import timedelta
from typing import List, Optional, Union

import torch

logger = logging.getLogger(__name__)
_DEFAULT_PORT_BASE = 61000


def _square_brace_expand(node_list: str) -> List[str]:
    """Expand SLURM's compressed node lists: ``node[001-003,007],gpu5`` -> individual host names."""
    out: List[str] = []
    parts = _split_top_level_commas(node_list)
    for part in parts:
        m = re.match(r"^(.*?)\[([^\]]+)\](.*)$", part)
        if not m:
            if part:
                out.append(part)
            continue
        prefix, body, suffix = m.groups()
        for item in body.split(","):
            if "-" in item:
                lo, hi = item.split("-")
                width = len(lo)
                for i in range(int(lo), int(hi) + 1):
                    out.extend(_square_brace_expand(f"{prefix}{str(i).zfill(width)}{suffix}"))
            else:
                out.extend(_square_brace_expand(f"{prefix}{item}{suffix}"))
    return out


def _split_top_level_commas(s: str) -> List[str]:
    parts, depth, cur = [], 0, ""
    for ch in s:
        if ch == "[":
            depth += 1
        elif ch == "]":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    if cur:
        parts.append(cur)
    return parts


class LevanterSlurmCluster:
    """SLURM environment parsing (src/levanter/distributed.py:52-197): node list, tasks per node, local device ids
    from ``CUDA_VISIBLE_DEVICES``, and a coordinator port derived from the job id."""

    _JOBID = "SLURM_JOB_ID"
    _NODE_LIST_CHOICES = ["SLURM_STEP_NODELIST", "SLURM_JOB_NODELIST", "SLURM_NODELIST"]
    _TASKS_PER_NODE = "SLURM_STEP_TASKS_PER_NODE"
    _VISIBLE_DEVICES = "CUDA_VISIBLE_DEVICES"
    _NODE_NAME = "SLURMD_NODENAME"

    @classmethod
    def is_env_present(cls) -> bool:
        return cls._JOBID in os.environ and "SLURM_PROCID" in os.environ

    @classmethod
    def _node_list(cls) -> Optional[str]:
        for k in cls._NODE_LIST_CHOICES:
            if k in os.environ:
                return os.environ[k]
        return None

    @classmethod
    def get_coordinator_address(cls) -> str:
        nodes = cls._node_list()
        if nodes is None:
            raise ValueError("no SLURM node list in the environment")
        first = _square_brace_expand(nodes)[0]
        port = int(os.environ[cls._JOBID]) % (2**12) + (65535 - 2**12 + 1)
        return f"{first}:{port}"

    @classmethod
    def get_process_count(cls) -> int:
        return int(os.environ["SLURM_NTASKS"])

    @classmethod
    def get_process_id(cls) -> int:
        return int(os.environ["SLURM_PROCID"])

    @classmethod
    def get_tasks_per_node(cls) -> List[int]:
        """Parse ``SLURM_STEP_TASKS_PER_NODE`` such as ``2(x3),1`` -> ``[2, 2, 2, 1]``."""
        spec = os.environ.get(cls._TASKS_PER_NODE) or os.environ.get("SLURM_TASKS_PER_NODE")
        if spec is None:
            return [1]
        out: List[int] = []
        for item in spec.split(","):
            m = re.match(r"^(\d+)(?:\(x(\d+)\))?$", item.strip())
            if not m:
                raise ValueError(f"cannot parse tasks-per-node entry {item!r}")
            out.extend([int(m.group(1))] * int(m.group(2) or 1))
        return out

    @classmethod
    def get_local_process_id(cls) -> int:
        if "SLURM_LOCALID" in os.environ:
            return int(os.environ["SLURM_LOCALID"])
        return 0

    @classmethod
    def get_local_device_ids_for_process(cls) -> Optional[List[int]]:
        """Split the node's visible devices evenly among the tasks on this node."""
        local_id = cls.get_local_process_id()
        nodes = _square_brace_expand(cls._node_list() or "")
        tasks = cls.get_tasks_per_node()
        name = os.environ.get(cls._NODE_NAME)
        n_local = tasks[nodes.index(name)] if (name in nodes and nodes.index(name) < len(tasks)) else tasks[0]
        vis = os.environ.get(cls._VISIBLE_DEVICES)
        if vis is None:
            return None
        devs = [int(x) for x in vis.split(",") if x.strip() != ""]
        if n_local <= 0 or len(devs) % n_local != 0:
            logger.warning(f"visible devices {devs} do not divide evenly among {n_local} local tasks")
            return None
        per = len(devs) // n_local
        return devs[local_id * per:(local_id + 1) * per]


@dataclass(frozen=True)
class DistributedConfig:
    coordinator_address: Optional[str] = None   # host:port of process 0
    num_processes: Optional[int] = None
    process_id: Optional[int] = None
    local_device_ids: Optional[Union[int, List[int]]] = None
    backend: Optional[str] = None               # nccl | gloo (default: nccl with CUDA, else gloo)
    timeout_minutes: float = 30.0

    def _is_distributed(self) -> bool:
        if self.coordinator_address is not None or self.num_processes is not None or self.process_id is not None:
            return True
        if "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1:
            return True
        return LevanterSlurmCluster.is_env_present() and LevanterSlurmCluster.get_process_count() > 1

    def initialize(self) -> None:
        """Initialise ``torch.distributed`` from explicit fields, the torchrun environment, or SLURM."""
        import torch.distributed as dist

        if dist.is_initialized() or not self._is_distributed():
            return
        env = os.environ
        if "WORLD_SIZE" in env and "RANK" in env and self.coordinator_address is None:
            world, rank = int(env["WORLD_SIZE"]), int(env["RANK"])
            addr = f"{env.get('MASTER_ADDR', '127.0.0.1')}:{env.get('MASTER_PORT', '29500')}"
            local_rank = int(env.get("LOCAL_RANK", "0"))
        elif LevanterSlurmCluster.is_env_present() and self.coordinator_address is None:
            world = self.num_processes or LevanterSlurmCluster.get_process_count()
            rank = self.process_id if self.process_id is not None else LevanterSlurmCluster.get_process_id()
            addr = LevanterSlurmCluster.get_coordinator_address()
            ids = LevanterSlurmCluster.get_local_device_ids_for_process()
            local_rank = ids[0] if ids else LevanterSlurmCluster.get_local_process_id()
        else:
            if self.coordinator_address is None or self.num_processes is None or self.process_id is None:
                raise ValueError("coordinator_address, num_processes and process_id must all be given")
            world, rank, addr = self.num_processes, self.process_id, self.coordinator_address
            ids = self.local_device_ids
            local_rank = (ids if isinstance(ids, int) else ids[0]) if ids is not None else rank % max(torch.cuda.device_count(), 1)
        backend = self.backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if torch.cuda.is_available():
            torch.cuda.set_device(local_rank % torch.cuda.device_count())
        host, port = addr.rsplit(":", 1)
        logger.info(f"initialising torch.distributed: backend={backend} rank={rank}/{world} coordinator={addr}")
        kwargs = {}
        if backend == "nccl" and torch.cuda.is_available():
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, init_method=f"tcp://{host}:{port}", world_size=world, rank=rank,
                                timeout=timedelta(minutes=self.timeout_minutes), **kwargs)


@dataclass
class RayConfig:
    """Accepted for config compatibility (src/levanter/distributed.py:376-384); preprocessing here uses local worker
    processes, so no Ray cluster is started."""

    address: Optional[str] = None
    start_workers: bool = True
    auto_start_cluster: bool = True

    def initialize(self):
        if self.address is not None:
            logger.info("a Ray address was configured; this framework tokenises with local worker processes instead")
        if self.auto_start_cluster and self.address is not None:
            auto_ray_cluster(address=self.address, start_workers=self.start_workers)


_ray_initialized = False


def auto_ray_cluster(address: Optional[str] = None, namespace: Optional[str] = "levanter", start_workers: bool = True,
                     fail_if_cluster_already_initialized: bool = False, **kwargs) -> bool:
    """Join (or, on the first SLURM node, start) a Ray cluster for users whose own preprocessing uses Ray
    (src/levanter/distributed.py:200-312).  The address comes from the argument, ``RAY_ADDRESS``, or the first node of the
    SLURM allocation with a port derived from the job id.  Nothing in this framework needs Ray (caches are built by local
    worker processes), so without the ``ray`` package this logs and returns False instead of failing; a second call is ignored
    as in the reference.  Returns True when ``ray.init`` ran."""
    global _ray_initialized
    if _ray_initialized:
        logger.warning("auto_ray_cluster has already been called. Ignoring subsequent calls.")
        return False
    try:
        import ray  # type: ignore
    except ImportError:
        logger.info("ray is not installed: no Ray cluster is started (none is needed by this framework)")
        return False
    if address is None:
        address = os.environ.get("RAY_ADDRESS")
    if address is None and LevanterSlurmCluster.is_env_present():
        cluster = LevanterSlurmCluster()
        host = cluster.get_coordinator_address().split(":")[0]
        port = 6379 + int(os.environ.get("SLURM_JOB_ID", "0")) % 1000
        address = f"{host}:{port}"
        if cluster.get_process_id() == 0 and is_local_leader():
            import subprocess

            subprocess.run(["ray", "start", "--head", "--port", str(port)], check=False)
        elif start_workers and is_local_leader():
            import subprocess

            subprocess.run(["ray", "start", "--address", address], check=False)
    if ray.is_initialized() and fail_if_cluster_already_initialized:
        raise RuntimeError("a Ray cluster is already initialised in this process")
    ray.init(address=address, namespace=namespace, ignore_reinit_error=not fail_if_cluster_already_initialized, **kwargs)
    _ray_initialized = True
    return True


def is_local_leader() -> bool:
    """True for exactly one process per node (by ``LOCAL_RANK``/``SLURM_LOCALID``; falls back to a file lock)."""
    for k in ("LOCAL_RANK", "SLURM_LOCALID"):
        if k in os.environ:
            return int(os.environ[k]) == 0
    try:
        import atexit
        import tempfile

        from filelock import FileLock, Timeout

        path = os.path.join(tempfile.gettempdir(), f"levanter_b200_leader_{os.environ.get('SLURM_JOB_ID', 'local')}.lock")
        lock = FileLock(path)
        try:
            lock.acquire(timeout=0.1)
            atexit.register(lock.release)
            return True
        except Timeout:
            return False
    except ImportError:
        return True


def barrier_sync(timeout: float = 200.0) -> None:
    """Named barrier with a timeout (src/levanter/utils/jax_utils.py:117-134)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def sync_global_devices(name: str = "sync", timeout: float = 200.0) -> None:
    """Every process reaches this point before any goes on (the reference's barrier before uploads,
    src/levanter/utils/cloud_utils.py:169; src/levanter/compat/hf_checkpoints.py:1099).  ``name`` only labels the log line."""
    logger.debug(f"barrier: {name}")
    barrier_sync(timeout)


def broadcast_one_to_all(obj, src: int = 0):
    """Ship a small Python object from one process to all (run-id seed, checkpoint-save decision)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=src)
    return box[0]


def process_index() -> int:
    """Rank of this process in the job (0 when ``torch.distributed`` is not initialised and no launcher variable is set)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.get_rank()
    return int(os.environ.get("RANK", os.environ.get("SLURM_PROCID", "0")))


def process_count() -> int:
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size()
    return int(os.environ.get("WORLD_SIZE", os.environ.get("SLURM_NTASKS", "1")))
