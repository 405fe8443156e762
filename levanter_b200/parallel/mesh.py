"""Device mesh with the reference's three logical axes ``(replica, data, model)``
(src/levanter/utils/jax_utils.py:328-348, src/levanter/trainer.py:798-875).

One process drives one GPU.  ``model`` (tensor parallel) is the fastest-varying axis so that a TP group sits on
adjacent ranks, ``data`` (FSDP shards + data parallel) comes next and ``replica`` (pure data-parallel replicas of the
sharded state, HSDP) is outermost.  Groups are ``torch.distributed`` process groups: NCCL on GPUs, gloo on CPU.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class MeshAxis:
    name: str
    size: int
    rank: int
    group: Optional[dist.ProcessGroup]
    ranks: List[int]


class DeviceMesh:
    def __init__(self, replica: int = 1, data: Optional[int] = None, model: int = 1, *, world_size: Optional[int] = None,
                 rank: Optional[int] = None, create_groups: bool = True):
        initialized = dist.is_available() and dist.is_initialized()
        self.world_size = world_size if world_size is not None else (dist.get_world_size() if initialized else 1)
        self.rank = rank if rank is not None else (dist.get_rank() if initialized else 0)
        if data is None or data == -1:
            if self.world_size % (replica * model) != 0:
                raise ValueError(f"world size {self.world_size} not divisible by replica*model = {replica * model}")
            data = self.world_size // (replica * model)
        if replica * data * model != self.world_size:
            raise ValueError(f"mesh {replica}x{data}x{model} does not match world size {self.world_size}")
        self.shape = (replica, data, model)
        r = self.rank
        self.model_rank = r % model
        self.data_rank = (r // model) % data
        self.replica_rank = r // (model * data)
        self.axes = {}
        for name, size in (("replica", replica), ("data", data), ("model", model)):
            ranks = self.ranks_along(name)
            group = None
            if create_groups and initialized and size > 1:
                group = self._make_group(name)
            self.axes[name] = MeshAxis(name, size, ranks.index(self.rank), group, ranks)
        # batch axis = (replica, data): all ranks with the same model rank
        self.batch_ranks = [q for q in range(self.world_size) if q % model == self.model_rank]
        self.batch_group = None
        if create_groups and initialized and len(self.batch_ranks) > 1:
            if replica == 1:
                self.batch_group = self.axes["data"].group
            elif data == 1:
                self.batch_group = self.axes["replica"].group
            else:
                self.batch_group = self._make_custom_groups(
                    [[q for q in range(self.world_size) if q % model == m] for m in range(model)])

    def coords(self, rank: int):
        replica, data, model = self.shape
        return rank // (model * data), (rank // model) % data, rank % model

    def ranks_along(self, axis: str, rank: Optional[int] = None) -> List[int]:
        replica, data, model = self.shape
        rr, dr, mr = self.coords(self.rank if rank is None else rank)
        if axis == "model":
            return [rr * data * model + dr * model + m for m in range(model)]
        if axis == "data":
            return [rr * data * model + d * model + mr for d in range(data)]
        if axis == "replica":
            return [q * data * model + dr * model + mr for q in range(replica)]
        raise KeyError(axis)

    def _make_group(self, axis: str):
        seen = []
        for q in range(self.world_size):
            ranks = self.ranks_along(axis, q)
            if ranks not in seen:
                seen.append(ranks)
        return self._make_custom_groups(seen)

    def _make_custom_groups(self, groups: List[List[int]]):
        mine = None
        for ranks in groups:  # every process must create every group, in the same order
            g = dist.new_group(ranks)
            if self.rank in ranks:
                mine = g
        return mine

    # -- sizes the trainer needs (src/levanter/trainer.py:757-844) ------------------------------------------------
    @property
    def replica_size(self) -> int:
        return self.shape[0]

    @property
    def data_size(self) -> int:
        return self.shape[1]

    @property
    def model_size(self) -> int:
        return self.shape[2]

    @property
    def batch_size_divisor(self) -> int:
        """Number of distinct data shards = replica * data."""
        return self.shape[0] * self.shape[1]

    @property
    def batch_index(self) -> int:
        return self.replica_rank * self.shape[1] + self.data_rank

    @property
    def data_group(self):
        return self.axes["data"].group

    @property
    def model_group(self):
        return self.axes["model"].group

    @property
    def replica_group(self):
        return self.axes["replica"].group


def create_fsdp_mesh(replica_ici_axis_size: int = 1, data_axis_size: Optional[int] = None, model_axis_size: int = 1,
                     replica_dcn_axis_size: int = 1) -> DeviceMesh:
    """Mesh from the trainer's axis sizes; the ``dcn`` (multi-slice) replica factor multiplies the replica axis."""
    return DeviceMesh(replica_ici_axis_size * replica_dcn_axis_size, data_axis_size, model_axis_size)


def local_device() -> torch.device:
    if torch.cuda.is_available():
        idx = int(os.environ.get("LOCAL_RANK", "0")) % max(torch.cuda.device_count(), 1)
        return torch.device("cuda", idx)
    return torch.device("cpu")
