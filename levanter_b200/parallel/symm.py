"""Symmetric (peer-mapped) device buffers for the fused compute+collective kernels.

A buffer allocated here has the same size on every rank of a process group and, after the rendezvous, every rank knows the
device address of every peer's copy: kernels read and write peers directly over NVLink.  Built on
``torch.distributed._symmetric_memory`` (CUDA virtual-memory handles exchanged between the processes of one node)."""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist


class SymmetricBuffer:
    """``tensor`` is this rank's copy; ``peer_ptrs[r]`` the address of rank ``r``'s copy as seen from this device."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group):
        import torch.distributed._symmetric_memory as symm_mem

        if group is None:
            group = dist.group.WORLD
        self.group = group
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.world = self.handle.world_size
        self.rank = self.handle.rank
        self.peer_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self._c_ptrs = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        try:  # one address that reaches every rank's copy through the switch (0 when the fabric has no such mapping)
            self.multicast_ptr = int(self.handle.multicast_ptr or 0)
        except Exception:  # noqa: BLE001
            self.multicast_ptr = 0

    @property
    def c_ptrs(self):
        """``void* const*`` argument for the kernel launchers (a host array; the launcher copies it into kernel parameters)."""
        return self._c_ptrs

    def barrier(self, channel: int = 0) -> None:
        """All ranks' work queued so far on the current stream is complete and visible before any rank goes on (a device-side
        barrier on the signal pads: the host does not block)."""
        self.handle.barrier(channel=channel)


def p2p_available(group) -> bool:
    if not (torch.cuda.is_available() and dist.is_available() and dist.is_initialized()):
        return False
    try:
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
    except Exception:  # noqa: BLE001
        return False
    return dist.get_world_size(group) > 1
