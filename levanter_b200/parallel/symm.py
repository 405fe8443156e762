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

    total_bytes = 0  # bytes allocated through this class by this process (the caching allocator's statistics do not see them)

    def __init__(self, numel: int, dtype: torch.dtype, device, group):
        SymmetricBuffer.total_bytes += int(numel) * torch.empty((), dtype=dtype).element_size()
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


def wait_for_flag(flag: "torch.Tensor", target: int, limit_seconds: float = 1.0, *, system_scope: bool = True):
    """Wait on the device (one thread, bounded) until ``flag[0] >= target``.  Returns ``(reached, last_value, waited_seconds)``
    after a synchronisation of the current stream; a wait that ran out also leaves ``flag wait timed out`` in the library's
    status word, which the caller clears with ``ops.lib.check_status`` (it raises) or ``ops.lib.clear_status``.  The CUDA
    context stays usable whatever the outcome."""
    import torch

    from ..ops import lib

    assert flag.is_cuda and flag.dtype == torch.int32
    result = torch.zeros(4, dtype=torch.int32, device=flag.device)
    f = lib.fn("lvb_flag_wait_probe", [lib.c_void_p, lib.c_int, lib.ctypes.c_ulonglong, lib.c_int, lib.c_void_p, lib.c_void_p, lib.c_void_p])
    rc = f(flag.data_ptr(), int(target), int(limit_seconds * 1e9), 1 if system_scope else 0, result.data_ptr(),
           lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_flag_wait_probe")
    r = result.tolist()
    waited = ((r[3] & 0xFFFFFFFF) << 32 | (r[2] & 0xFFFFFFFF)) * 1e-9
    return r[0] == 1, r[1], waited
