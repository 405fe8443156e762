"""ctypes binding to the in-tree sm_100a kernel library.

The library is loaded lazily the first time a kernel is needed.  On a machine
with a CUDA device a missing or unloadable library is an error (never a silent
fallback to eager PyTorch); on a CPU-only machine :func:`available` is False and
callers use their PyTorch reference implementations.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from . import build as _build

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_status: dict[int, torch.Tensor] = {}

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_float = ctypes.c_float
c_longlong = ctypes.c_longlong


def cuda_ok() -> bool:
    return torch.cuda.is_available()


_tls = threading.local()


class reference_ops:
    """Context manager: inside it :func:`available` is False on this thread, so every op takes its differentiable PyTorch
    statement.  Used for passes that need second derivatives (Sophia's Hessian-vector product): the hand-written kernels
    define first derivatives only."""

    def __enter__(self):
        self._prev = getattr(_tls, "reference", 0)
        _tls.reference = self._prev + 1
        return self

    def __exit__(self, *exc):
        _tls.reference = self._prev
        return False


def available() -> bool:
    """True when the native kernels can run here (a CUDA device of compute capability 10.x)."""
    if getattr(_tls, "reference", 0):
        return False
    if not cuda_ok():
        return False
    major, _ = torch.cuda.get_device_capability()
    return major == 10


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.lib_path()
            if not path.exists():
                path = _build.build()
            _lib = ctypes.CDLL(str(path))
    return _lib


launch_count = 0  # kernels launched through this binding since import (see count_launches)


def fn(name: str, argtypes: list, restype=c_int, launches: int = 1):
    """Bind an ``extern "C"`` launcher.  ``launches`` is how many kernels one call puts on the stream; the running total
    is kept in ``launch_count`` so benchmarks can report how many of this library's kernels ran in a timed region."""
    f = getattr(load(), name)
    f.argtypes = argtypes
    f.restype = restype
    if launches <= 0:
        return f

    def counted(*args):
        global launch_count
        launch_count += launches
        return f(*args)

    counted.__name__ = name
    return counted


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def status_buffer() -> torch.Tensor:
    """Per-device int32[8] word that kernels write a timeout / bounds code into."""
    dev = torch.cuda.current_device()
    buf = _status.get(dev)
    if buf is None:
        buf = torch.zeros(8, dtype=torch.int32, device=f"cuda:{dev}")
        if _wait_limit_ms:
            buf[4] = _wait_limit_ms
        _status[dev] = buf
    return buf


class KernelStatusError(RuntimeError):
    pass


_wait_limit_ms = 0


def set_wait_limit(seconds: float) -> None:
    """Limit of the kernels' bounded waits (default 2 s).  Set it above the largest skew expected between ranks: a rank that
    reaches a peer-synchronised kernel later than that (a rank-0-only hook, an uneven checkpoint copy) makes its peers' waits
    run out, which the step loop then reports as :class:`KernelStatusError`."""
    global _wait_limit_ms
    _wait_limit_ms = max(0, int(seconds * 1000))
    for buf in _status.values():
        buf[4] = _wait_limit_ms


def check_status(reset: bool = True) -> None:
    """Read the status word (device->host sync) and raise if a kernel recorded a failure."""
    if not _status:
        return
    for dev, buf in _status.items():
        vals = buf.tolist()
        if vals[0] != 0:
            if reset:
                buf[:4].zero_()
            names = {1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bad argument", 4: "bounds check"}
            hint = ""
            if vals[0] == 4 and vals[2] in (30, 31, 32):
                hint = (": the expert-parallel exchange received more rows than its capacity and dropped some; raise "
                        "expert_capacity_factor or select ep_comm: nccl")
            elif vals[0] in (1, 2):
                hint = ": a peer did not arrive within the wait limit (see TrainerConfig.kernel_wait_limit)"
            raise KernelStatusError(
                f"kernel status on cuda:{dev}: {names.get(vals[0], vals[0])} "
                f"(cta={vals[1]}, site={vals[2]}, extra={vals[3]}){hint}"
            )


def clear_status() -> None:
    """Zero the status word without raising (after a time-out the caller expected)."""
    for buf in _status.values():
        buf[:4].zero_()


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        names = {-1: "bad argument", -2: "CUDA launch error", -3: "tensor-map encode failed", -4: "size beyond limit"}
        raise RuntimeError(f"{what}: {names.get(rc, rc)}")
