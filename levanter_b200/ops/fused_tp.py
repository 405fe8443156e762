"""Tensor-parallel GEMMs with their collective fused in, for the sequence-parallel layout (activations split by rows over
the ranks of the model axis; weights split by columns or rows as in Megatron).

* :func:`all_gather_matmul` (column-parallel side): ``Y[M, N/W] = concat_r(X_r) W_shard^T``.  No gathered copy of ``X`` is
  ever made: the GEMM's TMA producer reads each row block straight from the memory of the rank that owns it, so the
  transfer of block ``i + 1`` overlaps the tensor-core work on block ``i`` inside one kernel.
* :func:`matmul_reduce_scatter` (row-parallel side): ``Y_r[M/W, N] = sum_s (X_s W_s^T)[rows of r]``.  The GEMM epilogue stores
  every finished tile into the staging slot of the rank that owns those rows (peer stores, tile by tile while later tiles
  are still being computed); after a barrier each rank sums its ``W`` slots.

Both need the activation / staging buffers in symmetric memory (:class:`levanter_b200.parallel.symm.SymmetricBuffer`).  The
reference obtains these collectives from XLA's SPMD partitioner (src/levanter/trainer.py:846-875)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..parallel.symm import SymmetricBuffer
from . import lib

_f = {}


def _fn(name, argtypes, launches=1):
    if name not in _f:
        _f[name] = lib.fn(name, argtypes, launches=launches)
    return _f[name]


def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def all_gather_matmul(x_sym: SymmetricBuffer, rows: int, k: int, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                      bias: Optional[torch.Tensor] = None, sync: bool = True) -> torch.Tensor:
    """``x_sym.tensor[:rows * k]`` viewed ``[rows, k]`` (bf16) is this rank's shard; ``w[N, k]`` bf16.  Returns ``[W * rows, N]``."""
    c = lib
    W = x_sym.world
    N = w.shape[0]
    M = rows * W
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=w.device)
    if sync:
        x_sym.barrier(0)  # every rank's shard is complete
    f = _fn("lvb_gemm_allgather_a", [c.c_void_p, c.c_int, c.c_void_p, c.c_void_p] + [c.c_int] * 7 + [c.c_float, c.c_void_p, c.c_void_p, c.c_void_p])
    flags = 0
    if bias is not None:
        flags |= 4 | (16 if bias.dtype == torch.float32 else 0)
    rc = f(x_sym.c_ptrs, W, w.data_ptr(), out.data_ptr(), M, N, k, k, w.stride(0), out.stride(0), flags, 1.0, lib.ptr(bias),
           lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_gemm_allgather_a")
    if sync:
        x_sym.barrier(1)  # peers are done reading this rank's shard: it may be overwritten
    return out


def matmul_reduce_scatter(x: torch.Tensor, w: torch.Tensor, staging: SymmetricBuffer, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[M, k_shard]``, ``w[N, k_shard]`` bf16 partial operands; ``staging``: fp32 symmetric buffer of at least ``M * N``
    elements, laid out ``[W, M / W, N]``.  Returns this rank's ``[M / W, N]`` bf16 rows of the summed product."""
    c = lib
    W, r = staging.world, staging.rank
    M, K = x.shape
    N = w.shape[0]
    rows = M // W
    slot = rows * N
    ptrs = _ptr_array([p + r * slot * 4 for p in staging.peer_ptrs])  # this rank's slot in every rank's staging buffer
    f = _fn("lvb_gemm_scatter_c", [c.c_void_p, c.c_void_p, c.c_void_p] + [c.c_int] * 8 + [c.c_float, c.c_void_p, c.c_void_p])
    rc = f(x.data_ptr(), w.data_ptr(), ptrs, W, M, N, K, x.stride(0), w.stride(0), N, 1, 1.0, lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_gemm_scatter_c")
    staging.barrier(0)  # every rank's partial tiles have landed
    if out is None:
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
    g = _fn("lvb_sum_slots", [c.c_void_p, c.c_longlong, c.c_int, c.c_void_p, c.c_void_p, c.c_longlong, c.c_void_p])
    rc = g(staging.tensor.data_ptr(), slot, W, 0, out.data_ptr(), slot, lib.stream_ptr())
    lib.check_rc(rc, "lvb_sum_slots")
    staging.barrier(1)  # the staging buffer may be reused
    return out
