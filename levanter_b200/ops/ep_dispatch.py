"""Bindings of the expert-parallel exchange kernels (``csrc/ep_dispatch.cu``): the count all-gather by peer stores and the
row push / pull that carries the router's permutation.  The functions take raw peer addresses so that the same kernels can
be driven by symmetric memory across processes (``parallel/expert.py``) or, in tests, by several buffers on one device that
stand in for the ranks (the kernels never wait on one another, so running the ranks' launches one after the other is the
same computation)."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import lib

PAD = 128

_f = {}


def _bind():
    if not _f:
        P, I = lib.c_void_p, lib.c_int
        _f["counts"] = lib.fn("lvb_ep_counts_push", [P, P, I, I, I, P])
        _f["rows"] = lib.fn("lvb_ep_rows", [I, P, I, I, I, P, P, I, P, I, I, I, P, P, I, P, P])


def ptr_array(ptrs: Sequence[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def counts_push(counts: torch.Tensor, table_ptrs, world: int, rank: int) -> None:
    """Write ``counts[E]`` (int32) into row ``rank`` of every rank's ``[world, E]`` table."""
    _bind()
    assert counts.dtype == torch.int32 and counts.is_contiguous()
    rc = _f["counts"](counts.data_ptr(), ctypes.cast(table_ptrs, ctypes.c_void_p), world, rank, counts.numel(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_ep_counts_push")


def rows(push: bool, table: torch.Tensor, world: int, rank: int, local: torch.Tensor, index: Optional[torch.Tensor], div: int,
         buf_ptrs, num_rows: int, cap: int, offsets: Optional[torch.Tensor] = None, tile_group: Optional[torch.Tensor] = None,
         clear_padding: bool = False) -> None:
    """Move this rank's ``num_rows`` expert-sorted rows to (``push``) or from the owners' buffers; see the kernel file."""
    _bind()
    E = table.numel() // world
    assert table.dtype == torch.int32 and local.is_contiguous() and local.element_size() == 2
    assert index is None or (index.dtype == torch.int64 and index.is_contiguous())
    rc = _f["rows"](1 if push else 0, table.data_ptr(), world, rank, E, local.data_ptr(), lib.ptr(index), div,
                    ctypes.cast(buf_ptrs, ctypes.c_void_p), local.shape[-1], num_rows, cap, lib.ptr(offsets), lib.ptr(tile_group),
                    1 if clear_padding else 0, lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_ep_rows")


def capacity_rows(rows_per_rank: int, n_local: int, factor: float) -> int:
    """Rows of the exchange buffer: ``factor`` times a balanced share plus the worst-case padding, a multiple of 128."""
    need = int(rows_per_rank * factor) + n_local * (PAD - 1)
    return (need + PAD - 1) // PAD * PAD
