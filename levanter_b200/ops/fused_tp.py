"""Tensor-parallel GEMMs with their collective fused in, for the sequence-parallel layout (activations split by rows over
the ranks of the model axis; weights split by columns or rows as in Megatron).

* :func:`all_gather_matmul` (column-parallel side): ``Y[M, N/W] = concat_r(X_r) W_shard^T`` in ONE kernel.  The tile raster
  starts with this rank's own rows; meanwhile a copy warp in every CTA pulls the other ranks' shards over NVLink into local
  memory with bulk copies (each remote byte crosses the link once), nearest rank first, and bumps an arrival counter per
  128-row block; the TMA producer waits on that counter (bounded) before it multiplies a remote block.
* :func:`matmul_reduce_scatter` (row-parallel side): ``Y_r[M/W, N] = sum_s (X_s W_s^T)[rows of r]`` in ONE kernel.  The raster
  starts with the rows of the next rank; the epilogue stores every finished fp32 tile into the staging slot of the rank that
  owns those rows (peer stores, while later tiles are still being computed) and bumps that rank's per-tile counter; the
  own rows come last, and each CTA finally sums its share of the own rows' tiles over the slots as their counters fill.

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
    """``x_sym.tensor[:rows * k]`` viewed ``[rows, k]`` (bf16) is this rank's shard; ``w[N, k]`` bf16.  Returns ``[W * rows, N]``.

    With ``sync`` the call is bracketed by two cross-rank barriers (shards complete before, shards reusable after); a caller
    that orders the ranks itself passes ``sync=False``."""
    c = lib
    W = x_sym.world
    N = w.shape[0]
    M = rows * W
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=w.device)
    scratch = x_sym.__dict__.setdefault("_gather_scratch", {})
    if (M, k) not in scratch:
        n_cnt = _fn("lvb_gemm_allgather_a_counters", [c.c_int], launches=0)(M)
        scratch[(M, k)] = (torch.empty(M * k, dtype=torch.bfloat16, device=w.device), torch.zeros(n_cnt, dtype=torch.int32, device=w.device))
    a_local, a_cnt = scratch[(M, k)]
    if sync:
        x_sym.barrier(0)  # every rank's shard is complete
    f = _fn("lvb_gemm_allgather_a", [c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p] + [c.c_int] * 6
            + [c.c_float, c.c_void_p, c.c_void_p, c.c_void_p], launches=2)
    flags = 0
    if bias is not None:
        flags |= 4 | (16 if bias.dtype == torch.float32 else 0)
    rc = f(x_sym.c_ptrs, x_sym.rank, W, a_local.data_ptr(), a_cnt.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, k, w.stride(0),
           out.stride(0), flags, 1.0, lib.ptr(bias), lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_gemm_allgather_a")
    if sync:
        x_sym.barrier(1)  # peers are done reading this rank's shard: it may be overwritten
    return out


def scatter_m_order(M: int, world: int, rank: int, block: int = 128) -> list:
    """Order in which a reduce-scatter GEMM visits the ``block``-row blocks of an ``M``-row product (128 rows for the one-CTA
    kernel, 256 for the CTA-pair kernel): the blocks are dealt out to the ranks that own them in turn (a block belongs to
    the owner of its first row), next rank first and own rank last in each round, so that every rank's rows are produced at a
    steady rate by all ranks at once."""
    rows = M // world
    per_owner = [[] for _ in range(world)]
    for b in range((M + block - 1) // block):
        per_owner[min((b * block) // rows, world - 1)].append(b)
    owners = [(rank + 1 + i) % world for i in range(world)]
    order = []
    for i in range(max(len(x) for x in per_owner)):
        for d in owners:
            if i < len(per_owner[d]):
                order.append(per_owner[d][i])
    return order


_m_order_cache = {}


def m_order_tensor(M: int, world: int, rank: int, device, block: int = 128) -> torch.Tensor:
    key = (M, world, rank, str(device), block)
    t = _m_order_cache.get(key)
    if t is None:
        t = _m_order_cache[key] = torch.tensor(scatter_m_order(M, world, rank, block), dtype=torch.int32, device=device)
    return t


def rs_counters(rows: int, N: int) -> int:
    """Arrival counters of one staging area for an owner's ``[rows, N]`` slice (one per 32 rows x column tile)."""
    return ((rows + 31) // 32) * ((N + 255) // 256 if N > 128 else 1)


def reduce_scatter_staging_elems(M: int, N: int, dtype: torch.dtype = torch.float32) -> int:
    """Elements of ``dtype`` (fp32 or bf16) of symmetric staging that :func:`matmul_reduce_scatter` needs for an ``[M, N]``
    product: two areas (used alternately), each of ``W`` slots plus its int32 arrival counters."""
    return 2 * _rs_area_elems(M, N, dtype)


def _rs_area_elems(M, N, dtype):
    cnt = rs_counters(M, N)  # an upper bound on the counters of one rank's slice, whatever the number of ranks
    return (M * N + cnt * (4 // dtype.itemsize) + 127) // 128 * 128  # keeps the second area 256-byte aligned


def _rs_fn():
    c = lib
    return _fn("lvb_gemm_reduce_scatter", [c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_void_p,
                                           c.c_longlong, c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int] + [c.c_int] * 6
               + [c.c_float, c.c_void_p, c.c_void_p])


def _rs_pair_fn():
    c = lib
    return _fn("lvb_gemm_reduce_scatter_pair", [c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_void_p,
                                                c.c_longlong, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int] + [c.c_int] * 6
               + [c.c_float, c.c_void_p, c.c_void_p])


def reduce_scatter_gemm(a: torch.Tensor, b: torch.Tensor, mn_major: bool, slots, cnts, rank: int, world: int, staging_ptr: int, slot_elems: int,
                        staging_f32: bool, target: int, out: torch.Tensor, accumulate: bool, M: int, N: int, K: int, alpha: float) -> None:
    """One launch of the fused GEMM -> reduce-scatter (see ``lvb_gemm_reduce_scatter`` in ``csrc/gemm_bf16.cu`` for the
    protocol): the CTA-pair kernel for fp32 staging and more than 128 output columns, the one-CTA kernel otherwise."""
    from .gemm import PAIR_ENABLED

    out_f32 = 1 if out.dtype == torch.float32 else 0
    if PAIR_ENABLED and staging_f32 and N > 128:
        rc = _rs_pair_fn()(a.data_ptr(), b.data_ptr(), int(mn_major), int(mn_major), slots, cnts, rank, world, staging_ptr, slot_elems, target,
                           m_order_tensor(M, world, rank, a.device, 256).data_ptr(), out.data_ptr(), out.stride(0), out_f32, int(accumulate),
                           M, N, K, a.stride(0), b.stride(0), N, float(alpha), lib.status_buffer().data_ptr(), lib.stream_ptr())
        lib.check_rc(rc, "lvb_gemm_reduce_scatter_pair")
        return
    rc = _rs_fn()(a.data_ptr(), b.data_ptr(), int(mn_major), int(mn_major), slots, cnts, rank, world, staging_ptr, slot_elems,
                  1 if staging_f32 else 0, target, m_order_tensor(M, world, rank, a.device).data_ptr(), out.data_ptr(), out.stride(0), out_f32,
                  int(accumulate), M, N, K, a.stride(0), b.stride(0), N, float(alpha), lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_gemm_reduce_scatter")


def matmul_reduce_scatter(x: torch.Tensor, w: torch.Tensor, staging: SymmetricBuffer, out: Optional[torch.Tensor] = None,
                          _local_only: bool = False) -> torch.Tensor:
    """``x[M, k_shard]``, ``w[N, k_shard]`` bf16 partial operands; ``staging``: symmetric buffer of at least
    :func:`reduce_scatter_staging_elems` elements, used for products of this one shape only.  Its dtype picks the precision
    of the partial products on the wire: fp32, or bf16 (half the traffic; what a bf16 NCCL reduce-scatter rounds to).  The
    sum itself is always fp32.  Returns this rank's ``[M / W, N]`` rows of the summed product (bf16, or the dtype of ``out``).

    No barrier and no counter reset happen per call: the kernel alternates between the buffer's two areas and its arrival
    counters only grow (the first call on a buffer clears it and synchronises the ranks once)."""
    W, r = staging.world, staging.rank
    M, K = x.shape
    N = w.shape[0]
    rows = M // W
    slot = rows * N
    st = staging.tensor
    es = st.dtype.itemsize
    area = _rs_area_elems(M, N, st.dtype)
    assert st.dtype in (torch.float32, torch.bfloat16) and st.numel() >= 2 * area, "staging buffer"
    state = staging.__dict__.setdefault("_rs_state", {"shape": (M, N), "calls": 0})
    assert state["shape"] == (M, N), "a reduce-scatter staging buffer serves one product shape"
    if state["calls"] == 0:
        st.zero_()
        staging.barrier(0)  # every rank's counters are clear before anyone adds to them
    n = state["calls"]
    state["calls"] = n + 1
    base = (n & 1) * area * es  # byte offset of this call's area
    target = W * (n // 2 + 1)
    if out is None:
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
    slots = _ptr_array([p + base + r * slot * es for p in staging.peer_ptrs])  # this rank's slot in every rank's area
    cnts = _ptr_array([p + base + W * slot * es for p in staging.peer_ptrs])
    if _local_only:
        # timing aid: the same kernel with every store kept on this GPU (slot d of the own area stands in for rank d's
        # memory; the counters still fill up, the sums are meaningless).  Shows what the NVLink stores cost.
        own = staging.peer_ptrs[r]
        slots = _ptr_array([own + base + d * slot * es for d in range(W)])
        cnts = _ptr_array([own + base + W * slot * es] * W)
    reduce_scatter_gemm(x, w, False, slots, cnts, r, W, st.data_ptr() + base, slot, st.dtype == torch.float32, target, out, False, M, N, K, 1.0)
    return out
