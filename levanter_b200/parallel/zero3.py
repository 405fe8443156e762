"""Layer streaming for fully sharded training (ZeRO-3 / FSDP): the decoder layers' weight matrices exist only as ``1/W`` row
slices per rank; a layer's full weights are assembled just before they are needed and its weight gradients leave the GPU as
they are produced.

What the reference gets from sharding annotations (parameters stored sharded along ``embed`` over ``data``, XLA inserting a
per-layer all-gather in the scan body and a reduce-scatter of the gradients, src/levanter/trainer.py:206-210, 552-580,
862-875, docs/Levanter-1.0-Release.md:293-345) is an explicit schedule here:

* every streamed matrix ``[N, K]`` is cut by rows: rank ``r`` holds rows ``[r N/W, (r+1) N/W)`` in ``w_shard`` (compute dtype,
  peer-readable), and the fp32 master weights, optimizer moments and gradient accumulator of the same rows;
* two staging slots hold whole layers; layer ``l`` always lives in slot ``l % 2``, so a module parameter is a fixed view of its
  slot and what autograd saved in the forward pass is valid again in the backward pass once the layer has been re-assembled;
* ``ensure(l)`` (forward and backward pre-hooks of layer ``l``) makes layer ``l`` resident, ``prefetch`` names the layer that
  comes next (``l + 1`` going forward, ``l - 1`` going backward, ``L - 2`` at the turn);
* transports: ``nccl`` = one library all-gather per matrix when the layer is needed and one reduce-scatter per weight
  gradient (also the CPU/gloo path and the oracle of the tests); ``peer`` = the gather is a *copy job* (a table of 16 KB
  units: peer shard -> staging slot) that rides on the GEMM kernels of the layer before (a seventh warp per CTA issues bulk
  copies over NVLink while the tensor cores work, ``ops/csrc/gemm_bf16.cu``), and the weight-gradient GEMM stores its tiles
  straight into the owner's staging slots and sums the slots as they fill (``lvb_gemm_reduce_scatter``), so a rank ends the
  backward pass holding only its reduced fp32 gradient rows.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

COPY_UNIT = 16384  # bytes per unit of a copy job (the kernels' kCopyUnit)
ROW_GROUP = 32     # rows per unit of the reduce-scatter epilogue


@dataclass
class StreamParam:
    name: str
    param: nn.Parameter
    layer: int
    shape: Tuple[int, int]
    rows: int         # rows per rank
    stage_off: int    # elements, inside a staging slot
    shard_off: int    # elements, inside the per-rank streamed shard space (w_shard, and master/moments/gradients after stream_lo)

    @property
    def shard_numel(self) -> int:
        return self.rows * self.shape[1]


def eligible(p: torch.Tensor, world: int) -> bool:
    """Matrices whose rows split evenly into groups of 32 per rank and whose rows are whole 128-byte lines."""
    return (p.dim() == 2 and p.shape[0] % (world * ROW_GROUP) == 0 and p.shape[1] % 64 == 0 and getattr(p, "ep_dim", None) is None)


class GradSink:
    """Receiver of one streamed weight's gradient: ``sink(dy, x)`` computes ``dy^T x / W`` and leaves this rank's rows of the
    sum over ranks added to its fp32 gradient shard."""

    def __init__(self, streamer: "LayerStreamer", sp: StreamParam):
        self.streamer, self.sp = streamer, sp

    def __call__(self, dy2: torch.Tensor, x2: torch.Tensor) -> None:
        self.streamer.weight_grad(self.sp, dy2, x2)


class LayerStreamer:
    def __init__(self, layers: List[List[Tuple[str, nn.Parameter]]], modules: List[nn.Module], *, world: int, rank: int, group,
                 device: torch.device, compute_dtype: torch.dtype, comm: str):
        self.world, self.rank, self.group, self.device, self.cd = world, rank, group, device, compute_dtype
        self.modules = modules
        self.n_layers = len(layers)
        self.params: List[StreamParam] = []
        self.by_layer: List[List[StreamParam]] = []
        shard_off = 0
        slot_elems = 0
        for l, plist in enumerate(layers):
            row: List[StreamParam] = []
            stage_off = 0
            for name, p in plist:
                sp = StreamParam(name, p, l, (p.shape[0], p.shape[1]), p.shape[0] // world, stage_off, shard_off)
                row.append(sp)
                self.params.append(sp)
                stage_off += p.numel()
                shard_off += sp.shard_numel
            slot_elems = max(slot_elems, stage_off)
            self.by_layer.append(row)
        self.shard_numel = shard_off
        self.slot_elems = slot_elems
        self.layer_shard_off = [row[0].shard_off if row else 0 for row in self.by_layer]
        self.resident = [-1, -1]
        self.comm = comm
        self._sym_w = self._sym_stage = None
        self._pending: Optional[Tuple[int, int]] = None  # (layer being prefetched, next unit of its copy job)
        self._tables: Dict[tuple, Tuple[torch.Tensor, int]] = {}
        self._rs_calls = 0
        self._rs_uses: Dict[tuple, List[int]] = {}
        self._rs_cnt_n: Dict[tuple, int] = {}
        self.stats = {"gathers_standalone": 0, "units_on_gemms": 0, "units_standalone": 0, "fused_weight_grads": 0, "library_weight_grads": 0}
        use_peer = comm in ("p2p", "multimem") and device.type == "cuda" and compute_dtype == torch.bfloat16
        if use_peer:
            from .symm import SymmetricBuffer, p2p_available

            use_peer = p2p_available(group)
            if use_peer:
                try:
                    self._sym_w = SymmetricBuffer(self.shard_numel, compute_dtype, device, group)
                    self._alloc_scatter_arena()
                except Exception as e:  # noqa: BLE001 - every rank takes the same path: the rendezvous is collective
                    import logging

                    logging.getLogger(__name__).warning(f"symmetric memory unavailable ({e}); layer streaming uses library collectives")
                    self._sym_w = self._sym_stage = None
                    use_peer = False
        self.peer = use_peer
        self.w_shard = self._sym_w.tensor if use_peer else torch.zeros(self.shard_numel, dtype=compute_dtype, device=device)
        self.slots = [torch.zeros(slot_elems, dtype=compute_dtype, device=device) for _ in range(2)]
        self.grad_shard: Optional[torch.Tensor] = None  # set by the engine: fp32 view of the streamed region of its gradient shard

    def attach(self) -> None:
        """Take the parameters over (call once their initial values have been copied into the shards): every streamed parameter
        becomes a view of its staging slot, its weight gradient goes to a :class:`GradSink`, and the layers get their hooks."""
        for sp in self.params:
            sp.param.data = self.slots[sp.layer % 2][sp.stage_off:sp.stage_off + sp.param.numel()].view(sp.shape)
            sp.param.grad_sink = GradSink(self, sp)
            sp.param.register_post_accumulate_grad_hook(self._make_autograd_grad_hook(sp))
        for l, m in enumerate(self.modules):
            m.register_forward_pre_hook(self._make_fwd_hook(l))
            m.register_full_backward_pre_hook(self._make_bwd_hook(l))
        if self.peer:
            from ..ops.gemm import set_copy_job_provider

            set_copy_job_provider(self.take_copy_job)

    # ------------------------------------------------------------------------------------------ hooks
    def _make_fwd_hook(self, l: int) -> Callable:
        def hook(module, args):
            self.ensure(l)
            if l + 1 < self.n_layers:
                self.prefetch(l + 1)
            elif torch.is_grad_enabled() and self.n_layers >= 2:
                self.prefetch(l - 1)  # the backward pass starts with this layer and needs the one before it next

        return hook

    def _make_bwd_hook(self, l: int) -> Callable:
        def hook(module, grad_output):
            self.ensure(l)
            if l >= 1:
                self.prefetch(l - 1)

        return hook

    def _make_autograd_grad_hook(self, sp: StreamParam) -> Callable:
        def hook(param):
            g = param.grad
            if g is not None:
                param.grad = None
                self.reduce_full_grad(sp, g)

        return hook

    # ------------------------------------------------------------------------------------------ residency
    def invalidate(self) -> None:
        """The shards changed (optimizer step, checkpoint load): nothing in the staging slots is current any more."""
        self.resident = [-1, -1]
        self._pending = None

    def ensure(self, l: int) -> None:
        s = l % 2
        if self.resident[s] == l:
            if self._pending is not None and self._pending[0] == l:
                self._flush_pending()  # the copy job of this very layer has not been carried out completely yet
            return
        if self._pending is not None:
            self._flush_pending()
        self.gather_now(l)

    def prefetch(self, l: int) -> None:
        s = l % 2
        if self.resident[s] == l:
            return
        if self._pending is not None:
            if self._pending[0] == l:
                return
            self._flush_pending()
        if not self.peer:
            return  # the library transport gathers a layer when it is needed
        self.resident[s] = l
        self._pending = (l, 0)

    def gather_now(self, l: int) -> None:
        if self.peer:
            table, n_units = self._table_for(l)
            self._launch_copy(l, table, 0, n_units)
            self.stats["gathers_standalone"] += 1
            self.stats["units_standalone"] += n_units
        else:
            slot = self.slots[l % 2]
            for sp in self.by_layer[l]:
                out = slot[sp.stage_off:sp.stage_off + sp.param.numel()]
                dist.all_gather_into_tensor(out, self.w_shard[sp.shard_off:sp.shard_off + sp.shard_numel], group=self.group)
        self.resident[l % 2] = l

    # ------------------------------------------------------------------------------------------ copy jobs (peer transport)
    def _table_for(self, l: int) -> Tuple[torch.Tensor, int]:
        """Units of layer ``l``'s gather: for every matrix in the order the layer uses them, for every rank starting with the
        next one (this rank's own rows last), 16 KB pieces of that rank's slice -> their place in the staging slot.  Source
        offsets are relative to the layer's start in the shard space, so layers of equal structure share a table."""
        key = tuple((sp.shape, sp.stage_off, sp.shard_off - self.layer_shard_off[l]) for sp in self.by_layer[l])
        hit = self._tables.get(key)
        if hit is not None:
            return hit
        es = self.w_shard.element_size()
        rows = []
        for sp in self.by_layer[l]:
            nbytes = sp.shard_numel * es
            for i in range(self.world):
                r = (self.rank + 1 + i) % self.world
                src0 = (sp.shard_off - self.layer_shard_off[l]) * es
                dst0 = (sp.stage_off + r * sp.shard_numel) * es
                for off in range(0, nbytes, COPY_UNIT):
                    n = min(COPY_UNIT, nbytes - off)
                    rows.append((r, (src0 + off) // 16, (dst0 + off) // 16, n // 16))
        t = torch.tensor(rows, dtype=torch.int32, device=self.device).contiguous()
        self._tables[key] = (t, len(rows))
        return self._tables[key]

    def _src_ptrs(self, l: int):
        base = self.layer_shard_off[l] * self.w_shard.element_size()
        return (ctypes.c_void_p * self.world)(*[p + base for p in self._sym_w.peer_ptrs])

    def _launch_copy(self, l: int, table: torch.Tensor, u0: int, u1: int) -> None:
        from ..ops import lib

        c = lib
        f = lib.fn("lvb_copy_job", [c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_void_p])
        rc = f(table.data_ptr(), u0, u1, self._src_ptrs(l), self.world, self.slots[l % 2].data_ptr(), 0, lib.status_buffer().data_ptr(),
               lib.stream_ptr())
        lib.check_rc(rc, "lvb_copy_job")

    def _flush_pending(self) -> None:
        l, u = self._pending
        table, n_units = self._table_for(l)
        if u < n_units:
            self._launch_copy(l, table, u, n_units)
            self.stats["units_standalone"] += n_units - u
        self._pending = None

    def take_copy_job(self, flops: float):
        """Called by the GEMM binding before a launch: a share of the pending copy job sized to the GEMM (so that the copy
        warps are done before the tensor cores are), or ``None``.  Returns ``(table_ptr, u0, u1, src_ptrs, world, dst_ptr)``."""
        if self._pending is None:
            return None
        l, u = self._pending
        table, n_units = self._table_for(l)
        if u >= n_units:
            self._pending = None
            return None
        # a GEMM of `flops` lasts about flops / 1.4e15 s; let its copy warps move what ~350 GB/s carries in that time
        take = max(64, int(flops / 1.4e15 * 350e9 / COPY_UNIT))
        u1 = min(n_units, u + take)
        self._pending = (l, u1) if u1 < n_units else None
        self.stats["units_on_gemms"] += u1 - u
        return table.data_ptr(), u, u1, self._src_ptrs(l), self.world, self.slots[l % 2].data_ptr()

    # ------------------------------------------------------------------------------------------ weight gradients
    def _grad_rows(self, sp: StreamParam) -> torch.Tensor:
        return self.grad_shard[sp.shard_off:sp.shard_off + sp.shard_numel].view(sp.rows, sp.shape[1])

    def reduce_full_grad(self, sp: StreamParam, g: torch.Tensor) -> None:
        """A whole ``[N, K]`` gradient (from autograd, or from a GEMM the fused path does not cover): average over the ranks
        with the library's reduce-scatter and add this rank's rows to the gradient shard."""
        g = g.reshape(sp.shape).to(torch.float32).contiguous()
        out = torch.empty(sp.rows, sp.shape[1], dtype=torch.float32, device=g.device)
        dist.reduce_scatter_tensor(out, g, op=dist.ReduceOp.SUM, group=self.group)
        self._grad_rows(sp).add_(out, alpha=1.0 / self.world)
        self.stats["library_weight_grads"] += 1

    def weight_grad(self, sp: StreamParam, dy2: torch.Tensor, x2: torch.Tensor) -> None:
        from ..ops.gemm import gemm

        if not self.peer:
            self.reduce_full_grad(sp, gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32))
            return
        self._fused_weight_grad(sp, dy2, x2)

    def _alloc_scatter_arena(self) -> None:
        """Symmetric staging of the fused reduce-scatter: two data areas (used alternately from call to call, each as large as
        the largest streamed matrix in fp32) followed by two sets of arrival counters per distinct matrix shape."""
        from ..ops.fused_tp import rs_counters
        from .symm import SymmetricBuffer

        self._rs_area = max(sp.shape[0] * sp.shape[1] for sp in self.params)
        self._rs_area = (self._rs_area + 63) // 64 * 64
        shapes = sorted({sp.shape for sp in self.params})
        self._rs_cnt_off: Dict[tuple, int] = {}
        off = 2 * self._rs_area  # in fp32 elements == int32 elements
        for shp in shapes:
            n = (rs_counters(shp[0] // self.world, shp[1]) + 63) // 64 * 64
            self._rs_cnt_off[shp] = off
            self._rs_uses[shp] = [0, 0]
            off += 2 * n
            self._rs_cnt_n[shp] = n
        self._sym_stage = SymmetricBuffer(off, torch.float32, self.device, self.group)  # zeroed: the counters start at 0
        self._sym_stage.barrier(0)

    def _fused_weight_grad(self, sp: StreamParam, dy2: torch.Tensor, x2: torch.Tensor) -> None:
        from ..ops.fused_tp import _ptr_array, reduce_scatter_gemm
        from ..ops.gemm import _rowmajor_2d

        W, r = self.world, self.rank
        dy2, x2 = _rowmajor_2d(dy2), _rowmajor_2d(x2)
        T, N = dy2.shape
        K = x2.shape[1]
        assert (N, K) == sp.shape and x2.shape[0] == T
        parity = self._rs_calls & 1
        self._rs_calls += 1
        uses = self._rs_uses[sp.shape]
        uses[parity] += 1
        target = (W * uses[parity]) & 0xFFFFFFFF  # the kernel compares differences modulo 2^32
        if target >= 1 << 31:
            target -= 1 << 32
        slot = sp.rows * K  # fp32 elements per slot
        data_off = parity * self._rs_area * 4
        cnt_off = (self._rs_cnt_off[sp.shape] + parity * self._rs_cnt_n[sp.shape]) * 4
        peers = self._sym_stage.peer_ptrs
        slots = _ptr_array([p + data_off + r * slot * 4 for p in peers])  # this rank's slot in every rank's area
        cnts = _ptr_array([p + cnt_off for p in peers])
        out = self._grad_rows(sp)
        reduce_scatter_gemm(dy2, x2, True, slots, cnts, r, W, peers[r] + data_off, slot, True, target, out, True, N, K, T, 1.0 / W)
        self.stats["fused_weight_grads"] += 1

    # ------------------------------------------------------------------------------------------ whole tensors (export, checkpoints)
    def gather_full(self, sp: StreamParam, shard_rows: torch.Tensor) -> torch.Tensor:
        """``[N, K]`` from every rank's ``[N / W, K]`` rows of some per-rank state (master weights, a moment)."""
        out = torch.empty(sp.shape, dtype=shard_rows.dtype, device=shard_rows.device)
        dist.all_gather_into_tensor(out.view(-1), shard_rows.reshape(-1).contiguous(), group=self.group)
        return out
