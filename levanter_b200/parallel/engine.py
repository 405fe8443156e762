"""Sharded parameter / gradient / optimizer-state engine (FSDP over the mesh's ``data`` axis, replicas over ``replica``).

What the reference expresses with sharding annotations (parameters and optimizer state stored sharded along ``embed``
over ``data``; XLA all-gathers weights and reduce-scatters gradients, src/levanter/trainer.py:206-210,552-580,
862-875) is laid out explicitly here, sized for 180 GB of HBM per GPU:

* every trainable parameter lives in one flat **compute-dtype** buffer (``param_flat``); module parameters are views
  into it, grouped into per-layer *buckets*;
* weight gradients are accumulated in one flat **fp32** buffer (``grad_flat``): the tcgen05 GEMM epilogue adds each
  ``dW`` straight into its ``main_grad`` view, other parameters' ``.grad`` are folded in after backward;
* each bucket is cut into ``W`` equal slices; rank ``r`` owns slice ``r`` of every bucket: fp32 master weights and
  optimizer moments exist only for owned slices (ZeRO-style), so their memory drops by ``W`` while the bf16 weights
  and the fp32 gradient accumulator stay resident (20 B/param/W + 6 B/param; Llama-2-7B on 8 GPUs: about 57 GB);
* a step = reduce-scatter of each bucket's gradients (average over data ranks, then all-reduce over replicas),
  global-norm clip, optimizer update on the owned slices, and an all-gather of the refreshed compute-dtype slices.
  Because weights stay resident, communication is one reduce-scatter plus one all-gather *per step*, not per
  micro-batch and not per layer pass.

With ``zero_stage=3`` (more than one data rank, sharded optimizer) the weight matrices of the decoder layers leave this
scheme: they are cut by rows, every rank keeps only its rows (compute-dtype copy, fp32 master, moments, fp32 gradient
accumulator), whole layers are assembled in two staging slots just before use and weight gradients are reduce-scattered as
they are produced (``parallel/zero3.py``).  Everything else (embeddings, LM head, norms, biases) stays in the flat buffers
described above.  ``zero_stage=1`` is the scheme above for all parameters.

Optimizers run on ``{param path: 1-D view of the owned slice}`` trees, so any element-wise transformation chain works
sharded.  Optimizers that need whole matrices (Muon, SOAP, Kron, ...) run with ``shard_optimizer=False``: gradients are
all-reduced and every rank updates full tensors.  AdamW has a fused CUDA path (``ops/csrc/optim.cu``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config import Policy
from ..optim import transforms as T
from ..optim.config import AdamConfig, OptimizerConfig, ParamInfo

ALIGN = 128  # elements; keeps every parameter 256-byte aligned in the bf16 buffer (TMA needs 16 bytes)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class ParamSlot:
    name: str
    param: nn.Parameter
    shape: Tuple[int, ...]
    numel: int
    offset: int  # in the flat buffers
    bucket: int
    ep_dim: Optional[int] = None  # expert-parallel parameters: the axis the experts are sliced over (each rank holds its slice)
    streamed: bool = False  # zero-3: lives outside the flat buffers (``offset`` is a virtual position past their end)


@dataclass
class Bucket:
    index: int
    name: str
    start: int
    end: int  # padded: (end - start) % (W * ALIGN) == 0
    slots: List[ParamSlot] = field(default_factory=list)
    local: bool = False  # rank-local parameters (expert parallelism): owned whole by this rank, never reduced or gathered

    def shard_range(self, rank: int, world: int) -> Tuple[int, int]:
        if self.local:
            return self.start, self.end
        n = (self.end - self.start) // world
        return self.start + rank * n, self.start + (rank + 1) * n


def default_bucket_of(model: nn.Module) -> Callable[[str], str]:
    """Bucket = one entry of the largest ``nn.ModuleList`` (the stack of decoder layers); everything else is 'root'."""
    best_name, best_len = None, 0
    for name, mod in model.named_modules():
        if isinstance(mod, nn.ModuleList) and len(mod) > best_len:
            best_name, best_len = name, len(mod)

    def bucket_of(param_name: str) -> str:
        if best_name is not None and param_name.startswith(best_name + "."):
            rest = param_name[len(best_name) + 1:]
            return f"{best_name}.{rest.split('.', 1)[0]}"
        return "root"

    return bucket_of


class ShardedEngine:
    def __init__(self, model: nn.Module, mp: Policy, mesh=None, *, device=None, shard_optimizer: bool = True,
                 grad_reduce_dtype: torch.dtype = torch.float32, is_trainable: Optional[Callable[[str], bool]] = None,
                 bucket_of: Optional[Callable[[str], str]] = None, comm: Optional[str] = None, zero_stage: int = 1):
        """``comm``: ``"nccl"`` (library reduce-scatter / all-gather per bucket) or ``"p2p"`` (gradient pull-reduce and AdamW with
        an all-gather epilogue as two kernels over peer-mapped buffers); ``"multimem"`` is the same through the switch's multicast mapping (one reduced load, one broadcast store per
        element).  Default: ``LEVANTER_B200_COMM`` if set, else ``multimem``, degrading to ``p2p`` and ``nccl`` when the fabric
        or the runtime lacks what the mode needs."""
        import os as _os

        self.comm = (comm or _os.environ.get("LEVANTER_B200_COMM", "multimem")).lower()  # nccl | p2p | multimem
        self._sym_param = self._sym_grad = None
        self.model = model
        self.mp = mp
        self.mesh = mesh
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.world = mesh.data_size if mesh is not None else 1
        self.rank = mesh.data_rank if mesh is not None else 0
        self.data_group = mesh.data_group if mesh is not None else None
        self.replica_group = mesh.replica_group if (mesh is not None and mesh.replica_size > 1) else None
        self.model_group = mesh.model_group if (mesh is not None and mesh.model_size > 1) else None
        self.shard_optimizer = shard_optimizer or self.world == 1
        self.grad_reduce_dtype = grad_reduce_dtype
        self.stream = None  # zero-3 layer streamer
        self.zero_stage = 3 if (zero_stage == 3 and self.world > 1 and self.shard_optimizer and mp.param_dtype == torch.float32) else 1
        self._build_layout(is_trainable, bucket_of or default_bucket_of(model))
        self.opt = None
        self.opt_state = None
        self.fused_adam: Optional["FusedAdamW"] = None
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.capture_updates = False  # set by a hook before a step whose parameter change it wants to read
        self.last_updates: Optional[Dict[str, torch.Tensor]] = None

    # ------------------------------------------------------------------------------------------ layout
    def _build_layout(self, is_trainable, bucket_of):
        W = self.world
        cd, pd = self.mp.compute_dtype, self.mp.param_dtype
        seen: Dict[int, str] = {}
        named: List[Tuple[str, nn.Parameter]] = []
        for name, p in self.model.named_parameters():
            if id(p) in seen:
                continue
            seen[id(p)] = name
            trainable = p.requires_grad and (is_trainable is None or is_trainable(name))
            if trainable and W > 1 and getattr(p, "ep_dim", None) is not None and not self.shard_optimizer:
                raise NotImplementedError(f"{name} is expert-parallel: rank-local parameters need the sharded optimizer")
            if not trainable:
                p.requires_grad_(False)
                if p.is_floating_point():
                    p.data = p.data.to(device=self.device, dtype=cd)
                continue
            named.append((name, p))
        # expert-parallel parameters (a different slice of the experts on every rank) get buckets of their own, which this
        # rank owns whole: their gradients already hold every rank's tokens (the token exchange brought them here), so they
        # are scaled, not reduced, and their new weights are not gathered
        is_local = {name: (W > 1 and getattr(p, "ep_dim", None) is not None) for name, p in named}
        plain_bucket_of = bucket_of

        def bucket_of(name: str) -> str:  # noqa: F811
            return plain_bucket_of(name) + ("#experts" if is_local[name] else "")

        # zero-3: the weight matrices of the layer stack are streamed (see parallel/zero3.py); the rest is laid out below
        stream_layers: Dict[str, List[Tuple[str, nn.Parameter]]] = {}
        if self.zero_stage == 3:
            from .zero3 import eligible

            keep = []
            for name, p in named:
                b = plain_bucket_of(name)
                if b != "root" and not is_local[name] and eligible(p, W):
                    stream_layers.setdefault(b, []).append((name, p))
                else:
                    keep.append((name, p))
            if stream_layers:
                named = keep
            else:
                self.zero_stage = 1
        order: Dict[str, int] = {}
        for name, _ in named:
            order.setdefault(bucket_of(name), len(order))
        named.sort(key=lambda np_: order[bucket_of(np_[0])])  # stable: keeps registration order inside a bucket
        self.buckets: List[Bucket] = []
        self.slots: List[ParamSlot] = []
        off = 0
        cur: Optional[Bucket] = None
        for name, p in named:
            b = bucket_of(name)
            if cur is None or cur.name != b:
                if cur is not None:
                    cur.end = cur.start + _round_up(off - cur.start, W * ALIGN)
                    off = cur.end
                cur = Bucket(len(self.buckets), b, off, off, local=is_local[name])
                self.buckets.append(cur)
            slot = ParamSlot(name, p, tuple(p.shape), p.numel(), off, cur.index, getattr(p, "ep_dim", None) if is_local[name] else None)
            cur.slots.append(slot)
            self.slots.append(slot)
            off = _round_up(off + p.numel(), ALIGN)
        if cur is not None:
            cur.end = cur.start + _round_up(off - cur.start, W * ALIGN)
            off = cur.end
        self.total = off
        use_p2p = False
        if self.comm in ("p2p", "multimem") and W > 1 and self.shard_optimizer and self.device.type == "cuda" and cd == torch.bfloat16:
            from .symm import p2p_available

            use_p2p = p2p_available(self.data_group)
        if use_p2p:
            from .symm import SymmetricBuffer

            try:
                self._sym_param = SymmetricBuffer(self.total, cd, self.device, self.data_group)
                self._sym_grad = SymmetricBuffer(self.total, torch.float32, self.device, self.data_group)
            except Exception as e:  # noqa: BLE001 - every rank takes the same path: the rendezvous is collective
                import logging

                logging.getLogger(__name__).warning(f"symmetric memory unavailable ({e}); using NCCL collectives")
                self._sym_param = self._sym_grad = None
                use_p2p = False
        if use_p2p:
            self.param_flat, self.grad_flat = self._sym_param.tensor, self._sym_grad.tensor
            if self.comm == "multimem" and not (self._sym_param.multicast_ptr and self._sym_grad.multicast_ptr):
                self.comm = "p2p"  # no multicast mapping on this fabric: plain peer loads and stores
            self._p2p_scratch = torch.zeros(1024, dtype=torch.float32, device=self.device)
            self._p2p_sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        else:
            self.comm = "nccl"
            self.param_flat = torch.zeros(self.total, dtype=cd, device=self.device)
            self.grad_flat = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        # owned slices, concatenated bucket by bucket
        self.shard_numel = sum(b.end - b.start if b.local else (b.end - b.start) // W for b in self.buckets) if self.shard_optimizer else self.total
        self.stream_lo = self.shard_numel  # zero-3: the streamed matrices' rows follow the owned slices in every per-rank buffer
        if stream_layers:
            from .zero3 import LayerStreamer

            names = list(stream_layers.keys())
            modules = [self.model.get_submodule(b) for b in names]
            self.stream = LayerStreamer([stream_layers[b] for b in names], modules, world=W, rank=self.rank, group=self.data_group,
                                        device=self.device, compute_dtype=cd, comm=self.comm if use_p2p or self.comm == "nccl" else "nccl")
            self.shard_numel += self.stream.shard_numel
        self.has_local = any(b.local for b in self.buckets)
        self.master_is_param = (pd == cd and W == 1) or (pd == cd and not self.shard_optimizer)
        if self.master_is_param:
            self.master = self.param_flat
        else:
            self.master = torch.zeros(self.shard_numel, dtype=pd, device=self.device)
        self.grad_shard = self.grad_flat if (W == 1 or not self.shard_optimizer) else torch.zeros(
            self.shard_numel, dtype=torch.float32, device=self.device)
        # (param name -> list of (local offset, flat offset, length)) for the owned part of each parameter
        self.segments: Dict[str, Tuple[int, int, int]] = {}
        self._shapes: Dict[str, Tuple[int, ...]] = {s.name: s.shape for s in self.slots}
        local = 0
        self._bucket_local_start: List[int] = []
        for b in self.buckets:
            lo, hi = (b.start, b.end) if not self.shard_optimizer else b.shard_range(self.rank, W)
            self._bucket_local_start.append(local)
            for s in b.slots:
                a, e = max(s.offset, lo), min(s.offset + s.numel, hi)
                if a < e:
                    self.segments[s.name] = (local + (a - lo), a, e - a)
            local += hi - lo
        if self.stream is not None:
            st = self.stream
            st.grad_shard = self.grad_shard[self.stream_lo:]
            virt = self.total
            with torch.no_grad():
                for sp in st.params:
                    slot = ParamSlot(sp.name, sp.param, sp.shape, sp.param.numel(), virt, -1, None, streamed=True)
                    self.slots.append(slot)
                    self._shapes[sp.name] = sp.shape
                    lo = self.stream_lo + sp.shard_off
                    self.segments[sp.name] = (lo, virt + self.rank * sp.shard_numel, sp.shard_numel)
                    mine = sp.param.data[self.rank * sp.rows:(self.rank + 1) * sp.rows].reshape(-1)
                    self.master[lo:lo + sp.shard_numel].copy_(mine)
                    st.w_shard[sp.shard_off:sp.shard_off + sp.shard_numel].copy_(mine)
                    virt += sp.param.numel()
            st.attach()
            if st.peer:
                st._sym_w.barrier(1)  # every rank's rows are in place before anyone assembles a layer from them
        # move the data: master slices take the original (param-dtype) values, the flat buffer their compute-dtype cast
        with torch.no_grad():
            for s in self.slots:
                if s.streamed:
                    continue
                src = s.param.data
                seg = self.segments.get(s.name)
                if seg is not None and not self.master_is_param:
                    l0, f0, n = seg
                    a = f0 - s.offset
                    self.master[l0:l0 + n].copy_(src.reshape(-1)[a:a + n])
                view = self.param_flat[s.offset:s.offset + s.numel].view(s.shape)
                view.copy_(src)
                s.param.data = view
                s.param.main_grad = self.grad_flat[s.offset:s.offset + s.numel].view(s.shape)

    def init_master_from_model(self, source: Optional[Dict[str, torch.Tensor]] = None) -> None:
        """Fill the master weights (param dtype) from ``source`` (name -> full tensor, e.g. fp32 initial values) or from
        the current compute-dtype parameters."""
        if self.master_is_param:
            return
        with torch.no_grad():
            for s in self.slots:
                seg = self.segments.get(s.name)
                if seg is None:
                    continue
                lo, fo, n = seg
                if s.streamed and not (source is not None and s.name in source):
                    continue  # the parameter is a view of a staging slot: the master rows already hold its values
                src = source[s.name].reshape(-1) if source is not None and s.name in source else s.param.data.reshape(-1)
                a = fo - s.offset
                self.master[lo:lo + n].copy_(src[a:a + n].to(self.master.dtype))
        self.sync_streamed_from_master()

    def sync_streamed_from_master(self) -> None:
        """zero-3: refresh the compute-dtype rows that peers gather from after the master rows were set from outside (a
        checkpoint, an initial state)."""
        if self.stream is not None:
            with torch.no_grad():
                self.stream.w_shard.copy_(self.master[self.stream_lo:])
            self.stream.invalidate()
            if self.stream.peer:
                self.stream._sym_w.barrier(1)

    # ------------------------------------------------------------------------------------------ trees
    def _shaped(self, name: str, flat: torch.Tensor) -> torch.Tensor:
        """A segment that covers its whole parameter is presented in the parameter's shape (matrix optimizers need it)."""
        shape = self._shapes.get(name)
        if shape is not None and flat.numel() == math.prod(shape):
            return flat.view(shape)
        return flat

    def master_tree(self) -> Dict[str, torch.Tensor]:
        return {name: self._shaped(name, self.master[lo:lo + n]) for name, (lo, fo, n) in self.segments.items()}

    def grad_tree(self) -> Dict[str, torch.Tensor]:
        return {name: self._shaped(name, self.grad_shard[lo:lo + n] if self.grad_shard is not self.grad_flat
                                   else self.grad_flat[fo:fo + n])
                for name, (lo, fo, n) in self.segments.items()}

    def param_names(self) -> List[str]:
        return [s.name for s in self.slots]

    # ------------------------------------------------------------------------------------------ optimizer
    def set_optimizer(self, optimizer, *, optimizer_config: Optional[OptimizerConfig] = None, num_train_steps: int = 0,
                      use_fused: Optional[bool] = None) -> None:
        """``optimizer`` is a GradientTransformation; when ``optimizer_config`` is an eligible ``AdamConfig`` and the
        parameters are on a B200 the fused CUDA AdamW is used instead (same mathematics, one pass)."""
        from ..ops import lib

        self.opt = optimizer
        fused_ok = (optimizer_config is not None and isinstance(optimizer_config, AdamConfig)
                    and optimizer_config.fused_kernel_eligible() and self.device.type == "cuda" and lib.available()
                    and self.master.dtype == torch.float32 and self.shard_optimizer)
        if use_fused is False:
            fused_ok = False
        if fused_ok:
            self.fused_adam = FusedAdamW(self, optimizer_config, num_train_steps)
            self.opt_state = None
        else:
            self.fused_adam = None
            self.opt_state = optimizer.init(self.master_tree())

    # ------------------------------------------------------------------------------------------ gradients
    def zero_grad(self) -> None:
        self.grad_flat.zero_()
        if self.stream is not None:
            self.grad_shard[self.stream_lo:].zero_()  # the streamed rows accumulate here during the backward passes
        for s in self.slots:
            s.param.grad = None

    def collect_grads(self) -> None:
        """Fold autograd ``.grad`` (parameters whose gradient did not go through a ``main_grad`` GEMM epilogue) into
        the fp32 accumulator."""
        for s in self.slots:
            g = s.param.grad
            if g is not None and not s.streamed:  # (a streamed matrix's gradient was reduced the moment autograd produced it)
                s.param.main_grad.add_(g.to(torch.float32).view(s.shape))
                s.param.grad = None

    def reduce_grads(self, scale: float = 1.0) -> None:
        """Average gradients over the data axis into the owned slices (and over replicas)."""
        W = self.world
        if self.stream is not None and scale != 1.0:
            self.grad_shard[self.stream_lo:].mul_(scale)  # already averaged over the ranks, row slice by row slice
        if self._sym_grad is not None:
            self._p2p_reduce_grads(scale)
            if self.replica_group is not None:
                dist.all_reduce(self.grad_shard, op=dist.ReduceOp.AVG, group=self.replica_group)
            return
        if scale != 1.0:
            self.grad_flat.mul_(scale)
        if W > 1:
            if self.shard_optimizer:
                for b, lstart in zip(self.buckets, self._bucket_local_start):
                    inp = self.grad_flat[b.start:b.end]
                    if b.local:  # the average over ranks of a gradient that already sums every rank's tokens
                        self.grad_shard[lstart:lstart + (b.end - b.start)].copy_(inp).div_(W)
                        continue
                    n = (b.end - b.start) // W
                    out = self.grad_shard[lstart:lstart + n]
                    if self.grad_reduce_dtype != torch.float32:
                        tmp = inp.to(self.grad_reduce_dtype)
                        o2 = torch.empty(n, dtype=self.grad_reduce_dtype, device=self.device)
                        dist.reduce_scatter_tensor(o2, tmp, op=dist.ReduceOp.AVG, group=self.data_group)
                        out.copy_(o2)
                    else:
                        dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.AVG, group=self.data_group)
            else:
                dist.all_reduce(self.grad_flat, op=dist.ReduceOp.AVG, group=self.data_group)
        if self.replica_group is not None:
            dist.all_reduce(self.grad_shard, op=dist.ReduceOp.AVG, group=self.replica_group)

    def _p2p_reduce_grads(self, scale: float) -> None:
        """Every rank pulls and sums its owned range of every bucket from all peers' gradient buffers (one kernel per bucket);
        the sum of squares of the reduced range comes out of the same pass."""
        from ..ops import lib

        c = lib
        f = getattr(self, "_f_rs", None)
        if f is None:
            f = self._f_rs = lib.fn("lvb_p2p_reduce_scatter", [c.c_void_p, c.c_int, c.c_int, c.c_longlong, c.c_longlong, c.c_float,
                                                                c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p], launches=2)
        W = self.world
        self._sym_grad.barrier(0)  # every rank has finished writing its gradients
        self._p2p_sumsq.zero_()
        fm = None
        if self.comm == "multimem":
            fm = getattr(self, "_f_mrs", None)
            if fm is None:
                fm = self._f_mrs = lib.fn("lvb_mm_reduce_scatter", [c.c_void_p, c.c_longlong, c.c_longlong, c.c_float, c.c_void_p, c.c_void_p,
                                                                    c.c_void_p, c.c_void_p], launches=2)
        for b, lstart in zip(self.buckets, self._bucket_local_start):
            lo, hi = b.shard_range(self.rank, W)
            out = self.grad_shard[lstart:lstart + (hi - lo)]
            if b.local:  # a "reduction" over this rank alone: scale, copy and sum of squares in the same kernel
                rc = f(self._self_ptrs(self._sym_grad), 1, 0, lo, hi - lo, float(scale) / W, out.data_ptr(), self._p2p_sumsq.data_ptr(),
                       self._p2p_scratch.data_ptr(), lib.stream_ptr())
            elif fm is not None:
                rc = fm(self._sym_grad.multicast_ptr, lo, hi - lo, float(scale) / W, out.data_ptr(), self._p2p_sumsq.data_ptr(),
                        self._p2p_scratch.data_ptr(), lib.stream_ptr())
            else:
                rc = f(self._sym_grad.c_ptrs, W, self.rank, lo, hi - lo, float(scale) / W, out.data_ptr(), self._p2p_sumsq.data_ptr(),
                       self._p2p_scratch.data_ptr(), lib.stream_ptr())
            lib.check_rc(rc, "lvb_p2p_reduce_scatter")
        self._p2p_sumsq_valid = True

    def _self_ptrs(self, buf):
        """A one-entry peer table holding this rank's own copy of a symmetric buffer (for rank-local buckets)."""
        import ctypes

        cache = self.__dict__.setdefault("_self_ptr_cache", {})
        key = id(buf)
        if key not in cache:
            cache[key] = (ctypes.c_void_p * 1)(buf.peer_ptrs[buf.rank])
        return cache[key]

    def grad_sumsq(self) -> torch.Tensor:
        """Sum of squared gradients over *all* parameters (device scalar), reduced over the mesh."""
        from ..ops import lib

        g = self.grad_shard
        if self._sym_grad is not None and getattr(self, "_p2p_sumsq_valid", False) and self.replica_group is None:
            sq = self._p2p_sumsq.clone()
            self._p2p_sumsq_valid = False
            if self.stream is not None:  # the reduce kernels covered the flat buffers only
                from ..ops.optim_kernels import sumsq

                sq = sq + sumsq(g[self.stream_lo:])
        elif self.device.type == "cuda" and lib.available():
            from ..ops.optim_kernels import sumsq

            sq = sumsq(g)
        else:
            sq = (g.float() ** 2).sum().reshape(1)
        if self.world > 1 and self.shard_optimizer:
            dist.all_reduce(sq, group=self.data_group)
        if self.model_group is not None:
            # tensor-parallel shards hold disjoint slices of the sharded weights; replicated ones are counted once
            rep = self._replicated_sumsq()
            part = sq - rep
            dist.all_reduce(part, group=self.model_group)
            sq = part + rep
        return sq

    def _replicated_sumsq(self) -> torch.Tensor:
        tot = torch.zeros(1, dtype=torch.float32, device=self.device)
        gt = self.grad_tree()
        for s in self.slots:
            if getattr(s.param, "tp_dim", None) is None and s.name in gt:
                tot += (gt[s.name].float() ** 2).sum()
        if self.world > 1 and self.shard_optimizer:
            dist.all_reduce(tot, group=self.data_group)
        return tot

    # ------------------------------------------------------------------------------------------ step
    def step(self, *, grad_scale: float = 1.0, loss: Optional[torch.Tensor] = None, **extra) -> None:
        """collect -> reduce -> optimizer update on owned slices -> refresh compute-dtype parameters everywhere."""
        self.collect_grads()
        before = self.master.clone() if self.capture_updates else None
        if self.stream is not None and self.stream.peer:
            # peers may still be pulling this rank's weight rows for their last layers: nobody overwrites rows before all are done
            self.stream._sym_w.barrier(0)
        self.reduce_grads(grad_scale)
        if self.fused_adam is not None:
            self.fused_adam.step()
        else:
            grads = self.grad_tree()
            params = self.master_tree()
            from ..ops.newton_schulz import set_layer_parallel_group

            T.set_norm_reduce_group(self.data_group if (self.world > 1 and self.shard_optimizer) else None)
            # unsharded optimizer on several data ranks: every rank holds the same gradients, so matrix-valued work
            # (Newton-Schulz) is dealt out over them instead of being repeated on each
            set_layer_parallel_group(self.data_group if (self.world > 1 and not self.shard_optimizer) else None)
            batch_groups = [g for g in (self.data_group if self.world > 1 else None, self.replica_group) if g is not None]
            T.set_objective_reduce_group(batch_groups or None)
            if self.model_group is not None:
                # tensor parallelism: norms count a sliced weight's parts on all model ranks and a replicated weight once
                T.set_model_parallel_norm(self.model_group, [s.name for s in self.slots if getattr(s.param, "tp_dim", None) is not None])
            try:
                updates, self.opt_state = self.opt.update(grads, self.opt_state, params, loss=loss, **extra)
            finally:
                T.set_norm_reduce_group(None)
                T.set_objective_reduce_group(None)
                set_layer_parallel_group(None)
                T.set_model_parallel_norm(None, None)
            T.apply_updates(params, updates)
        if before is not None:
            # what this step added to the owned master slices (weight decay and learning rate included), for hooks that watch it
            delta = self.master - before
            self.last_updates = {name: self._shaped(name, delta[lo:lo + n]) for name, (lo, fo, n) in self.segments.items()}
            self.capture_updates = False
        self.publish_params()
        if self._sym_grad is not None:
            # peers read this rank's gradients and write this rank's weights: nobody may run ahead into the next step
            self._sym_param.barrier(1)
        if self.stream is not None:
            self.stream.invalidate()
            if self.stream.peer:
                self.stream._sym_w.barrier(1)  # every rank's new rows are in place before anyone gathers them
        self.zero_grad()

    def publish_params(self) -> None:
        """Write the owned master slices into ``param_flat`` (cast to compute dtype) and all-gather every bucket."""
        W = self.world
        if self.master_is_param:
            return
        if self.stream is not None and (self.fused_adam is None or not self.fused_adam.writes_compute_copy):
            self.stream.w_shard.copy_(self.master[self.stream_lo:])
        if not self.shard_optimizer or W == 1:
            if self.fused_adam is None or not self.fused_adam.writes_compute_copy:
                self.param_flat.copy_(self.master)
            return
        if self._sym_param is not None and self.fused_adam is not None and self.fused_adam.writes_compute_copy:
            return  # the optimizer kernel stored the new weights into every peer's buffer
        for b, lstart in zip(self.buckets, self._bucket_local_start):
            lo, hi = b.shard_range(self.rank, W)
            n = hi - lo
            own = self.param_flat[lo:hi]
            if self.fused_adam is None or not self.fused_adam.writes_compute_copy:
                own.copy_(self.master[lstart:lstart + n])
            if not b.local:
                dist.all_gather_into_tensor(self.param_flat[b.start:b.end], own, group=self.data_group)

    # ------------------------------------------------------------------------------------------ state export
    def full_master(self) -> Dict[str, torch.Tensor]:
        """name -> full parameter tensor in param dtype (gathers slices; used by checkpointing and export)."""
        return self._gather_named(self.master)

    def _gather_named(self, shard: torch.Tensor) -> Dict[str, torch.Tensor]:
        W = self.world
        if W == 1 or not self.shard_optimizer:
            flat = shard
        else:
            flat = torch.empty(self.total, dtype=shard.dtype, device=self.device)
            local_full: Dict[str, torch.Tensor] = {}
            for b, lstart in zip(self.buckets, self._bucket_local_start):
                if b.local:
                    local_full.update(self._gather_local_bucket(b, shard[lstart:lstart + (b.end - b.start)]))
                    continue
                n = (b.end - b.start) // W
                dist.all_gather_into_tensor(flat[b.start:b.end], shard[lstart:lstart + n].contiguous(), group=self.data_group)
            out = {s.name: local_full[s.name] if s.ep_dim is not None else flat[s.offset:s.offset + s.numel].view(s.shape)
                   for s in self.slots if not s.streamed}
            if self.stream is not None:
                for sp in self.stream.params:
                    lo = self.stream_lo + sp.shard_off
                    out[sp.name] = self.stream.gather_full(sp, shard[lo:lo + sp.shard_numel])
            return out
        return {s.name: flat[s.offset:s.offset + s.numel].view(s.shape) for s in self.slots}

    def _gather_local_bucket(self, b: Bucket, mine: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Full tensors of a rank-local bucket: every rank's slice of the experts, concatenated along the expert axis."""
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine.contiguous(), group=self.data_group)
        out = {}
        for s in b.slots:
            o = s.offset - b.start
            out[s.name] = torch.cat([p[o:o + s.numel].view(s.shape) for p in parts], dim=s.ep_dim)
        return out

    def _full_shape(self, s: ParamSlot) -> Tuple[int, ...]:
        if s.ep_dim is None:
            return s.shape
        return tuple(d * self.world if i == s.ep_dim else d for i, d in enumerate(s.shape))

    def _own_part(self, s: ParamSlot, full: torch.Tensor) -> torch.Tensor:
        """This rank's part of a full tensor: all of it, or its slice of the experts."""
        if s.ep_dim is None or full.shape[s.ep_dim] == s.shape[s.ep_dim]:
            return full
        n = s.shape[s.ep_dim]
        return full.narrow(s.ep_dim, self.rank * n, n)

    def deferred_named(self, shard: torch.Tensor) -> Dict[str, Any]:
        """name -> leaf for checkpoint writing.  Unsharded state yields plain views; sharded state yields
        ``DeferredLeaf`` objects that all-gather one bucket at a time (the last gathered bucket is cached), so writing
        a checkpoint never holds more than one bucket of gathered state."""
        from ..tensorstore_serialization import DeferredLeaf

        W = self.world
        if W == 1 or not self.shard_optimizer:
            return {s.name: shard[s.offset:s.offset + s.numel].view(s.shape) for s in self.slots}
        cache: Dict[str, Any] = {"bucket": -1, "flat": None}

        def fetch(slot: ParamSlot) -> torch.Tensor:
            if slot.ep_dim is not None:
                if cache["bucket"] != slot.bucket:
                    b = self.buckets[slot.bucket]
                    lstart = self._bucket_local_start[slot.bucket]
                    cache["bucket"], cache["flat"] = slot.bucket, self._gather_local_bucket(b, shard[lstart:lstart + (b.end - b.start)])
                return cache["flat"][slot.name]
            if cache["bucket"] != slot.bucket:
                b = self.buckets[slot.bucket]
                lstart = self._bucket_local_start[slot.bucket]
                n = (b.end - b.start) // W
                flat = torch.empty(b.end - b.start, dtype=shard.dtype, device=self.device)
                dist.all_gather_into_tensor(flat, shard[lstart:lstart + n].contiguous(), group=self.data_group)
                cache["bucket"], cache["flat"] = slot.bucket, flat
            b = self.buckets[slot.bucket]
            o = slot.offset - b.start
            return cache["flat"][o:o + slot.numel].view(slot.shape)

        out = {s.name: DeferredLeaf(lambda s=s: fetch(s), self._full_shape(s), shard.dtype) for s in self.slots if not s.streamed}
        if self.stream is not None:
            for sp in self.stream.params:
                lo = self.stream_lo + sp.shard_off
                out[sp.name] = DeferredLeaf(lambda sp=sp, lo=lo: self.stream.gather_full(sp, shard[lo:lo + sp.shard_numel]), sp.shape, shard.dtype)
        return out

    def scatter_named(self, full: Dict[str, torch.Tensor], shard: torch.Tensor) -> None:
        """Inverse of :meth:`_gather_named`: copy the owned part of each full tensor into ``shard``."""
        with torch.no_grad():
            for s in self.slots:
                seg = self.segments.get(s.name)
                if seg is None or s.name not in full:
                    continue
                lo, fo, n = seg
                a = fo - s.offset
                shard[lo:lo + n].copy_(self._own_part(s, full[s.name]).reshape(-1)[a:a + n].to(shard.dtype))

    def load_full_params(self, full: Dict[str, torch.Tensor]) -> None:
        """Set parameters (master and compute copies) from full tensors."""
        with torch.no_grad():
            for s in self.slots:
                if s.name in full and not s.streamed:
                    s.param.data.copy_(self._own_part(s, full[s.name]).to(device=self.device, dtype=self.param_flat.dtype).reshape(s.shape))
        if not self.master_is_param:
            self.scatter_named({k: v.to(self.device) for k, v in full.items()}, self.master)
        self.sync_streamed_from_master()

    def optimizer_state_tree(self, deferred: bool = False) -> Any:
        """Optimizer state with every tensor leaf at its full parameter shape (for checkpoints).  With ``deferred`` the
        leaves of sharded state are ``DeferredLeaf`` objects gathered only while being written."""
        if self.fused_adam is not None:
            return self.fused_adam.state_tree(deferred=deferred)
        if deferred:
            return _map_state(self.opt_state, self._deferred_leaf_tree)
        return _map_state(self.opt_state, self._gather_leaf_tree)

    def _deferred_leaf_tree(self, tree: Dict[str, torch.Tensor]) -> Dict[str, Any]:
        if self.world == 1 or not self.shard_optimizer:
            return self._gather_leaf_tree(tree)
        shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=self.device)
        for name, (lo, fo, n) in self.segments.items():
            if tree.get(name) is not None:
                shard[lo:lo + n].copy_(tree[name].reshape(-1))
        return self.deferred_named(shard)

    def _gather_leaf_tree(self, tree: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self.world == 1 or not self.shard_optimizer:
            out = {}
            for s in self.slots:
                if s.name in tree and tree[s.name] is not None:
                    out[s.name] = tree[s.name].view(s.shape)
            return out
        shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=self.device)
        for name, (lo, fo, n) in self.segments.items():
            if tree.get(name) is not None:
                shard[lo:lo + n].copy_(tree[name].reshape(-1))
        full = self._gather_named(shard)
        keys = set()
        # a leaf may be absent on this rank but present on another; every masked-in parameter is exported
        return {k: v for k, v in full.items()}

    def load_optimizer_state_tree(self, state: Any) -> None:
        if self.fused_adam is not None:
            self.fused_adam.load_state_tree(state)
            return

        def scatter(tree):
            out = {}
            for name, (lo, fo, n) in self.segments.items():
                if tree.get(name) is not None:
                    s = next(sl for sl in self.slots if sl.name == name)
                    a = fo - s.offset
                    out[name] = self._own_part(s, tree[name]).reshape(-1)[a:a + n].to(device=self.device, dtype=torch.float32).clone()
            return out

        self.opt_state = _map_state(state, scatter)


def _is_param_tree(x) -> bool:
    return isinstance(x, dict) and len(x) > 0 and all(isinstance(k, str) for k in x) and \
        all((v is None or isinstance(v, torch.Tensor)) for v in x.values()) and any("." in k or k.endswith(("weight", "bias")) for k in x)


def _map_state(state, fn):
    """Apply ``fn`` to every parameter-shaped sub-tree of an optimizer state; keep scalars and structure."""
    if _is_param_tree(state):
        return fn(state)
    if isinstance(state, tuple) and hasattr(state, "_fields"):
        return type(state)(*[_map_state(v, fn) for v in state])
    if isinstance(state, tuple):
        return tuple(_map_state(v, fn) for v in state)
    if isinstance(state, list):
        return [_map_state(v, fn) for v in state]
    if isinstance(state, dict):
        return {k: _map_state(v, fn) for k, v in state.items()}
    return state


class FusedAdamW:
    """AdamW on the owned fp32 slices with ``ops/csrc/optim.cu``: one pass computes moments, bias correction, decoupled
    weight decay and the step, and writes both the fp32 master and the compute-dtype copy.  Global-norm clipping stays on
    the device (sum of squares -> tiny all-reduce -> clip coefficient kernel)."""

    writes_compute_copy = True

    def __init__(self, engine: ShardedEngine, cfg: AdamConfig, num_train_steps: int):
        self.e = engine
        self.cfg = cfg
        self.schedule = cfg.lr_scheduler(num_train_steps)
        self.count = 0
        dev = engine.device
        self.m = torch.zeros(engine.shard_numel, dtype=torch.float32, device=dev)
        self.v = torch.zeros(engine.shard_numel, dtype=torch.float32, device=dev)
        self.coef = torch.ones(1, dtype=torch.float32, device=dev)
        self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
        mask_fn = cfg.build_weight_decay_mask(ParamInfo(engine.model))
        names = list(engine.segments.keys())
        mask = mask_fn({k: None for k in names}) if mask_fn is not None else {k: True for k in names}
        # contiguous runs of equal weight decay over the local slice (gaps are padding: no decay, zero grads)
        runs: List[Tuple[int, int, float]] = []
        starts = set(engine._bucket_local_start)
        if engine.stream is not None:
            starts.add(engine.stream_lo)  # a run never spans the flat buffers' slices and the streamed rows
        for name in sorted(names, key=lambda k: engine.segments[k][0]):
            lo, fo, n = engine.segments[name]
            wd = cfg.weight_decay if (mask.get(name, True) and cfg.weight_decay > 0) else 0.0
            crosses = any(runs[-1][0] < b <= lo for b in starts) if runs else False
            if runs and runs[-1][2] == wd and not crosses:
                runs[-1] = (runs[-1][0], lo + n, wd)
            else:
                runs.append((lo, lo + n, wd))
        self.runs = runs
        self.learning_rate = float(self.schedule(0))

    def step(self) -> None:
        from ..ops.optim_kernels import adamw, clip_coef

        e, c = self.e, self.cfg
        lr = float(self.schedule(self.count))
        self.learning_rate = lr
        self.count += 1
        bc1 = 1.0 - c.beta1 ** self.count
        bc2 = 1.0 - c.beta2 ** self.count
        sq = e.grad_sumsq()
        clip_coef(sq, float(c.max_grad_norm or 0.0), self.coef, self.norm)
        e.last_grad_norm = self.norm
        W = e.world
        if e._sym_param is not None:
            from ..ops import lib

            cc = lib
            f = getattr(self, "_f_ag", None)
            if f is None:
                f = self._f_ag = lib.fn("lvb_p2p_adamw_allgather", [cc.c_void_p] * 5 + [cc.c_int, cc.c_int, cc.c_longlong, cc.c_longlong]
                                        + [cc.c_float] * 7 + [cc.c_void_p, cc.c_int, cc.c_void_p])
            for lo, hi, wd in self.runs:
                if hi <= lo:
                    continue
                if e.stream is not None and lo >= e.stream_lo:
                    self._step_streamed(lo, hi, wd, lr, bc1, bc2)
                    continue
                hi8 = lo + ((hi - lo + 7) // 8) * 8  # the tail up to the next 8 is layout padding (zero weights, zero gradients)
                if e.has_local and self._run_is_local(lo):  # rank-local experts: the new weights go to this rank's buffer only
                    rc = f(e.master[lo:hi8].data_ptr(), self.m[lo:hi8].data_ptr(), self.v[lo:hi8].data_ptr(), e.grad_shard[lo:hi8].data_ptr(),
                           e._self_ptrs(e._sym_param), 1, 0, self._local_to_flat(lo), hi8 - lo, lr, c.beta1, c.beta2, c.epsilon, wd, bc1, bc2,
                           self.coef.data_ptr(), int(c.nesterov), lib.stream_ptr())
                    lib.check_rc(rc, "lvb_p2p_adamw_allgather")
                    continue
                if e.comm == "multimem":
                    fm = getattr(self, "_f_mag", None)
                    if fm is None:
                        fm = self._f_mag = lib.fn("lvb_mm_adamw_allgather", [cc.c_void_p] * 5 + [cc.c_longlong, cc.c_longlong] + [cc.c_float] * 7
                                                  + [cc.c_void_p, cc.c_int, cc.c_void_p])
                    rc = fm(e.master[lo:hi8].data_ptr(), self.m[lo:hi8].data_ptr(), self.v[lo:hi8].data_ptr(), e.grad_shard[lo:hi8].data_ptr(),
                            e._sym_param.multicast_ptr, self._local_to_flat(lo), hi8 - lo, lr, c.beta1, c.beta2, c.epsilon, wd, bc1, bc2,
                            self.coef.data_ptr(), int(c.nesterov), lib.stream_ptr())
                    lib.check_rc(rc, "lvb_mm_adamw_allgather")
                    continue
                rc = f(e.master[lo:hi8].data_ptr(), self.m[lo:hi8].data_ptr(), self.v[lo:hi8].data_ptr(), e.grad_shard[lo:hi8].data_ptr(),
                       e._sym_param.c_ptrs, W, e.rank, self._local_to_flat(lo), hi8 - lo, lr, c.beta1, c.beta2, c.epsilon, wd, bc1, bc2,
                       self.coef.data_ptr(), int(c.nesterov), lib.stream_ptr())
                lib.check_rc(rc, "lvb_p2p_adamw_allgather")
            return
        for lo, hi, wd in self.runs:
            if hi <= lo:
                continue
            if e.stream is not None and lo >= e.stream_lo:
                self._step_streamed(lo, hi, wd, lr, bc1, bc2)
                continue
            # compute-dtype destination: the owned slice inside param_flat
            dst = self._compute_view(lo, hi)
            adamw(e.master[lo:hi], self.m[lo:hi], self.v[lo:hi], e.grad_shard[lo:hi], dst, lr, c.beta1, c.beta2, c.epsilon,
                  wd, bc1, bc2, self.coef, 1.0, c.nesterov)

    def _step_streamed(self, lo: int, hi: int, wd: float, lr: float, bc1: float, bc2: float) -> None:
        """zero-3 rows: the new compute-dtype values go to this rank's own rows; peers pull them when they assemble a layer."""
        from ..ops.optim_kernels import adamw

        e, c = self.e, self.cfg
        s0 = e.stream_lo
        adamw(e.master[lo:hi], self.m[lo:hi], self.v[lo:hi], e.grad_shard[lo:hi], e.stream.w_shard[lo - s0:hi - s0], lr, c.beta1, c.beta2,
              c.epsilon, wd, bc1, bc2, self.coef, 1.0, c.nesterov)

    def _run_is_local(self, lo: int) -> bool:
        e = self.e
        for b, ls in zip(reversed(e.buckets), reversed(e._bucket_local_start)):
            if lo >= ls:
                return b.local
        return False

    def _local_to_flat(self, lo: int) -> int:
        e = self.e
        for b, ls in zip(reversed(e.buckets), reversed(e._bucket_local_start)):
            if lo >= ls:
                start = b.shard_range(e.rank, e.world)[0] if e.shard_optimizer else b.start
                return start + (lo - ls)
        raise IndexError(lo)

    def _compute_view(self, lo: int, hi: int) -> torch.Tensor:
        f = self._local_to_flat(lo)
        return self.e.param_flat[f:f + (hi - lo)]

    def _grad_view(self, lo: int, hi: int) -> torch.Tensor:
        f = self._local_to_flat(lo)
        return self.e.grad_flat[f:f + (hi - lo)]

    # state in the reference's optax tree shape: inject_hyperparams(chain(clip, scale_by_adam, ...))
    def state_tree(self, deferred: bool = False):
        e = self.e
        mu = e.deferred_named(self.m) if deferred else e._gather_named(self.m)
        nu = e.deferred_named(self.v) if deferred else e._gather_named(self.v)
        idx = 1 if self.cfg.max_grad_norm else 0
        inner = [T.EmptyState()] * (idx + 1)
        inner[idx] = T.ScaleByAdamState(self.count, mu, nu)
        return T.InjectHyperparamsState(self.count, {"learning_rate": self.learning_rate},
                                        {"learning_rate": T.ScaleByScheduleState(self.count)}, tuple(inner))

    def load_state_tree(self, state) -> None:
        self.count = int(state.count)
        for st in state.inner_state:
            if isinstance(st, T.ScaleByAdamState) or (hasattr(st, "mu") and hasattr(st, "nu")):
                self.e.scatter_named({k: v.to(self.e.device) for k, v in st.mu.items()}, self.m)
                self.e.scatter_named({k: v.to(self.e.device) for k, v in st.nu.items()}, self.v)
