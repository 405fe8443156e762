"""Tensor-parallel regions (Megatron style) over the mesh's ``model`` axis.

The reference gets TP from axis names (``tensor_parallel_axes: [mlp, heads]`` mapped to the ``model`` mesh axis,
src/levanter/trainer.py:677,851-855) and lets XLA insert the collectives.  Here the column-parallel side (q/k/v,
gate/up) needs no forward communication and an all-reduce of the input gradient; the row-parallel side (o_proj,
down_proj) all-reduces its forward output.

The all-reduce itself runs on this library's kernels when the model axis lives on one NVSwitch node: the tensor is staged
in a symmetric buffer and reduced in place, by ``multimem.ld_reduce`` / ``multimem.st`` through the switch or by peer loads
and stores (``ops/csrc/p2p_collectives.cu``); ``LEVANTER_B200_TP_COMM=nccl`` (or a CPU group) keeps NCCL / gloo, which is
also the oracle in the tests.  ``ops.fused_tp`` has the GEMMs with the collective fused in."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist


ONE_SHOT_MAX_BYTES = 2 << 20  # tensors up to this size take the single-launch all-reduce


class _UseNccl(Exception):
    pass


class _CopyToRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_reduce(g.contiguous()), None


class _ReduceFromRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        return tp.all_reduce(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return g, None


class _RowLinearFn(torch.autograd.Function):
    """``y = all_reduce(x W^T)`` with the collective split around the product (see ``TensorParallel.matmul_all_reduce``).  The
    backward pass needs no communication: ``dx = dy W`` stays local to the rank's columns, ``dW = dy^T x`` goes where
    ``ops.gemm`` puts weight gradients (the engine's fp32 accumulator, a gradient sink, or autograd)."""

    @staticmethod
    def forward(ctx, x, weight, tp):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        y = tp.matmul_all_reduce(x2, weight)
        ctx.save_for_backward(x2, weight)
        ctx.x_shape = shp
        ctx.weight_ref = weight
        return y.view(*shp[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm

        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            sink = getattr(ctx.weight_ref, "grad_sink", None)
            main_grad = getattr(ctx.weight_ref, "main_grad", None)
            if sink is not None:
                sink(dy2, x2)
            elif main_grad is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        return dx, dw, None


class TensorParallel:
    def __init__(self, group: Optional[dist.ProcessGroup], size: int, rank: int, comm: Optional[str] = None):
        self.group = group
        self.size = size
        self.rank = rank
        self.comm = (comm or os.environ.get("LEVANTER_B200_TP_COMM", "auto")).lower()  # auto | multimem | p2p | nccl
        self._os = None           # symmetric areas + counters of the one-shot kernel
        self._os_calls = 0
        self._sym = None          # symmetric staging buffer (bytes), grown on demand by every rank at the same call
        self._sym_failed = False
        self.kernel_all_reduces = 0

    @staticmethod
    def from_mesh(mesh) -> Optional["TensorParallel"]:
        ax = mesh.axes["model"]
        if ax.size <= 1:
            return None
        tp = TensorParallel(ax.group, ax.size, ax.rank)
        tp.mesh = mesh  # models that also slice experts over the data axis find that axis's group here
        return tp

    def copy_to_region(self, x: torch.Tensor) -> torch.Tensor:
        return _CopyToRegion.apply(x, self)

    def reduce_from_region(self, x: torch.Tensor) -> torch.Tensor:
        return _ReduceFromRegion.apply(x, self)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of ``x`` over the model axis, in place when possible."""
        x = x.contiguous()
        if self._kernel_path_ok(x):
            try:
                nbytes = x.numel() * x.element_size()
                if nbytes <= ONE_SHOT_MAX_BYTES and nbytes % 16 == 0 and self.comm in ("auto", "p2p", "multimem"):
                    return self._one_shot_all_reduce(x)
                if self.comm == "auto":
                    raise _UseNccl()  # large tensors: NCCL measured faster than the staged two-shot kernels (2 GPUs)
                return self._kernel_all_reduce(x)
            except _UseNccl:
                pass
            except Exception:  # noqa: BLE001  (no symmetric memory on this fabric, allocation failure): NCCL from now on
                if self.comm in ("multimem", "p2p"):
                    raise
                self._sym_failed = True
        dist.all_reduce(x, group=self.group)
        return x

    # -- own kernels over symmetric memory -----------------------------------------------------------------------
    def _agree(self, ok: bool, device) -> None:
        """All ranks got their buffer, or none uses the kernel path (decided over NCCL so that no rank is left alone)."""
        flag = torch.tensor([1 if ok else 0], device=device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            raise RuntimeError("symmetric memory is not available on every rank of the model axis")

    def _one_shot_all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Small tensors (decode-size activations): one launch, push to every peer + arrival counters (see the kernel)."""
        from ..ops import lib
        from .symm import SymmetricBuffer

        W, cap = self.size, ONE_SHOT_MAX_BYTES
        area = W * cap
        if self._os is None:
            try:
                buf = SymmetricBuffer(2 * area + 2 * 64 * 4, torch.uint8, x.device, self.group)  # zeroed: counters start at 0
                ok = True
            except Exception:  # noqa: BLE001
                buf, ok = None, False
            self._agree(ok, x.device)
            buf.barrier(0)  # nobody pushes into an area whose counters are not cleared yet
            self._os, self._os_calls, self._os_arrivals = buf, 0, [0, 0]
        sym = self._os
        n = self._os_calls
        self._os_calls = n + 1
        parity = n & 1
        nbytes = x.numel() * x.element_size()
        blocks = max(1, min(torch.cuda.get_device_properties(x.device).multi_processor_count, -(-(nbytes // 16) // 256)))
        stage = (ctypes.c_void_p * W)(*[p + parity * area for p in sym.peer_ptrs])
        flags = (ctypes.c_void_p * W)(*[p + 2 * area + parity * 64 * 4 for p in sym.peer_ptrs])
        c = lib
        f = lib.fn("lvb_all_reduce_one_shot", [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_longlong, c.c_longlong,
                                               c.c_int, c.c_int, c.c_int, c.c_void_p, c.c_void_p])
        # the counters only grow: after this call each of them has received `blocks` more arrivals (one per block of the pusher)
        # (kept modulo 2^32 and handed over as a signed 32-bit value; the kernel compares differences, so wrapping is harmless)
        self._os_arrivals[parity] = (self._os_arrivals[parity] + blocks) & 0xFFFFFFFF
        target = self._os_arrivals[parity] - (1 << 32) if self._os_arrivals[parity] >= (1 << 31) else self._os_arrivals[parity]
        rc = f(x.data_ptr(), x.data_ptr(), stage, flags, sym.rank, W, nbytes, cap, blocks, target,
               1 if x.dtype == torch.float32 else 0, lib.status_buffer().data_ptr(), lib.stream_ptr())
        lib.check_rc(rc, "lvb_all_reduce_one_shot")
        self.kernel_all_reduces += 1
        return x

    def _kernel_path_ok(self, x: torch.Tensor) -> bool:
        if self.comm == "nccl" or self._sym_failed or not x.is_cuda or self.size <= 1 or self.size > 8:
            return False
        if x.dtype not in (torch.bfloat16, torch.float32):
            return False
        from ..ops import lib

        return lib.available()

    def _kernel_all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops import lib
        from .symm import SymmetricBuffer

        es = x.element_size()
        vec = (16 // es) * self.size
        n = x.numel()
        n_pad = -(-n // vec) * vec
        need = n_pad * es
        if self._sym is None or self._sym.tensor.numel() < need:
            # every rank reaches this line at the same call with the same size, so the rendezvous inside is collective; the
            # ranks then agree (over NCCL) that all of them got their buffer, so that no rank is left alone on either path
            try:
                sym_new = SymmetricBuffer(max(need, 64 << 20), torch.uint8, x.device, self.group)
                ok = 1
            except Exception:  # noqa: BLE001
                sym_new, ok = None, 0
            flag = torch.tensor([ok], device=x.device, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            if int(flag.item()) == 0:
                raise RuntimeError("symmetric memory is not available on every rank of the model axis")
            self._sym = sym_new
        sym = self._sym
        stage = sym.tensor[:need].view(x.dtype)
        stage[:n].copy_(x.reshape(-1))
        if n_pad > n:
            stage[n:].zero_()
        use_mc = sym.multicast_ptr != 0 and self.comm != "p2p"
        if self.comm == "multimem" and not use_mc:
            raise RuntimeError("no multicast mapping on this fabric")
        c = lib
        f = lib.fn("lvb_all_reduce_symmetric", [c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_longlong, c.c_int, c.c_void_p])
        sym.barrier(0)  # every rank's input is staged
        rc = f(sym.multicast_ptr if use_mc else 0, sym.c_ptrs, sym.rank, self.size, n_pad, 1 if x.dtype == torch.float32 else 0, lib.stream_ptr())
        lib.check_rc(rc, "lvb_all_reduce_symmetric")
        sym.barrier(1)  # every rank's slice has been published
        x.reshape(-1).copy_(stage[:n])
        self.kernel_all_reduces += 1
        return x

    # -- row-parallel projection with the all-reduce split around the GEMM ------------------------------------------------
    def fused_row_linear_ok(self, x2: torch.Tensor, w: torch.Tensor) -> bool:
        from ..ops import lib
        from ..ops.gemm import PAIR_ENABLED

        T, N = x2.shape[0], w.shape[0]
        if not torch.is_grad_enabled():
            # inference: prefill batches come in ever-changing token counts, and the staging arena keeps arrival counters
            # per distinct shape; those calls take the all-reduce after a plain GEMM
            return False
        ok = bool(self.comm in ("auto", "p2p", "multimem") and not self._sym_failed and x2.is_cuda and lib.available() and PAIR_ENABLED
                  and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 1 < self.size <= 8 and T % (self.size * 32) == 0
                  and T >= 2048 and N > 128 and N % 8 == 0 and x2.shape[1] % 8 == 0)
        if ok:
            st = self.__dict__.get("_rs")
            if st is not None and st["arena"] is not None and (T, N) not in st["cnt"] and (T * N + 63) // 64 * 64 <= st["area"]:
                from ..ops.fused_tp import rs_counters

                n = (rs_counters(T // self.size, N) + 63) // 64 * 64
                ok = st["cnt_next"] + 2 * n <= st["cnt_cap"]  # no room for another shape's counters: the plain path
        return ok

    def matmul_all_reduce(self, x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``sum over ranks of x2 @ w.T`` on every rank (``x2 [T, K_local]``, ``w [N, K_local]``): the row-parallel projection of a
        tensor-parallel block.  The reduce-scatter half of the all-reduce is fused into the GEMM (tile by tile the epilogue
        stores partial products into the staging slots of the rank that owns the rows, which sums them as they arrive,
        ``ops/fused_tp.py``); the all-gather half is one copy kernel that pulls every rank's reduced rows over NVLink."""
        from ..ops import lib
        from ..ops.fused_tp import _ptr_array, reduce_scatter_gemm, rs_counters
        from .symm import SymmetricBuffer

        W, r = self.size, self.rank
        T, K = x2.shape
        N = w.shape[0]
        rows = T // W
        st = self.__dict__.setdefault("_rs", {"arena": None, "area": 0, "cnt": {}, "calls": 0, "uses": {}, "slice": None, "tables": {}})
        need = (T * N + 63) // 64 * 64
        if st["arena"] is None or need > st["area"]:
            # every rank reaches this with the same shapes, so the allocation is collective; counters of all shapes start over
            cnt_cap = 8 * ((rs_counters(rows, N) + 63) // 64 * 64) * 2
            st["area"], st["cnt"], st["uses"], st["cnt_next"] = need, {}, {}, 2 * need
            st["arena"] = SymmetricBuffer(2 * need + cnt_cap, torch.float32, x2.device, self.group)
            st["cnt_cap"] = 2 * need + cnt_cap
            st["arena"].barrier(0)
        key = (T, N)
        if key not in st["cnt"]:
            n = (rs_counters(rows, N) + 63) // 64 * 64
            assert st["cnt_next"] + 2 * n <= st["cnt_cap"], "too many distinct row-parallel shapes for the staging arena"
            st["cnt"][key], st["uses"][key] = (st["cnt_next"], n), [0, 0]
            st["cnt_next"] += 2 * n
        if st["slice"] is None or st["slice"].tensor.numel() < rows * N:
            st["slice"] = SymmetricBuffer(rows * N, torch.bfloat16, x2.device, self.group)
        parity = st["calls"] & 1
        st["calls"] += 1
        st["uses"][key][parity] += 1
        target = (W * st["uses"][key][parity]) & 0xFFFFFFFF
        if target >= 1 << 31:
            target -= 1 << 32
        slot = rows * N
        data_off = parity * st["area"] * 4
        cnt_off = (st["cnt"][key][0] + parity * st["cnt"][key][1]) * 4
        peers = st["arena"].peer_ptrs
        slots = _ptr_array([p + data_off + r * slot * 4 for p in peers])
        cnts = _ptr_array([p + cnt_off for p in peers])
        mine = st["slice"].tensor[:rows * N].view(rows, N)
        reduce_scatter_gemm(x2, w, False, slots, cnts, r, W, peers[r] + data_off, slot, True, target, mine, False, T, N, K, 1.0)
        st["slice"].barrier(0)  # every rank's reduced rows are complete; a rank overwrites its rows only inside its next product,
        #                         whose units need a contribution from every peer, i.e. after every peer's pull below
        y = torch.empty(T, N, dtype=torch.bfloat16, device=x2.device)
        tkey = (rows * N, W, r)
        if tkey not in st["tables"]:
            nbytes = rows * N * 2
            tab = []
            for i in range(W):
                src = (r + 1 + i) % W
                for off in range(0, nbytes, 16384):
                    tab.append((src, off // 16, (src * nbytes + off) // 16, min(16384, nbytes - off) // 16))
            st["tables"][tkey] = (torch.tensor(tab, dtype=torch.int32, device=x2.device), len(tab))
        table, n_units = st["tables"][tkey]
        c = lib
        f = lib.fn("lvb_copy_job", [c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_void_p])
        rc = f(table.data_ptr(), 0, n_units, st["slice"].c_ptrs, W, y.data_ptr(), 0, lib.status_buffer().data_ptr(), lib.stream_ptr())
        lib.check_rc(rc, "lvb_copy_job")
        self.fused_row_linears = getattr(self, "fused_row_linears", 0) + 1
        return y

    def row_linear(self, x: torch.Tensor, linear) -> torch.Tensor:
        """Row-parallel projection without its bias: ``all_reduce(x @ W_local.T)``, on the fused path when the shapes allow."""
        w = linear.weight
        x2 = x.reshape(-1, x.shape[-1])
        if type(linear).__name__ == "Linear" and w.dtype == x.dtype and self.fused_row_linear_ok(x2, w):
            return _RowLinearFn.apply(x, w, self)
        return self.reduce_from_region(linear(x, skip_bias=True))

    def all_gather_last_dim(self, x: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


def shard_full_state_(model: torch.nn.Module, full_state: dict, tp: Optional["TensorParallel"], ep=None) -> None:
    """Fill a tensor-parallel ``model`` from the tensors of the unsharded model: every parameter marked ``tp_dim`` takes
    this rank's slice along that dimension (heads and MLP columns are contiguous per rank), the others are copied whole.
    Parameters marked ``ep_dim`` (experts sliced over the ranks of ``ep``) take that group's slice of the expert axis.
    Used to serve (or continue training) a checkpoint on a model axis of any size."""
    rank = tp.rank if tp is not None else 0
    with torch.no_grad():
        for name, p in model.named_parameters():
            src = full_state[name]
            edim = getattr(p, "ep_dim", None)
            if edim is not None and ep is not None and src.shape[edim] != p.shape[edim]:
                n = p.shape[edim]
                src = src.narrow(edim, ep.rank * n, n)
            dim = getattr(p, "tp_dim", None)
            if dim is not None and src.shape != p.shape:
                n = p.shape[dim]
                src = src.narrow(dim, rank * n, n)
            if src.shape != p.shape:
                raise ValueError(f"{name}: cannot place {tuple(full_state[name].shape)} into {tuple(p.shape)} (tp_dim={dim})")
            p.copy_(src.to(p.dtype))


def gather_full_state(model: torch.nn.Module, tp: Optional["TensorParallel"]) -> dict:
    """Inverse of :func:`shard_full_state_`: name -> unsharded tensor, assembled from every rank's slice along ``tp_dim``
    (collective over the model axis; parameters without ``tp_dim`` are returned as they are)."""
    out = {}
    with torch.no_grad():
        for name, p in model.named_parameters():
            dim = getattr(p, "tp_dim", None)
            if tp is None or tp.size <= 1 or dim is None:
                out[name] = p.detach().clone()
                continue
            parts = [torch.empty_like(p) for _ in range(tp.size)]
            dist.all_gather(parts, p.detach().contiguous(), group=tp.group)
            out[name] = torch.cat(parts, dim=dim)
    return out


def build_sharded_from_seed(build, tp: Optional["TensorParallel"], ep=None):
    """A tensor-parallel model whose weights are this rank's slices of the model that ``build(tp=None)`` creates, so that a
    run on a model axis of any size starts from the same weights as an unsharded run with the same seed.  ``ep``: the
    expert-parallel group of a model built with sliced experts (its ``ep_dim`` parameters take their slice as well)."""
    if tp is None or tp.size <= 1:
        return build(tp=None)
    full = build(tp=None)
    model = build(tp=tp)
    if ep is None:  # a model that sliced its experts by itself carries the group on its expert blocks
        ep = next((m.ep for m in model.modules() if getattr(m, "ep", None) is not None), None)
    shard_full_state_(model, {n: p.detach() for n, p in full.named_parameters()}, tp, ep)
    del full
    return model
