"""PSGD-Kron (src/levanter/optim/kron.py): Kronecker-factored preconditioning ``P = Q^T Q`` with one triangular (or
diagonal) factor per tensor dimension, fitted online with the PSGD whitening criterion.

Per step: momentum ``mu = b1 mu + (1 - b1) g`` (bias-corrected); with probability from the annealed schedule
(1.0 for ``flat_start`` steps, then ``exp`` decay to 0.03, :176-192) each factor takes one normalised gradient step of size
``preconditioner_lr`` on the criterion ``E[v^T P v + v^T P^-1 v]`` using a random probe ``v``; the update is ``P mu`` followed
by ``clip_by_block_rms(1.1)`` (:150), weight decay and ``-lr``.  Dimensions larger than ``max_size_triangular`` (or tensors
with fewer than ``min_ndim_triangular`` dims, or per ``memory_save_mode``) use diagonal factors.  Matrices may be partitioned
into ``block_size`` blocks and small dims merged up to ``target_merged_dim_size`` as in the reference."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, NamedTuple, Optional, Tuple, Union

import torch

from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .soap import _blocks, _merge_small_dims
from .transforms import GradientTransformation, Tree
from .util import scan_aware_clip_by_block_rms


def precond_update_prob_schedule(max_prob: float = 1.0, min_prob: float = 0.03, decay: float = 0.001, flat_start: int = 500):
    def _schedule(n):
        return float(min(max(max_prob * math.exp(-decay * (n - flat_start)), min_prob), max_prob))

    return _schedule


class KronState(NamedTuple):
    count: int
    mu: Tree
    Qs: Dict[str, Any]       # name -> list over blocks of [Q_0, Q_1, ...] (2-D upper-triangular or 1-D diagonal factors)
    update_counter: float


def _init_Q(shape: Tuple[int, ...], scale: float, max_size: int, min_ndim: int, memory_save_mode: Optional[str], device):
    nd = len(shape)
    if memory_save_mode is None:
        diag = [False] * nd
    elif memory_save_mode == "one_diag":
        big = max(range(nd), key=lambda i: shape[i]) if nd else 0
        diag = [i == big for i in range(nd)]
    elif memory_save_mode == "all_diag":
        diag = [True] * nd
    else:
        raise ValueError(f"invalid memory_save_mode {memory_save_mode!r}")
    Qs = []
    s = scale ** (1.0 / max(nd, 1))
    for i, size in enumerate(shape):
        if size == 1 or size > max_size or nd < min_ndim or diag[i]:
            Qs.append(s * torch.ones(size, dtype=torch.float32, device=device))
        else:
            Qs.append(s * torch.eye(size, dtype=torch.float32, device=device))
    return Qs


def _apply_Q(Qs, x, transpose_first=False):
    """Multiply each mode of ``x`` by its factor (``Q`` or ``Q^T``)."""
    for i, q in enumerate(Qs):
        if q.dim() == 1:
            shape = [1] * x.dim()
            shape[i] = -1
            x = x * q.view(shape)
        else:
            m = q.t() if transpose_first else q
            x = torch.movedim(torch.tensordot(m, x, dims=([1], [i])), 0, i)
    return x


def _solve_Q(Qs, x):
    """Multiply each mode of ``x`` by ``Q^-T`` (triangular solves)."""
    for i, q in enumerate(Qs):
        if q.dim() == 1:
            shape = [1] * x.dim()
            shape[i] = -1
            x = x / q.view(shape)
        else:
            xm = torch.movedim(x, i, 0)
            flat = xm.reshape(xm.shape[0], -1)
            sol = torch.linalg.solve_triangular(q.t(), flat, upper=False)
            x = torch.movedim(sol.reshape(xm.shape), 0, i)
    return x


def _update_precond(Qs, g, lr: float, probe_seed: Optional[int] = None):
    """One PSGD step on every factor: ``A = Q g`` (all modes), ``B = Q^-T v``-style conjugate with the probe folded into g.
    The probe is drawn from a generator seeded with ``probe_seed`` (a function of the optimizer's seed, the step and the
    leaf), so a resumed run and every rank draw the probes an uninterrupted run would."""
    if probe_seed is None:
        v = torch.randn_like(g)
    else:
        gen = torch.Generator(device=g.device)
        gen.manual_seed(probe_seed)
        v = torch.randn(g.shape, generator=gen, device=g.device, dtype=g.dtype)
    gn = g + math.sqrt(torch.finfo(torch.float32).eps) * g.abs().mean() * v
    A = _apply_Q(Qs, gn)
    Bc = _solve_Q(Qs, v)
    for i, q in enumerate(Qs):
        Am = torch.movedim(A, i, 0).reshape(A.shape[i], -1)
        Bm = torch.movedim(Bc, i, 0).reshape(Bc.shape[i], -1)
        if q.dim() == 1:
            t1 = (Am * Am).sum(1)
            t2 = (Bm * Bm).sum(1)
            q.sub_(lr / (t1 + t2).max().clamp_min(1e-30) * (t1 - t2) * q)
        else:
            t1 = Am @ Am.t()
            t2 = Bm @ Bm.t()
            norm = torch.linalg.matrix_norm(t1 + t2, ord="fro").clamp_min(1e-30)
            q.sub_(lr / norm * torch.triu(t1 - t2) @ q)


def scale_by_kron(b1: float = 0.9, normalize_grads: bool = False,
                  preconditioner_update_probability: Union[float, Callable[[int], float]] = precond_update_prob_schedule(),
                  max_size_triangular: int = 8192, min_ndim_triangular: int = 2, memory_save_mode: Optional[str] = None,
                  preconditioner_lr: float = 0.1, preconditioner_init_scale: float = 1.0, merge_small_dims: bool = False,
                  target_merged_dim_size: int = 2048, partition_grads_into_blocks: bool = False, block_size: int = 256,
                  seed: int = 0) -> GradientTransformation:

    def plan(p):
        shape = tuple(p.shape)
        if merge_small_dims and len(shape) > 1:
            shape = _merge_small_dims(shape, target_merged_dim_size)
        return shape

    def block_slices(shape):
        if not partition_grads_into_blocks or len(shape) != 2:
            return [tuple(slice(0, s) for s in shape)]
        return [(slice(r0, r1), slice(c0, c1)) for (r0, r1) in _blocks(shape[0], block_size) for (c0, c1) in _blocks(shape[1], block_size)]

    def init(params):
        mu = T.tree_zeros_like(params)
        Qs = {}
        for k, p in params.items():
            if p is None:
                continue
            shape = plan(p)
            Qs[k] = [_init_Q(tuple(sl.stop - sl.start for sl in bs), preconditioner_init_scale, max_size_triangular,
                             min_ndim_triangular, memory_save_mode, p.device) for bs in block_slices(shape)]
        return KronState(0, mu, Qs, 0.0)

    def update(updates, state, params=None, **extra):
        count = state.count + 1
        prob = preconditioner_update_probability(state.count) if callable(preconditioner_update_probability) else float(preconditioner_update_probability)
        counter = state.update_counter + prob
        do_update = counter >= 1.0
        if do_update:
            counter -= 1.0
        out = dict(updates)
        for leaf_index, k in enumerate(T.tree_keys(updates)):
            g = updates[k].float()
            if normalize_grads:
                g = g / (g.norm() + 1e-16)
            mu = state.mu[k]
            mu.mul_(b1).add_(g.to(mu.dtype), alpha=1 - b1)
            mhat = (mu / (1 - b1 ** count)).float()
            shape = plan(g)
            m2 = mhat.reshape(shape)
            res = torch.empty_like(m2)
            for block_index, (bs, Qs) in enumerate(zip(block_slices(shape), state.Qs[k])):
                blk = m2[bs]
                if do_update:
                    probe_seed = (seed * 1_000_003 + count * 7_919 + leaf_index * 104_729 + block_index) % (2 ** 63 - 1)
                    _update_precond(Qs, blk, preconditioner_lr, probe_seed)
                # P mu = Q^T (Q mu)
                res[bs] = _apply_Q(Qs, _apply_Q(Qs, blk), transpose_first=True)
            out[k] = res.reshape(updates[k].shape).to(updates[k].dtype)
        return out, KronState(count, state.mu, state.Qs, counter)

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("kron")
@dataclass(frozen=True)
class KronConfig(OptimizerConfig):
    beta1: float = 0.9
    weight_decay: float = 0.1
    max_grad_norm: Optional[float] = 1.0
    normalize_grads: bool = False
    preconditioner_update_probability: float = 0.05
    update_prob_flat_start: int = 500
    max_size_triangular: int = 25000
    min_ndim_triangular: int = 2
    memory_save_mode: Optional[str] = None
    preconditioner_lr: float = 0.1
    preconditioner_init_scale: float = 1.0
    mu_dtype: Optional[str] = None
    precond_dtype: Optional[str] = None
    precond_update_precision: Optional[str] = "tensorfloat32"
    precond_grads_precision: Optional[str] = None
    lax_map_scanned_layers: bool = False
    lax_map_batch_size: int = 8
    merge_small_dims: bool = True
    target_merged_dim_size: int = 8192
    partition_grads_into_blocks: bool = True
    block_size: int = 256
    params_sharding: Optional[Any] = None
    preconditioner_sharding: Optional[Any] = None
    needs_full_tensors = True

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        cache: Dict = {}
        sched = precond_update_prob_schedule(min_prob=self.preconditioner_update_probability, flat_start=self.update_prob_flat_start)
        kron = scale_by_kron(self.beta1, self.normalize_grads, sched, self.max_size_triangular, self.min_ndim_triangular,
                             self.memory_save_mode, self.preconditioner_lr, self.preconditioner_init_scale,
                             self.merge_small_dims, self.target_merged_dim_size, self.partition_grads_into_blocks, self.block_size)

        def _optimizer(learning_rate):
            comps = []
            if self.max_grad_norm:
                comps.append(T.clip_by_global_norm(self.max_grad_norm))
            comps.append(kron)
            comps.append(scan_aware_clip_by_block_rms(1.1))
            if self.weight_decay > 0:
                comps.append(_decay(self.weight_decay, mask_fn, cache))
            comps.append(T.scale_by_learning_rate(learning_rate))
            return T.chain(*comps)

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
