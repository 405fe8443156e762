"""SOAP: Adam in the eigenbasis of Shampoo's preconditioners (src/levanter/optim/soap.py).

For each 2-D block ``G`` (matrices are cut into ``block_size`` x ``block_size`` blocks when ``partition_grads_into_blocks``,
small dimensions merged up to ``target_merged_dim_size``, dimensions above ``max_precond_dim`` left un-preconditioned) the
state holds ``L = EMA(G G^T)``, ``R = EMA(G^T G)`` and their eigenbases ``Q_L, Q_R``; Adam's moments live in the rotated space
``Q_L^T G Q_R``; every ``precondition_frequency`` steps the bases are refreshed by one power-iteration + QR step (eigh the first
time) and the second moment is carried into the new basis.  1-D parameters use plain Adam."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, NamedTuple, Optional, Tuple, Union

import torch

from . import transforms as T
from .config import OptimizerConfig, ParamInfo, _decay
from .transforms import GradientTransformation, Tree


class ScaleBySoapState(NamedTuple):
    count: int
    exp_avg: Tree
    exp_avg_sq: Tree
    GG: Dict[str, Any]   # name -> list over blocks of (L, R) (None for un-preconditioned sides)
    Q: Dict[str, Any]    # name -> list over blocks of (Q_L, Q_R)


def _merge_small_dims(shape: Tuple[int, ...], target: int) -> Tuple[int, ...]:
    """Greedily merge adjacent dimensions while the product stays <= target (always ends with <= 2 dims for matrices)."""
    if len(shape) <= 1:
        return tuple(shape)
    out: List[int] = []
    cur = 1
    for s in shape:
        if cur * s <= target or cur == 1:
            cur *= s
        else:
            out.append(cur)
            cur = s
    out.append(cur)
    if len(out) > 2:
        out = [math.prod(out[:-1]), out[-1]]
    return tuple(out)


def _blocks(n: int, b: int) -> List[Tuple[int, int]]:
    return [(i, min(i + b, n)) for i in range(0, n, b)]


def scale_by_soap(b1: float = 0.95, b2: float = 0.95, shampoo_beta: float = -1.0, eps: float = 1e-8,
                  precondition_frequency: int = 10, max_precond_dim: int = 10000, merge_small_dims: bool = True,
                  one_diag: bool = False, target_merged_dim_size: int = 2048, partition_grads_into_blocks: bool = True,
                  block_size: int = 256) -> GradientTransformation:
    sb = shampoo_beta if shampoo_beta >= 0 else b2

    def plan(p: torch.Tensor):
        if p.dim() < 2:
            return None
        shape = _merge_small_dims(tuple(p.shape), target_merged_dim_size) if (merge_small_dims or p.dim() > 2) else tuple(p.shape)
        if len(shape) < 2:
            return None
        m, n = shape[0], math.prod(shape[1:])
        bs = block_size if partition_grads_into_blocks else max(m, n)
        return (m, n), _blocks(m, bs), _blocks(n, bs)

    def init(params):
        exp_avg = T.tree_zeros_like(params)
        exp_avg_sq = T.tree_zeros_like(params)
        GG, Q = {}, {}
        for k, p in params.items():
            if p is None:
                continue
            pl = plan(p)
            if pl is None:
                continue
            (m, n), rb, cb = pl
            ggs, qs = [], []
            for (r0, r1) in rb:
                for (c0, c1) in cb:
                    dl, dr = r1 - r0, c1 - c0
                    L = torch.zeros(dl, dl, dtype=torch.float32, device=p.device) if dl <= max_precond_dim else None
                    R = torch.zeros(dr, dr, dtype=torch.float32, device=p.device) if (dr <= max_precond_dim and not one_diag) else None
                    ggs.append([L, R])
                    qs.append([None, None])
            GG[k], Q[k] = ggs, qs
        return ScaleBySoapState(0, exp_avg, exp_avg_sq, GG, Q)

    def project(g, q, back=False):
        ql, qr = q
        if ql is not None:
            g = (ql @ g) if back else (ql.t() @ g)
        if qr is not None:
            g = (g @ qr.t()) if back else (g @ qr)
        return g

    def refresh_basis(gg, q, v_block):
        new_q = []
        for side, (m, qo) in enumerate(zip(gg, q)):
            if m is None:
                new_q.append(None)
                continue
            if qo is None:
                _, vec = torch.linalg.eigh(m + 1e-30 * torch.eye(m.shape[0], device=m.device))
                new_q.append(vec.flip(1))
            else:
                est = torch.diag(qo.t() @ m @ qo)
                order = torch.argsort(est, descending=True)
                qs = qo[:, order]
                if v_block is not None:
                    v_block.copy_(v_block.index_select(side, order))
                qn, _ = torch.linalg.qr(m @ qs)
                new_q.append(qn)
        return new_q

    def update(updates, state, params=None, **extra):
        count = state.count + 1
        out = dict(updates)
        for k in T.tree_keys(updates):
            g = updates[k]
            m1, v = state.exp_avg[k], state.exp_avg_sq[k]
            if k not in state.GG:
                m1.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                out[k] = (m1 / (1 - b1 ** count)) / (torch.sqrt(v / (1 - b2 ** count)) + eps)
                continue
            (m, n), rb, cb = plan(g)
            g2 = g.reshape(m, n).float()
            m2, v2 = m1.view(m, n), v.view(m, n)
            res = torch.empty_like(g2)
            bi = 0
            for (r0, r1) in rb:
                for (c0, c1) in cb:
                    gb = g2[r0:r1, c0:c1]
                    gg, q = state.GG[k][bi], state.Q[k][bi]
                    if gg[0] is not None:
                        gg[0].mul_(sb).add_(gb @ gb.t(), alpha=1 - sb)
                    if gg[1] is not None:
                        gg[1].mul_(sb).add_(gb.t() @ gb, alpha=1 - sb)
                    vb = v2[r0:r1, c0:c1]
                    if q[0] is None and q[1] is None and (gg[0] is not None or gg[1] is not None):
                        nq = refresh_basis(gg, q, None)  # first step: eigh of the first outer products
                        q[0], q[1] = nq
                    mb = m2[r0:r1, c0:c1]
                    mb.mul_(b1).add_(gb.to(mb.dtype), alpha=1 - b1)
                    gp = project(gb, q)
                    vb.mul_(b2).addcmul_(gp.to(vb.dtype), gp.to(vb.dtype), value=1 - b2)
                    mp = project(mb.float(), q)
                    step = (mp / (1 - b1 ** count)) / (torch.sqrt(vb.float() / (1 - b2 ** count)) + eps)
                    res[r0:r1, c0:c1] = project(step, q, back=True)
                    if count % precondition_frequency == 0:
                        vtmp = vb.clone()
                        nq = refresh_basis(gg, q, vtmp)
                        vb.copy_(vtmp)
                        q[0], q[1] = nq
                    bi += 1
            out[k] = res.reshape(g.shape).to(g.dtype)
        return out, ScaleBySoapState(count, state.exp_avg, state.exp_avg_sq, state.GG, state.Q)

    return GradientTransformation(init, update)


@OptimizerConfig.register_subclass("soap")
@dataclass(frozen=True)
class SoapConfig(OptimizerConfig):
    weight_decay: float = 0.0
    beta1: float = 0.95
    beta2: float = 0.95
    shampoo_beta: float = 0.95
    epsilon: float = 1e-8
    max_grad_norm: Optional[float] = 1.0
    schedule_list: Optional[List[str]] = None
    precondition_frequency: int = 10
    max_precond_dim: int = 10000
    merge_small_dims: bool = True
    one_diag: bool = False
    target_merged_dim_size: int = 2048
    mu_dtype: Optional[str] = None
    precond_dtype: Optional[str] = None
    partition_grads_into_blocks: bool = True
    block_size: int = 256
    needs_full_tensors = True

    def build(self, num_train_steps: int, param_info: Optional[ParamInfo] = None) -> GradientTransformation:
        mask_fn = self.build_weight_decay_mask(param_info)
        cache: Dict = {}
        # the preconditioner state must persist across the per-step rebuilds of inject_hyperparams
        soap = scale_by_soap(self.beta1, self.beta2, self.shampoo_beta, self.epsilon, self.precondition_frequency,
                             self.max_precond_dim, self.merge_small_dims, self.one_diag, self.target_merged_dim_size,
                             self.partition_grads_into_blocks, self.block_size)

        def _optimizer(learning_rate):
            comps = []
            if self.max_grad_norm:
                comps.append(T.clip_by_global_norm(self.max_grad_norm))
            comps.append(soap)
            if self.weight_decay > 0:
                comps.append(_decay(self.weight_decay, mask_fn, cache))
            comps.append(T.scale(-learning_rate))
            return T.chain(*comps)

        return T.inject_hyperparams(_optimizer)(learning_rate=self.lr_scheduler(num_train_steps))
