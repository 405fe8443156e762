"""Newton-Schulz orthogonalisation for Muon / Scion (src/levanter/optim/muon.py:171-202).

Five (or ten) iterations of ``A = X X^T; B = b A + c A^2; X = a X + B X`` with ``(a, b, c) = (3.4445, -4.7750, 2.0315)``
on the Frobenius-normalised matrix (transposed first when it is tall).  On a B200 the three products per iteration run on
the tcgen05 GEMM in bf16 with fp32 accumulation; none of them needs a transposed copy because the kernel reads either
operand K-major or MN-major.  The reference reshards each matrix over the whole mesh before iterating (:189-192); here a
call of :func:`zeropower_via_newtonschulz5` works on one whole local matrix, and :func:`orthogonalize_tree` deals the
matrices of a step out over the ranks that hold identical copies of them (largest first, to the least loaded rank), each
rank iterates its own share and broadcasts the results: the step costs ``1/W`` of the matrix products per rank plus one
pass of the orthogonalised matrices over the interconnect, and no matrix is ever cut up."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import lib
from .gemm import gemm

_A, _B, _C = 3.4445, -4.7750, 2.0315


def zeropower_via_newtonschulz5(X: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    assert X.dim() == 2
    out_dtype = X.dtype
    X = X.float()
    X = X / (X.norm() + eps)
    transpose = X.shape[0] > X.shape[1]
    if transpose:
        X = X.t()
    use_kernel = X.is_cuda and lib.available() and X.shape[0] % 8 == 0 and X.shape[1] % 8 == 0
    if use_kernel:
        # Three GEMMs per iteration and nothing between them: the polynomial's coefficients ride in the epilogues (alpha and
        # the residual operand).  With the iterate kept as X = s Xs:
        #   A   = s^2 Xs Xs^T                       alpha = s^2
        #   B'  = A + (c / b) A A                   alpha = c / b, residual A          (the true B is b B')
        #   Xs' = Xs + (b / a) B' Xs                alpha = b / a, residual Xs         (a X + B X = a s Xs'),   s' = a s
        Xs = X.contiguous().to(torch.bfloat16)
        s = 1.0
        for _ in range(steps):
            A = gemm(Xs, Xs, alpha=s * s)                                 # [m, m]
            Bp = gemm(A, A, b_mn=True, alpha=_C / _B, residual=A)         # A is symmetric; read as [K, N]
            Xs = gemm(Bp, Xs, b_mn=True, alpha=_B / _A, residual=Xs)      # [m, n]
            s *= _A
        X = Xs.float() * s
    else:
        for _ in range(steps):
            A = X @ X.t()
            Bm = _B * A + _C * (A @ A)
            X = _A * X + Bm @ X
    if transpose:
        X = X.t()
    return X.to(out_dtype)


_layer_group = None


def set_layer_parallel_group(group) -> None:
    """Ranks of ``group`` hold identical optimizer inputs (unsharded optimizer on data-parallel ranks): let them share the
    orthogonalisations.  ``None`` switches the sharing off."""
    global _layer_group
    _layer_group = group


def assign_owners(costs: Dict[str, float], world: int) -> Dict[str, int]:
    """Deterministic longest-processing-time assignment of matrices to ranks (the same on every rank)."""
    load = [0.0] * world
    owner: Dict[str, int] = {}
    for k in sorted(costs, key=lambda k: (-costs[k], k)):
        r = min(range(world), key=lambda i: (load[i], i))
        owner[k] = r
        load[r] += costs[k]
    return owner


def orthogonalize_tree(mats: Dict[str, torch.Tensor], steps: int = 5, eps: float = 1e-7) -> Dict[str, torch.Tensor]:
    """Newton-Schulz on every matrix of ``mats``, shared over the layer-parallel group when one is set."""
    import torch.distributed as dist

    group = _layer_group
    world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    if world <= 1:
        return {k: zeropower_via_newtonschulz5(m, steps=steps, eps=eps) for k, m in mats.items()}
    rank = dist.get_rank(group)
    owner = assign_owners({k: float(min(m.shape) ** 2 * max(m.shape)) for k, m in mats.items()}, world)
    out: Dict[str, torch.Tensor] = {}
    for k, m in mats.items():
        out[k] = zeropower_via_newtonschulz5(m, steps=steps, eps=eps).contiguous() if owner[k] == rank else torch.empty_like(m)
    pending = [dist.broadcast(out[k], src=dist.get_global_rank(group, owner[k]), group=group, async_op=True) for k in sorted(out)]
    for w in pending:
        w.wait()
    return out
