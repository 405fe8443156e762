"""Newton-Schulz orthogonalisation for Muon / Scion (src/levanter/optim/muon.py:171-202).

Five (or ten) iterations of ``A = X X^T; B = b A + c A^2; X = a X + B X`` with ``(a, b, c) = (3.4445, -4.7750, 2.0315)``
on the Frobenius-normalised matrix (transposed first when it is tall).  On a B200 the three products per iteration run on
the tcgen05 GEMM in bf16 with fp32 accumulation; none of them needs a transposed copy because the kernel reads either
operand K-major or MN-major.  The reference reshards each matrix over the whole mesh before iterating (:189-192); here
whole matrices are distributed round-robin over the data ranks by the optimizer, so every product is local."""
from __future__ import annotations

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
        Xb = X.contiguous().to(torch.bfloat16)
        for _ in range(steps):
            A = gemm(Xb, Xb)                                   # X X^T   [m, m]
            A2 = gemm(A, A, b_mn=True, out_dtype=torch.float32)  # A A (A is symmetric; read as [K, N])
            Bm = (_B * A.float() + _C * A2).to(torch.bfloat16)
            BX = gemm(Bm, Xb, b_mn=True, out_dtype=torch.float32)  # B X
            Xb = (_A * Xb.float() + BX).to(torch.bfloat16)
        X = Xb.float()
    else:
        for _ in range(steps):
            A = X @ X.t()
            Bm = _B * A + _C * (A @ A)
            X = _A * X + Bm @ X
    if transpose:
        X = X.t()
    return X.to(out_dtype)
