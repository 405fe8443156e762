"""The carried-state loop of the chunked gated delta rule (``csrc/delta_rule.cu``).

Given, for every chunk ``n`` of 64 tokens, the tiles that can be computed for all chunks at once

* ``w [.., N, C, dk]`` and ``u [.., N, C, dv]`` (the WY factors of the chunk),
* ``qg [.., N, C, dk]`` (queries times their decay from the chunk start), ``kd [.., N, C, dk]`` (keys times their decay to
  the chunk end), ``P [.., N, C, C]`` (decayed, causally masked query-key scores) and ``a [.., N]`` (decay over the chunk),

:func:`chunk_state_scan` runs ::

    v_new = u_n - w_n S;   o_n = qg_n S + P_n v_new;   S = a_n S + kd_n^T v_new

over the chunks and returns ``(o [.., N, C, dv], final S [.., dk, dv])``.  On a B200 both directions are one kernel launch
(the state never leaves shared memory); elsewhere the same loop runs on PyTorch ops, which is also the test oracle.  The
reference framework has no counterpart (the model family is an addition)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import lib

CHUNK = 64


def _supported(w: torch.Tensor, u: torch.Tensor) -> bool:
    return (w.is_cuda and lib.available() and w.shape[-2] == CHUNK and w.shape[-1] in (64, 128)
            and u.shape[-1] % 64 == 0 and w.dtype == torch.float32)


def chunk_state_scan_reference(w, qg, kd, P, u, a, S0: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The loop on PyTorch ops (differentiable by autograd)."""
    N = w.shape[-3]
    dk, dv = w.shape[-1], u.shape[-1]
    S = w.new_zeros(*w.shape[:-3], dk, dv) if S0 is None else S0.to(w.dtype)
    outs = []
    for n in range(N):
        v_new = u[..., n, :, :] - w[..., n, :, :] @ S
        outs.append(qg[..., n, :, :] @ S + P[..., n, :, :] @ v_new)
        S = S * a[..., n, None, None] + kd[..., n, :, :].transpose(-1, -2) @ v_new
    return torch.stack(outs, dim=-3), S


_fwd = _bwd = _slices = None


def _bind():
    global _fwd, _bwd, _slices
    if _fwd is None:
        P = lib.c_void_p
        _fwd = lib.fn("lvb_delta_rule_fwd", [P] * 10 + [lib.c_int] * 5 + [P])
        _bwd = lib.fn("lvb_delta_rule_bwd", [P] * 16 + [lib.c_int] * 5 + [P])
        _slices = lib.fn("lvb_delta_rule_bwd_slices", [lib.c_int], launches=0)


class _ChunkStateScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, qg, kd, P, u, a, S0, exact):
        _bind()
        lead = w.shape[:-3]
        N, C, dk = w.shape[-3:]
        dv = u.shape[-1]
        BH = 1
        for s in lead:
            BH *= s
        w, qg, kd, P, u, a = (t.contiguous() for t in (w, qg, kd, P, u, a))
        S0c = None if S0 is None else S0.float().contiguous()
        need_grad = any(ctx.needs_input_grad)
        out = torch.empty(*lead, N, C, dv, dtype=torch.float32, device=w.device)
        S_final = torch.empty(*lead, dk, dv, dtype=torch.float32, device=w.device)
        S_hist = torch.empty(*lead, N, dk, dv, dtype=torch.float32, device=w.device) if need_grad else None
        rc = _fwd(lib.ptr(w), lib.ptr(qg), lib.ptr(kd), lib.ptr(P), lib.ptr(u), lib.ptr(a), lib.ptr(S0c), lib.ptr(out),
                  lib.ptr(S_hist), lib.ptr(S_final), BH, N, dk, dv, int(exact), lib.stream_ptr())
        lib.check_rc(rc, "delta_rule_fwd")
        if need_grad:
            ctx.save_for_backward(w, qg, kd, P, u, a, S_hist)
        ctx.dims = (lead, BH, N, C, dk, dv, bool(exact), S0 is not None)
        return out, S_final

    @staticmethod
    def backward(ctx, dout, dS_final):
        w, qg, kd, P, u, a, S_hist = ctx.saved_tensors
        lead, BH, N, C, dk, dv, exact, has_s0 = ctx.dims
        dev = w.device
        ns = _slices(dv)
        dout = torch.zeros_like(u) if dout is None else dout.float().contiguous()
        dSf = None if dS_final is None else dS_final.float().contiguous()
        dw, dqg, dkd = (torch.empty(ns, *lead, N, C, dk, dtype=torch.float32, device=dev) for _ in range(3))
        dP = torch.empty(ns, *lead, N, C, C, dtype=torch.float32, device=dev)
        da = torch.empty(ns, *lead, N, dtype=torch.float32, device=dev)
        du = torch.empty_like(u)
        dS0 = torch.empty(*lead, dk, dv, dtype=torch.float32, device=dev) if has_s0 else None
        rc = _bwd(lib.ptr(w), lib.ptr(qg), lib.ptr(kd), lib.ptr(P), lib.ptr(u), lib.ptr(a), lib.ptr(S_hist), lib.ptr(dout),
                  lib.ptr(dSf), lib.ptr(dw), lib.ptr(dqg), lib.ptr(dkd), lib.ptr(dP), lib.ptr(da), lib.ptr(du), lib.ptr(dS0),
                  BH, N, dk, dv, int(exact), lib.stream_ptr())
        lib.check_rc(rc, "delta_rule_bwd")
        # the per-slice partial sums are added in slice order, so the gradients do not depend on scheduling
        return dw.sum(0), dqg.sum(0), dkd.sum(0), dP.sum(0), du, da.sum(0), dS0, None


def chunk_state_scan(w, qg, kd, P, u, a, S0: Optional[torch.Tensor] = None, *, exact: bool = False):
    """See the module docstring.  ``exact`` makes the kernel use fp32 FMAs instead of TF32 tensor-core products."""
    if not _supported(w, u):  # CPU, or a shape the kernel does not cover (chunk != 64, d_k not 64/128, d_v % 64 != 0)
        return chunk_state_scan_reference(w, qg, kd, P, u, a, S0)
    return _ChunkStateScan.apply(w, qg, kd, P, u, a, S0, exact)
