"""Python bindings of ``csrc/optim.cu``: deterministic sum of squares, clip coefficient, fused AdamW."""
from __future__ import annotations

import torch

from . import lib

_f = {}
_scratch = {}


def _get(name, argtypes):
    if name not in _f:
        _f[name] = lib.fn(name, argtypes)
    return _f[name]


def _scr(device) -> torch.Tensor:
    k = torch.cuda.current_device()
    if k not in _scratch:
        _scratch[k] = torch.empty(1024, dtype=torch.float32, device=device)
    return _scratch[k]


def sumsq(x: torch.Tensor, out: torch.Tensor = None, accumulate: bool = False) -> torch.Tensor:
    c = lib
    f = _get("lvb_sumsq", [c.c_void_p, c.c_longlong, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p])
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    x = x.contiguous()
    if x.numel() == 0:
        return out
    rc = f(x.data_ptr(), x.numel(), int(x.dtype == torch.bfloat16), _scr(x.device).data_ptr(), out.data_ptr(), int(accumulate),
           lib.stream_ptr())
    lib.check_rc(rc, "lvb_sumsq")
    return out


def clip_coef(sumsq_t: torch.Tensor, max_norm: float, coef: torch.Tensor, norm_out: torch.Tensor = None) -> None:
    c = lib
    f = _get("lvb_clip_coef", [c.c_void_p, c.c_float, c.c_void_p, c.c_void_p, c.c_void_p])
    rc = f(sumsq_t.data_ptr(), float(max_norm), coef.data_ptr(), lib.ptr(norm_out), lib.stream_ptr())
    lib.check_rc(rc, "lvb_clip_coef")


def adamw(p, m, v, g, p_lowp, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, grad_mul=1.0, nesterov=False) -> None:
    c = lib
    f = _get("lvb_adamw", [c.c_void_p] * 4 + [c.c_int, c.c_void_p, c.c_longlong] + [c.c_float] * 7 + [c.c_void_p, c.c_float, c.c_int, c.c_void_p])
    if g.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("gradients must be fp32 or bf16")
    if p_lowp is not None and p_lowp.dtype != torch.bfloat16:
        raise TypeError("the compute-dtype copy must be bf16")
    rc = f(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), int(g.dtype == torch.bfloat16), lib.ptr(p_lowp), p.numel(),
           float(lr), float(b1), float(b2), float(eps), float(wd), float(bc1), float(bc2), lib.ptr(grad_scale), float(grad_mul),
           int(nesterov), lib.stream_ptr())
    lib.check_rc(rc, "lvb_adamw")
