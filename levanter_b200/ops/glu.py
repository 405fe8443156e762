"""Gated activation ``act(gate) * up`` (``csrc/elementwise.cu``): SwiGLU / GeGLU MLPs
(src/levanter/models/llama.py:273-280)."""
from __future__ import annotations

import torch

from . import lib
from ..utils.activation import ActivationFunctionEnum

_ACT = {
    ActivationFunctionEnum.silu: 0, ActivationFunctionEnum.swish: 0, ActivationFunctionEnum.gelu_new: 1,
    ActivationFunctionEnum.gelu: 2, ActivationFunctionEnum.relu: 3, ActivationFunctionEnum.quick_gelu: 4,
}
_f = {}


def _fwd():
    if "f" not in _f:
        c = lib
        _f["f"] = lib.fn("lvb_glu_fwd", [c.c_void_p] * 3 + [c.c_int, c.c_int] + [c.c_longlong] * 3 + [c.c_int, c.c_void_p])
    return _f["f"]


def _bwd():
    if "b" not in _f:
        c = lib
        _f["b"] = lib.fn("lvb_glu_bwd", [c.c_void_p] * 5 + [c.c_int, c.c_int] + [c.c_longlong] * 5 + [c.c_int, c.c_void_p])
    return _f["b"]


class _GluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up, act):
        cols = gate.shape[-1]
        g2 = gate.reshape(-1, cols)
        u2 = up.reshape(-1, cols)
        if g2.stride(1) != 1:
            g2 = g2.contiguous()
        if u2.stride(1) != 1:
            u2 = u2.contiguous()
        out = torch.empty(g2.shape, dtype=gate.dtype, device=gate.device)
        rc = _fwd()(g2.data_ptr(), u2.data_ptr(), out.data_ptr(), g2.shape[0], cols, g2.stride(0), u2.stride(0), out.stride(0),
                    act, lib.stream_ptr())
        lib.check_rc(rc, "lvb_glu_fwd")
        ctx.save_for_backward(g2, u2)
        ctx.act = act
        ctx.shape = gate.shape
        return out.view(gate.shape)

    @staticmethod
    def backward(ctx, dout):
        g2, u2 = ctx.saved_tensors
        cols = g2.shape[1]
        d2 = dout.reshape(-1, cols)
        if d2.dtype != torch.bfloat16 or d2.stride(1) != 1:
            d2 = d2.to(torch.bfloat16).contiguous()
        dg = torch.empty(g2.shape, dtype=g2.dtype, device=g2.device)
        du = torch.empty(g2.shape, dtype=g2.dtype, device=g2.device)
        rc = _bwd()(d2.data_ptr(), g2.data_ptr(), u2.data_ptr(), dg.data_ptr(), du.data_ptr(), g2.shape[0], cols, d2.stride(0),
                    g2.stride(0), u2.stride(0), dg.stride(0), du.stride(0), ctx.act, lib.stream_ptr())
        lib.check_rc(rc, "lvb_glu_bwd")
        return dg.view(ctx.shape), du.view(ctx.shape), None


def gated_activation(gate: torch.Tensor, up: torch.Tensor, act: ActivationFunctionEnum) -> torch.Tensor:
    act = ActivationFunctionEnum(act) if not isinstance(act, ActivationFunctionEnum) else act
    if (gate.is_cuda and lib.available() and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16
            and gate.shape[-1] % 8 == 0 and act in _ACT):
        return _GluFn.apply(gate, up, _ACT[act])
    return act.to_fn()(gate) * up
