"""Element-wise / reduction CUDA kernels against PyTorch fp32 references of the same ops."""
import math

import pytest
import torch

from levanter_b200.layers.rotary import DefaultRotaryEmbeddingsConfig, Llama3RotaryEmbeddingsConfig
from levanter_b200.ops import cross_entropy as CE
from levanter_b200.ops import glu, lib, norm, optim_kernels, rope
from levanter_b200.utils.activation import ActivationFunctionEnum

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    scale = b.abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale}"


@pytest.mark.parametrize("rows,dim", [(64, 4096), (1000, 128), (33, 1024), (7, 8192), (300, 64)])
@pytest.mark.parametrize("ln", [False, True])
def test_norm_fwd_bwd(rows, dim, ln):
    torch.manual_seed(0)
    x = torch.randn(rows, dim, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).requires_grad_()
    b = (0.1 * torch.randn(dim, device="cuda")).requires_grad_() if ln else None
    y, _ = norm.fused_norm(x, w, b, 1e-5, layer_norm=ln)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().clone().requires_grad_()
    br = b.detach().clone().requires_grad_() if ln else None
    if ln:
        yr = torch.nn.functional.layer_norm(xr, (dim,), wr, br, 1e-5)
    else:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(g.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad)
    if ln:
        _close(b.grad, br.grad)


def test_norm_residual_and_gemma_offset():
    torch.manual_seed(1)
    x = torch.randn(96, 512, device="cuda").bfloat16().requires_grad_()
    r = torch.randn(96, 512, device="cuda").bfloat16().requires_grad_()
    w = (0.1 * torch.randn(512, device="cuda")).requires_grad_()
    y, h = norm.fused_norm(x, w, None, 1e-6, w_offset=1.0, residual=r)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    (y * gy).sum().backward(retain_graph=True)
    (h * gh).sum().backward()
    xr, rr, wr = x.detach().float().requires_grad_(), r.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    hr = xr + rr
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + wr)
    ((yr * gy.float()).sum() + (hr * gh.float()).sum()).backward()
    _close(y, yr)
    _close(h, hr)
    _close(x.grad, xr.grad)
    _close(r.grad, rr.grad)
    _close(w.grad, wr.grad)


@pytest.mark.parametrize("cfg", [DefaultRotaryEmbeddingsConfig(), Llama3RotaryEmbeddingsConfig()])
def test_rope(cfg):
    torch.manual_seed(2)
    B, S, H, KV, D = 2, 64, 8, 2, 128
    rot = cfg.build(D)
    q = torch.randn(B, S, H, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, S, KV, D, device="cuda").bfloat16().requires_grad_()
    q2, k2 = rope.apply_rope(q * 1, k * 1, rot, None)
    gq, gk = torch.randn_like(q2), torch.randn_like(k2)
    ((q2 * gq).sum() + (k2 * gk).sum()).backward()
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    pos = torch.arange(S, device="cuda")
    q3, k3 = rot(qr, pos), rot(kr, pos)
    ((q3 * gq.float()).sum() + (k3 * gk.float()).sum()).backward()
    _close(q2, q3)
    _close(k2, k3)
    _close(q.grad, qr.grad)
    _close(k.grad, kr.grad)
    # explicit per-token positions
    pos2 = torch.randint(0, 500, (B, S), device="cuda")
    q4, _ = rope.apply_rope(q.detach() * 1, k.detach() * 1, rot, pos2)
    _close(q4, rot(q.detach().float(), pos2))
    lib.check_status()


@pytest.mark.parametrize("act", [ActivationFunctionEnum.silu, ActivationFunctionEnum.gelu_new, ActivationFunctionEnum.gelu])
def test_glu(act):
    torch.manual_seed(3)
    gu = torch.randn(50, 2 * 264, device="cuda").bfloat16().requires_grad_()
    g, u = gu[:, :264], gu[:, 264:]
    out = glu.gated_activation(g, u, act)
    go = torch.randn_like(out)
    out.backward(go)
    gur = gu.detach().float().requires_grad_()
    outr = act.to_fn()(gur[:, :264]) * gur[:, 264:]
    outr.backward(go.float())
    _close(out, outr)
    _close(gu.grad, gur.grad)


@pytest.mark.parametrize("V,cap,z", [(1000, None, None), (32000, None, 1e-4), (50264, 30.0, None)])
def test_fused_linear_cross_entropy(V, cap, z):
    torch.manual_seed(4)
    T, E = 300, 256
    x = (0.5 * torch.randn(T, E, device="cuda")).bfloat16().requires_grad_()
    w = (0.05 * torch.randn(V, E, device="cuda")).bfloat16().requires_grad_()
    tgt = torch.randint(0, V, (T,), device="cuda")
    loss, lse = CE.fused_linear_cross_entropy(x, w, tgt, soft_cap=cap, z_weight=z, chunk_rows=128)
    gl = torch.rand(T, device="cuda")
    (loss * gl).sum().backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    logits = xr @ wr.t()
    if cap:
        logits = torch.tanh(logits / cap) * cap
    lz = torch.logsumexp(logits, -1)
    lr = lz - logits.gather(-1, tgt[:, None]).squeeze(-1)
    if z:
        lr = lr + z * lz * lz
    (lr * gl).sum().backward()
    _close(loss, lr, 1e-2)
    _close(x.grad, xr.grad, 3e-2)
    _close(w.grad, wr.grad, 3e-2)
    lib.check_status()


def test_adamw_and_sumsq():
    torch.manual_seed(5)
    n = 100_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    sq = optim_kernels.sumsq(g)
    assert abs(sq.item() - (g.double() ** 2).sum().item()) / sq.item() < 1e-5
    coef = torch.ones(1, device="cuda")
    nrm = torch.zeros(1, device="cuda")
    optim_kernels.clip_coef(sq, 1.0, coef, nrm)
    assert abs(nrm.item() - g.norm().item()) / nrm.item() < 1e-5
    p0 = p.clone()
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    optim_kernels.adamw(p, m, v, g, pb, lr, b1, b2, eps, wd, 1 - b1, 1 - b2, coef, 1.0, False)
    gs = g * coef
    mr = (1 - b1) * gs
    vr = (1 - b2) * gs * gs
    u = (mr / (1 - b1)) / ((vr / (1 - b2)).sqrt() + eps) + wd * p0
    pr = p0 - lr * u
    _close(p, pr, 1e-5)
    _close(pb, pr, 1e-2)
    _close(m, mr, 1e-5)
