"""Grouped tcgen05 GEMMs of the expert MLP (forward, input gradient, weight gradient) against fp32 PyTorch per expert."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(T, k, E, H, M, seed=0, skew=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(T, H, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_()
    w1 = (torch.randn(E, M, H, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_()
    w3 = (torch.randn(E, M, H, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_()
    w2 = (torch.randn(E, H, M, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_()
    if skew:  # one expert gets nothing, one gets most
        idx = torch.zeros(T, k, dtype=torch.long, device="cuda")
        idx[:, 1] = 1 + (torch.arange(T, device="cuda") % max(E - 2, 1))
    else:
        idx = torch.stack([torch.randperm(E, device="cuda", generator=g)[:k] for _ in range(T)])
    return x, w1, w3, w2, idx


@pytest.mark.parametrize("T,k,E,H,M,skew", [(300, 2, 4, 256, 512, False), (1000, 2, 8, 512, 1024, False), (200, 2, 4, 256, 384, True), (5, 1, 3, 128, 128, False)])
def test_grouped_mlp_kernel_matches_fp32(T, k, E, H, M, skew):
    from levanter_b200.ops import lib
    from levanter_b200.ops.moe import grouped_mlp_padded
    from levanter_b200.utils.activation import ActivationFunctionEnum

    x, w1, w3, w2, idx = _case(T, k, E, H, M, skew=skew)
    n0 = lib.launch_count
    out = grouped_mlp_padded(x, idx, w1, w3, w2, ActivationFunctionEnum.silu)
    gout = (torch.randn(out.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)) * 0.1).bfloat16()
    out.backward(gout)
    torch.cuda.synchronize()
    lib.check_status()
    assert lib.launch_count - n0 >= 9  # three grouped GEMMs forward, six backward
    got = [out.detach().float()] + [t.grad.float() for t in (x, w1, w3, w2)]
    # fp32 oracle, expert by expert
    xf, a, b, c = (t.detach().float().requires_grad_() for t in (x, w1, w3, w2))
    rows = []
    for t in range(T):
        for j in range(k):
            e = int(idx[t, j])
            h = torch.nn.functional.silu(xf[t] @ a[e].t()) * (xf[t] @ b[e].t())
            rows.append(h @ c[e].t())
    ref = torch.stack(rows)
    ref.backward(gout.float())
    want = [ref.detach(), xf.grad, a.grad, b.grad, c.grad]
    for name, u, v in zip(("out", "dx", "dw1", "dw3", "dw2"), got, want):
        err = (u - v).abs().max().item() / (v.abs().max().item() + 1e-6)
        assert err < 3e-2, (name, err)


def test_mixtral_block_uses_the_grouped_path_and_matches_cpu():
    from levanter_b200.models.mixtral import MixtralConfig

    cfg = MixtralConfig(seq_len=64, hidden_dim=256, intermediate_dim=512, num_layers=1, num_heads=2, num_kv_heads=1, n_routed_experts=4,
                        num_experts_per_tok=2, gradient_checkpointing=False)
    m = cfg.build(100, seed=0)
    ids = torch.randint(0, 100, (2, 64), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m.activations(ids)
        ref = ref[0] if isinstance(ref, tuple) else ref
        mg = m.to("cuda").to(torch.bfloat16)
        got = mg.activations(ids.cuda())
        got = got[0] if isinstance(got, tuple) else got
    # per token: bf16 rounding in attention can flip a near-tie of the router for an odd token, which changes that token's
    # output wholesale; every other token must agree closely
    tok_err = (got.float().cpu() - ref).abs().amax(-1) / ref.abs().max().item()
    assert tok_err.median().item() < 1e-2, tok_err.median().item()
    assert (tok_err > 5e-2).float().mean().item() <= 0.05, tok_err


@pytest.mark.parametrize("T,E,k", [(1000, 8, 2), (77, 16, 4), (5, 3, 1)])
def test_routing_kernel_matches_pytorch_forward_and_backward(T, E, k):
    from levanter_b200.ops import lib
    from levanter_b200.ops.moe import moe_route, moe_route_reference

    g = torch.Generator(device="cuda").manual_seed(0)
    z = (torch.randn(T, E, device="cuda", generator=g) * 2).requires_grad_()
    w, idx, counts, psum, lse = moe_route(z, k)
    zr = z.detach().clone().requires_grad_()
    wr, idxr, countsr, psumr, lser = moe_route_reference(zr, k)
    assert torch.equal(idx, idxr) and torch.equal(counts.long(), countsr.long())
    assert torch.allclose(w, wr, atol=1e-6) and torch.allclose(psum, psumr, atol=1e-4) and torch.allclose(lse, lser, atol=1e-5)
    gw = torch.randn(T, k, device="cuda", generator=g)
    gp = torch.randn(E, device="cuda", generator=g)
    gl = torch.randn(T, device="cuda", generator=g)
    ((w * gw).sum() + (psum * gp).sum() + (lse * gl).sum()).backward()
    ((wr * gw).sum() + (psumr * gp).sum() + (lser * gl).sum()).backward()
    torch.cuda.synchronize()
    lib.check_status()
    assert torch.allclose(z.grad, zr.grad, atol=2e-5, rtol=1e-4)
    # the probability sums are reduced in a fixed order: bitwise repeatable
    w2, _, _, psum2, _ = moe_route(z.detach(), k)
    assert torch.equal(psum2, psum.detach())
