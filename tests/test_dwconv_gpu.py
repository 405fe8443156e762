"""Depthwise causal convolution kernels (forward, input and weight/bias gradients) against conv1d in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,L,C,K,dtype,silu,bias", [
    (2, 200, 64, 4, torch.float32, True, False),
    (3, 129, 1024, 4, torch.bfloat16, True, False),
    (2, 64, 48, 3, torch.float32, False, True),
    (1, 70, 2056, 3, torch.bfloat16, False, True),
    (2, 5, 8, 2, torch.float32, True, True),
])
def test_causal_dwconv_matches_conv1d(B, L, C, K, dtype, silu, bias):
    from levanter_b200.ops import lib
    from levanter_b200.ops.dwconv import causal_dwconv, causal_dwconv_reference

    g = torch.Generator(device="cuda").manual_seed(L + C)
    x = torch.randn(B, L, C, device="cuda", generator=g).to(dtype).requires_grad_()
    w = (torch.randn(C, 1, K, device="cuda", generator=g) * 0.5).requires_grad_()
    b = torch.randn(C, device="cuda", generator=g).requires_grad_() if bias else None
    gy = torch.randn(B, L, C, device="cuda", generator=g).to(dtype)

    def run(fn, xin):
        for t in (xin, w, b):
            if t is not None:
                t.grad = None
        y = fn(xin, w, b, silu)
        y.backward(gy.to(y.dtype))
        return y.detach().float(), xin.grad.float().clone(), w.grad.clone(), None if b is None else b.grad.clone()

    x32 = x.detach().float().requires_grad_()
    ref = run(causal_dwconv_reference, x32)  # fp32 throughout
    n0 = lib.launch_count
    got = run(causal_dwconv, x)
    assert lib.launch_count - n0 == 4  # forward; gradient prologue + reduction; input gradient
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for name, a, r in zip(("y", "dx", "dw", "db"), got, ref):
        if r is None:
            continue
        err = (a - r).abs().max().item()
        assert err <= tol * (r.abs().max().item() + 1e-6), (name, err)


def test_gated_deltanet_layer_on_kernels_matches_cpu():
    from levanter_b200.models.gated_deltanet import GatedDeltaNetConfig, GatedDeltaNetLayer

    cfg = GatedDeltaNetConfig(seq_len=256, hidden_dim=128, intermediate_dim=256, num_layers=1, num_heads=2, head_k_dim=64, head_v_dim=64)
    torch.manual_seed(0)
    layer = GatedDeltaNetLayer(cfg)
    x = torch.randn(2, 200, 128)
    gy = torch.randn(2, 200, 128)
    xc = x.clone().requires_grad_()
    layer(xc).backward(gy)
    ref_gx = xc.grad.clone()
    ref_gw = layer.q_conv1d.weight.grad.clone()
    ref_y = layer(x).detach()
    layer.zero_grad()
    layer = layer.cuda()
    xg = x.cuda().requires_grad_()
    y = layer(xg)
    y.backward(gy.cuda())
    torch.testing.assert_close(y.detach().cpu(), ref_y, atol=3e-3, rtol=3e-2)
    torch.testing.assert_close(xg.grad.cpu(), ref_gx, atol=3e-3, rtol=3e-2)
    torch.testing.assert_close(layer.q_conv1d.weight.grad.cpu(), ref_gw, atol=3e-3, rtol=3e-2)
