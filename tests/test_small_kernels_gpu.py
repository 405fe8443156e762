"""Embedding gather / scatter-add, counter-based dropout and one-pass fp8 quantisation against PyTorch / NumPy statements of
the same operations."""
import numpy as np
import pytest
import torch

from levanter_b200.ops import lib

pytestmark = pytest.mark.gpu


def test_embedding_forward_and_deterministic_backward():
    from levanter_b200.ops.embedding import embedding

    torch.manual_seed(0)
    V, D, T = 1000, 256, 4096
    w = (torch.randn(V, D, device="cuda") * 0.1).bfloat16().requires_grad_()
    ids = torch.randint(0, 50, (4, T // 4), device="cuda")  # few distinct ids: long runs of repeats
    ids[0, :100] = torch.randint(0, V, (100,), device="cuda")
    y = embedding(ids, w)
    assert torch.equal(y, torch.nn.functional.embedding(ids, w))
    dy = (torch.randn(4, T // 4, D, device="cuda")).bfloat16()
    y.backward(dy)
    ref = torch.zeros(V, D, device="cuda", dtype=torch.float32).index_add_(0, ids.reshape(-1), dy.reshape(-1, D).float())
    assert torch.allclose(w.grad.float(), ref, atol=2e-2, rtol=2e-2)  # the gradient is rounded to bf16 on this path
    # into an fp32 accumulator: tight, and bitwise reproducible
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(V, D, device="cuda", dtype=torch.float32)
    embedding(ids, w2).backward(dy)
    first = w2.main_grad.clone()
    assert torch.allclose(first, ref, atol=1e-4, rtol=1e-5)
    w2.main_grad.zero_()
    embedding(ids, w2).backward(dy)
    assert torch.equal(first, w2.main_grad)
    torch.cuda.synchronize()
    lib.check_status()


def test_dropout_matches_the_numpy_generator_and_regenerates_its_mask():
    from levanter_b200.ops.dropout import dropout, philox_keep_mask

    torch.manual_seed(1)
    n, p, seed = 8 * 1000, 0.25, 0x1234_5678_9ABC
    x = torch.randn(n, device="cuda").bfloat16().requires_grad_()
    res = torch.randn(n, device="cuda").bfloat16()
    y = dropout(x, p, training=True, residual=res, seed=seed)
    keep = torch.from_numpy(philox_keep_mask(n, p, seed)).cuda()
    want = (res.float() + torch.where(keep, x.detach().float() / (1 - p), torch.zeros(()).cuda())).bfloat16()
    assert torch.equal(y, want)
    assert abs(keep.float().mean().item() - (1 - p)) < 0.02
    dy = torch.randn(n, device="cuda").bfloat16()
    y.backward(dy)
    assert torch.equal(x.grad, torch.where(keep, dy.float() / (1 - p), torch.zeros(()).cuda()).bfloat16())
    # eval mode and p = 0 are the identity (plus the residual)
    assert torch.equal(dropout(x.detach(), p, training=False), x.detach())


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("rows,cols", [(256, 512), (300, 200), (64, 72)])
def test_fp8_quantize_one_pass(fmt, rows, cols):
    from levanter_b200.ops.fp8 import E4M3, E5M2, quantize, quantize_with_history

    torch.manual_seed(2)
    dt = E4M3 if fmt == "e4m3" else E5M2
    x = (torch.randn(rows, cols, device="cuda") * 3).bfloat16()
    hist = torch.zeros(4, device="cuda")
    q, qt, inv = quantize_with_history(x, dt, hist, False, True)  # first use: the scale comes from the tensor itself
    amax = x.abs().amax().float()
    q_ref, inv_ref = quantize(x, dt, amax)
    assert torch.allclose(inv, inv_ref)
    # the kernel rounds x * scale to the nearest fp8 value as PyTorch's cast does
    assert (q.float() - q_ref.float()).abs().max() <= 0, (q.float() - q_ref.float()).abs().max()
    assert torch.equal(qt.view(torch.uint8), q.view(torch.uint8).t().contiguous())
    assert hist[0].item() == pytest.approx(amax.item()) and hist[1:].abs().sum().item() == 0
    # second use: the scale is the history's maximum, a larger tensor saturates instead of being rescanned
    x2 = x * 4
    q2, _, inv2 = quantize_with_history(x2, dt, hist, True, False)
    assert torch.allclose(inv2, inv_ref)
    fmax = 448.0 if fmt == "e4m3" else 57344.0
    assert q2.float().abs().max().item() == fmax
    assert hist[0].item() == pytest.approx(x2.abs().amax().item()) and hist[1].item() == pytest.approx(amax.item())


def test_fp8_linear_trains_with_delayed_scaling():
    from levanter_b200.nn import Linear
    from levanter_b200.ops.fp8 import Fp8Linear

    torch.manual_seed(3)
    lin = Linear(256, 384, device="cuda", dtype=torch.bfloat16)
    f8 = Fp8Linear.from_linear(lin, amax_history_length=4)
    x = torch.randn(512, 256, device="cuda").bfloat16().requires_grad_()
    for step in range(3):
        y = f8(x)
        ref = torch.nn.functional.linear(x.float(), lin.weight.float())
        assert ((y.float() - ref).abs().max() / ref.abs().max()).item() < 0.08
        g = torch.randn_like(y)
        lin.weight.grad = None
        x.grad = None
        y.backward(g)
        dref = g.float() @ lin.weight.float()
        assert ((x.grad.float() - dref).abs().max() / dref.abs().max()).item() < 0.12
        wref = g.float().t() @ x.detach().float()
        assert ((lin.weight.grad.float() - wref).abs().max() / wref.abs().max()).item() < 0.12
    torch.cuda.synchronize()
    lib.check_status()


@pytest.mark.parametrize("L,C", [(256, 48), (1024, 96), (2048, 40)])
def test_long_conv_matches_fft_convolution(L, C):
    from levanter_b200.ops.long_conv import fft_conv_reference, long_conv

    torch.manual_seed(4)
    u = torch.randn(2, 3, L, C, device="cuda").bfloat16().requires_grad_()
    k = (torch.randn(L, C, device="cuda") * torch.exp(-torch.arange(L, device="cuda").float() / 64)[:, None]).bfloat16().requires_grad_()
    bias = torch.randn(C, device="cuda").requires_grad_()
    y = long_conv(u, k, bias)
    ur, kr, br = u.detach().float().requires_grad_(), k.detach().float().requires_grad_(), bias.detach().clone().requires_grad_()
    yr = fft_conv_reference(ur, kr, br)
    scale = yr.abs().max().item()
    assert (y.float() - yr).abs().max().item() < 2e-2 * scale
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    assert (u.grad.float() - ur.grad).abs().max().item() < 2e-2 * ur.grad.abs().max().item()
    assert (k.grad.float() - kr.grad).abs().max().item() < 2e-2 * kr.grad.abs().max().item()
    assert torch.allclose(bias.grad, br.grad, rtol=1e-3, atol=1e-2)
    torch.cuda.synchronize()
    lib.check_status()


def test_lora_branch_through_the_gemm_epilogue():
    from levanter_b200.lora import LoraLinear
    from levanter_b200.nn import Linear

    torch.manual_seed(5)
    base = Linear(256, 384, device="cuda", dtype=torch.bfloat16)
    ll = LoraLinear.init(base, r=16, alpha=32.0, dropout_prob=0.0)
    with torch.no_grad():
        ll.lora.lora_B.weight.copy_(torch.randn_like(ll.lora.lora_B.weight) * 0.1)
    x = torch.randn(300, 256, device="cuda").bfloat16().requires_grad_()
    y = ll(x)
    ref = x.float() @ base.weight.float().t() + ll.lora.scale * ((x.float() @ ll.lora.lora_A.weight.float().t()) @ ll.lora.lora_B.weight.float().t())
    assert (y.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    A, B = ll.lora.lora_A.weight.detach().float().requires_grad_(), ll.lora.lora_B.weight.detach().float().requires_grad_()
    (xr @ base.weight.float().t() + ll.lora.scale * ((xr @ A.t()) @ B.t())).backward(g.float())
    for got, want in ((x.grad, xr.grad), (ll.lora.lora_A.weight.grad, A.grad), (ll.lora.lora_B.weight.grad, B.grad)):
        assert (got.float() - want).abs().max().item() < 3e-2 * want.abs().max().item()


def test_sophia_fused_update_matches_the_reference_statement():
    from levanter_b200.optim.sophia import _fused_update

    torch.manual_seed(6)
    n = 100_003
    g, mu, h, p = (torch.randn(n, device="cuda") for _ in range(4))
    h = h.abs() * 100 + 10  # gamma * h around 1: a mix of clipped and unclipped entries
    mu0 = mu.clone()
    stats = torch.zeros(4, device="cuda")
    b1, count, gamma, eps, rho = 0.96, 3, 0.01, 1e-12, 1.0
    u = _fused_update(g, mu, h, p, b1, 1 - b1 ** count, gamma, eps, rho, stats)
    m_ref = b1 * mu0 + (1 - b1) * g
    mh = m_ref / (1 - b1 ** count)
    raw = mh / torch.clamp(gamma * h, min=eps)
    assert torch.allclose(mu, m_ref, rtol=1e-6, atol=1e-7)
    err = (u - raw.clamp(-rho, rho)).abs().max().item()
    assert err < 1e-5, err  # the kernel divides with the fast-math reciprocal
    want = torch.stack([(mh ** 2).sum(), (h ** 2).sum(), (p ** 2).sum(), (raw.abs() < rho).float().sum()])
    assert torch.allclose(stats[:3], want[:3], rtol=1e-3)
    assert abs(stats[3].item() - want[3].item()) <= 5  # entries within rounding of the clipping threshold may count either way


@pytest.mark.parametrize("stride", [1, 2])
def test_three_tap_convolution_as_a_gemm_matches_conv1d(stride):
    """Whisper's stem convolutions: the im2col matrix is an overlapping-row view of the padded channels-last input."""
    import torch.nn.functional as F
    from levanter_b200.ops import conv1d as C

    torch.manual_seed(0)
    B, Ci, Co, T = 3, 80, 384, 3000 if stride == 1 else 1500
    x = torch.randn(B, Ci, T, device="cuda").bfloat16()
    w = (torch.randn(Co, Ci, 3, device="cuda") * 0.05).bfloat16().requires_grad_()
    b = torch.randn(Co, device="cuda").bfloat16().requires_grad_()
    xp = C.pad_channels_last(x).requires_grad_()
    assert C.kernel_ok(xp, w, stride)
    y = C.conv1d_k3(xp, w, b, stride)
    xr, wr, br = x.float().requires_grad_(), w.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    ref = F.conv1d(xr, wr, br, stride=stride, padding=1).transpose(1, 2)
    assert y.shape == ref.shape
    assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    g = torch.randn_like(ref)
    y.backward(g.bfloat16())
    ref.backward(g)
    torch.cuda.synchronize()
    lib.check_status()
    assert (w.grad.float() - wr.grad).abs().max() <= 2e-2 * wr.grad.abs().max()
    assert (b.grad.float() - br.grad).abs().max() <= 2e-2 * br.grad.abs().max()
    dx = xp.grad[:, 1 : T + 1].float().transpose(1, 2)
    assert (dx - xr.grad).abs().max() <= 2e-2 * xr.grad.abs().max()
    assert float(xp.grad[:, 0].abs().max()) < 1e30  # padding rows receive a finite (ignored) gradient


def test_newton_schulz_with_the_polynomial_in_the_gemm_epilogues_matches_fp32():
    from levanter_b200.ops.newton_schulz import zeropower_via_newtonschulz5

    torch.manual_seed(0)
    for shape in [(256, 512), (1024, 256), (384, 384)]:
        g = torch.randn(*shape, device="cuda")
        got = zeropower_via_newtonschulz5(g)
        with lib.reference_ops():
            want = zeropower_via_newtonschulz5(g)
        torch.cuda.synchronize()
        lib.check_status()
        assert (got - want).abs().max() <= 0.05 * want.abs().max()
        # no singular value overshoots the quintic's band (the smallest ones of a square random matrix stay small after 5 steps)
        assert torch.linalg.svdvals(got.float()).max() < 1.3
