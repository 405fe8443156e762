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
