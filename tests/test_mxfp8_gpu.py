"""Block-scaled fp8 on a B200: the quantiser against its PyTorch statement, the tcgen05 block-scaled GEMM against the fp32
product of the de-quantised operands, and a Linear layer's three products against the fp32 layer."""
import pytest
import torch

from levanter_b200.ops import lib

pytestmark = pytest.mark.gpu
if not (torch.cuda.is_available() and lib.available()):
    pytest.skip("needs a CUDA device and the native library", allow_module_level=True)

from levanter_b200.ops.fp8 import E4M3, E5M2, Fp8Linear, _mx_quantize_rows_reference, _sf_rows, mx_dequantize, mx_gemm, mx_quantize


@pytest.mark.parametrize("R,C", [(256, 384), (200, 160), (1024, 4096)])
@pytest.mark.parametrize("dt", [E4M3, E5M2])
def test_quantiser_matches_the_pytorch_statement(R, C, dt):
    torch.manual_seed(0)
    x = (torch.randn(R, C, device="cuda") * torch.logspace(-2, 2, C, device="cuda")).bfloat16()
    x[3, 32:64] = 0  # an all-zero block
    want_col = R % 32 == 0
    q, sf, qt, sft = mx_quantize(x, dt, True, want_col)
    torch.cuda.synchronize()
    q_ref, sf_ref = _mx_quantize_rows_reference(x, dt)
    assert torch.equal(_sf_rows(sf, R, C), _sf_rows(sf_ref, R, C))
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    blk = x.float().view(R, C // 32, 32).abs().amax(-1, keepdim=True)
    rel = 2.0 ** -4 if dt == E4M3 else 2.0 ** -3
    err = (mx_dequantize(q, sf).view(R, C // 32, 32) - x.float().view(R, C // 32, 32)).abs()
    assert bool((err <= 2 * rel * blk + 1e-30).all())
    if want_col:
        xt = x.float().t().reshape(C, R // 32, 32)
        err_t = (mx_dequantize(qt, sft).view(C, R // 32, 32) - xt).abs()
        assert bool((err_t <= 2 * rel * xt.abs().amax(-1, keepdim=True) + 1e-30).all())
    # rows of the last chunk beyond R carry scale 1
    Rp = -(-R // 128) * 128
    if Rp != R:
        full = sf.view(Rp // 128, -1, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(Rp, -1)
        assert bool((full[R:] == 127).all())


@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 128, 128), (256, 384, 512, 128), (200, 136, 256, 128), (512, 512, 1024, 256),
                                      (300, 520, 384, 256), (4096, 4096, 4096, 0)])
def test_block_scaled_gemm_matches_the_dequantised_product(M, N, K, bn):
    torch.manual_seed(1)
    a = (torch.randn(M, K, device="cuda") * torch.logspace(-1, 1, K, device="cuda")).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    aq, sa, _, _ = mx_quantize(a, E4M3)
    bq, sb, _, _ = mx_quantize(b, E5M2)
    got = mx_gemm(aq, sa, bq, sb, out_dtype=torch.float32, bn=bn)
    torch.cuda.synchronize()
    lib.check_status()
    want = mx_dequantize(aq, sa) @ mx_dequantize(bq, sb).t()
    assert (got - want).abs().max() <= 1e-3 * want.abs().max()
    # and close to the unquantised product, which is what the format is for
    exact = a.float() @ b.float().t()
    assert (got - exact).abs().max() <= 0.08 * exact.abs().max()
    bias = torch.randn(N, device="cuda")
    acc = torch.ones(M, N, device="cuda")
    mx_gemm(aq, sa, bq, sb, out=acc, accumulate=True, bias=bias, bn=bn)
    assert (acc - 1 - bias - want).abs().max() <= 1e-3 * want.abs().max()
    out16 = mx_gemm(aq, sa, bq, sb, bn=bn)
    assert out16.dtype == torch.bfloat16
    assert (out16.float() - want).abs().max() <= 1e-2 * want.abs().max()
    torch.cuda.synchronize()
    lib.check_status()


def test_block_scaled_linear_forward_and_backward():
    from levanter_b200.nn import Linear

    torch.manual_seed(2)
    lin = Linear(512, 384, bias=True).cuda()
    f8 = Fp8Linear.from_linear(lin, block_scaled=True)
    f8.weight.data = f8.weight.data.bfloat16()
    f8.bias.data = f8.bias.data.bfloat16()
    x = torch.randn(2, 128, 512, device="cuda").bfloat16().requires_grad_()
    y = f8(x)
    ref_x = x.detach().float().requires_grad_()
    ref_w = f8.weight.detach().float().requires_grad_()
    ref = torch.nn.functional.linear(ref_x, ref_w, f8.bias.detach().float())
    assert (y.float() - ref).abs().max() <= 0.06 * ref.abs().max()
    g = torch.randn_like(ref)
    y.backward(g.bfloat16())
    ref.backward(g)
    torch.cuda.synchronize()
    lib.check_status()
    assert (x.grad.float() - ref_x.grad).abs().max() <= 0.1 * ref_x.grad.abs().max()
    assert (f8.weight.grad.float() - ref_w.grad).abs().max() <= 0.1 * ref_w.grad.abs().max()
    # fp32 gradient accumulator owned by the engine: the weight-gradient GEMM adds into it
    f8.weight.grad = None
    f8.weight.main_grad = torch.zeros(384, 512, device="cuda")
    f8(x.detach().requires_grad_()).backward(g.bfloat16())
    assert f8.weight.grad is None
    assert (f8.weight.main_grad - ref_w.grad).abs().max() <= 0.1 * ref_w.grad.abs().max()
