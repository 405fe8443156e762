"""fp8 Linear: quantisation round trip, forward/backward against the fp32 layer (CPU path = the kernel's oracle), and
``quantize_linear_layers`` leaving parameter names untouched."""
import pytest
import torch

from levanter_b200.nn import Linear
from levanter_b200.ops.fp8 import E4M3, E5M2, Fp8Linear, fp8_gemm, quantize
from levanter_b200.quantization import QuantizationConfig, quantize_linear_layers


def test_quantize_round_trip():
    torch.manual_seed(0)
    x = torch.randn(64, 128) * 3
    for dt, tol in ((E4M3, 0.07), (E5M2, 0.13)):
        q, inv = quantize(x, dt)
        assert q.dtype == dt
        rel = ((q.float() * inv - x).abs().max() / x.abs().max()).item()
        assert rel < tol


def test_fp8_linear_matches_fp32_layer():
    torch.manual_seed(0)
    lin = Linear(128, 64, bias=True)
    f8 = Fp8Linear.from_linear(lin)
    x = torch.randn(4, 32, 128, requires_grad=True)
    y = f8(x)
    y_ref = torch.nn.functional.linear(x, lin.weight, lin.bias)
    assert (y - y_ref).abs().max() / y_ref.abs().max() < 0.08
    g = torch.randn_like(y)
    y.backward(g)
    gx, gw, gb = x.grad.clone(), lin.weight.grad.clone(), lin.bias.grad.clone()
    x.grad = None
    lin.weight.grad = None
    lin.bias.grad = None
    y_ref = torch.nn.functional.linear(x, lin.weight, lin.bias)
    y_ref.backward(g)
    for a, b in ((gx, x.grad), (gw, lin.weight.grad), (gb, lin.bias.grad)):
        assert (a - b).abs().max() / b.abs().max() < 0.15


def test_quantize_linear_layers_keeps_parameter_names():
    from levanter_b200.models.llama import LlamaConfig

    model = LlamaConfig(seq_len=32, hidden_dim=64, intermediate_dim=128, num_layers=1, num_heads=2, num_kv_heads=2).build(100, seed=0)
    names = [n for n, _ in model.named_parameters()]
    model = quantize_linear_layers(model, QuantizationConfig(fp8=True))
    assert [n for n, _ in model.named_parameters()] == names
    assert any(isinstance(m, Fp8Linear) for m in model.modules())
    assert not isinstance(model.lm_head, Fp8Linear) if hasattr(model, "lm_head") and model.lm_head is not None else True
    tokens = torch.randint(0, 100, (2, 32), dtype=torch.int32)
    from levanter_b200.models.lm_model import LmExample, compute_next_token_loss

    loss = compute_next_token_loss(model, LmExample.causal(tokens))
    loss.backward()
    assert torch.isfinite(loss)


def test_block_scale_layout_round_trip():
    from levanter_b200.ops.fp8 import _sf_chunks, _sf_rows

    sf = torch.randint(0, 255, (200, 12), dtype=torch.uint8)  # 200 rows, K = 384
    chunks = _sf_chunks(sf)
    assert chunks.numel() == 2 * 3 * 512
    assert torch.equal(_sf_rows(chunks, 200, 384), sf)
    # row r, block j of the first chunk sits at (r % 32) * 16 + (r / 32) * 4 + j
    assert int(chunks[(37 % 32) * 16 + (37 // 32) * 4 + 2]) == int(sf[37, 2])
    # second K chunk of the second row block
    assert int(chunks[(1 * 3 + 1) * 512 + (5 % 32) * 16 + 0 * 4 + 3]) == int(sf[128 + 5, 4 + 3])


def test_block_scaled_quantisation_error_is_bounded_per_block():
    from levanter_b200.ops.fp8 import E4M3, E5M2, mx_dequantize, mx_quantize

    torch.manual_seed(0)
    x = torch.randn(256, 384) * torch.logspace(-3, 3, 384)  # six orders of magnitude across the columns
    x = x.bfloat16()
    for dt, rel in ((E4M3, 2.0 ** -4), (E5M2, 2.0 ** -3)):
        q, sf, qt, sft = mx_quantize(x, dt, True, True)
        back = mx_dequantize(q, sf)
        blk = x.float().view(256, 12, 32).abs().amax(-1, keepdim=True)
        err = (back.view(256, 12, 32) - x.float().view(256, 12, 32)).abs()
        assert bool((err <= rel * blk + 1e-30).all())  # half an ulp of the block maximum's binade at worst
        back_t = mx_dequantize(qt, sft)
        blk_t = x.float().t().reshape(384, 8, 32).abs().amax(-1, keepdim=True)
        err_t = (back_t.view(384, 8, 32) - x.float().t().reshape(384, 8, 32)).abs()
        assert bool((err_t <= rel * blk_t + 1e-30).all())


def test_block_scaled_fp8_linear_matches_fp32_layer():
    from levanter_b200.ops.fp8 import Fp8Linear

    torch.manual_seed(1)
    lin = Linear(256, 128, bias=True)
    f8 = Fp8Linear.from_linear(lin, block_scaled=True)
    x = torch.randn(2, 64, 256).bfloat16().requires_grad_()
    w16 = lin.weight.detach().bfloat16()
    f8.weight.data = w16.clone()
    f8.bias.data = f8.bias.data.bfloat16()
    y = f8(x)
    ref_x = x.detach().float().requires_grad_()
    ref_w = w16.float().requires_grad_()
    ref = torch.nn.functional.linear(ref_x, ref_w, f8.bias.detach().float())
    assert (y.float() - ref).abs().max() <= 0.06 * ref.abs().max()
    g = torch.randn_like(ref)
    y.backward(g.bfloat16())
    ref.backward(g)
    assert (x.grad.float() - ref_x.grad).abs().max() <= 0.1 * ref_x.grad.abs().max()
    assert (f8.weight.grad.float() - ref_w.grad).abs().max() <= 0.1 * ref_w.grad.abs().max()


def test_quantization_config_selects_block_scaling():
    from levanter_b200.ops.fp8 import Fp8Linear

    model = torch.nn.Sequential(Linear(128, 128), Linear(128, 128))
    quantize_linear_layers(model, QuantizationConfig(fp8=True, scaling="block"))
    assert all(isinstance(m, Fp8Linear) and m.block_scaled for m in model)
    with pytest.raises(ValueError):
        QuantizationConfig(fp8=True, scaling="row")
