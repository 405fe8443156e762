"""fp8 Linear: quantisation round trip, forward/backward against the fp32 layer (CPU path = the kernel's oracle), and
``quantize_linear_layers`` leaving parameter names untouched."""
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
