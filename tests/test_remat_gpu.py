"""Checkpointed layers on the GPU keep the flash-attention outputs of the first pass: the gradients equal those of plain
recomputation bit for bit, and the forward kernel runs once per layer instead of twice."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_keep_attention_checkpointing_same_gradients_fewer_launches(monkeypatch):
    from levanter_b200.layers.attention import AttentionMask
    from levanter_b200.models.llama import LlamaConfig
    from levanter_b200.ops import _flash_impl, lib

    calls = {"fwd": 0}
    real_fwd2, real_fwd = _flash_impl._fwd2, _flash_impl._fwd

    def counting(getter):
        def get():
            f = getter()

            def wrapped(*a):
                calls["fwd"] += 1
                return f(*a)

            return wrapped

        return get

    monkeypatch.setattr(_flash_impl, "_fwd2", counting(real_fwd2))
    monkeypatch.setattr(_flash_impl, "_fwd", counting(real_fwd))
    out = {}
    for gc in ("full", True):
        cfg = LlamaConfig(seq_len=256, hidden_dim=256, intermediate_dim=512, num_layers=3, num_heads=2, num_kv_heads=1, gradient_checkpointing=gc)
        m = cfg.build(300, seed=0, device="cuda").to(torch.bfloat16).train()
        ids = torch.randint(0, 300, (2, 256), generator=torch.Generator().manual_seed(3)).cuda()
        calls["fwd"] = 0
        h = m.activations(ids, AttentionMask.causal())
        h.float().square().mean().backward()
        torch.cuda.synchronize()
        lib.check_status()
        out[gc] = ({n: q.grad.clone() for n, q in m.named_parameters() if q.grad is not None}, calls["fwd"])
    assert out["full"][1] == 6 and out[True][1] == 3  # 3 layers: forward + recomputation, against forward only
    for n, g in out["full"][0].items():
        assert torch.equal(g, out[True][0][n]), n
