"""Gated delta rule: the chunked scan against the step-by-step recurrence (values, final state, gradients) and a training
step of the language model."""
import pytest
import torch

from levanter_b200.models.gated_deltanet import GatedDeltaNetConfig, delta_rule_chunked_scan, delta_rule_recurrent
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss


def _inputs(B=2, H=3, L=70, dk=16, dv=24, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, H, L, dk, generator=g), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(B, H, L, dk, generator=g), dim=-1)
    v = torch.randn(B, H, L, dv, generator=g)
    gate = -torch.rand(B, H, L, generator=g) * 0.5
    beta = torch.rand(B, H, L, generator=g)
    return q, k, v, gate, beta


@pytest.mark.parametrize("chunk", [16, 32, 64])
def test_chunked_scan_matches_recurrence(chunk):
    q, k, v, g, beta = _inputs()
    o_ref, s_ref = delta_rule_recurrent(q, k, v, g, beta)
    o, s = delta_rule_chunked_scan(q, k, v, g, beta, chunk_size=chunk)
    torch.testing.assert_close(o, o_ref, atol=2e-4, rtol=1e-3)
    torch.testing.assert_close(s, s_ref, atol=2e-4, rtol=1e-3)


def test_chunked_scan_carries_state_and_gradients():
    q, k, v, g, beta = _inputs(L=48)
    o_full, _ = delta_rule_chunked_scan(q, k, v, g, beta, chunk_size=16)
    o1, s1 = delta_rule_chunked_scan(q[:, :, :20], k[:, :, :20], v[:, :, :20], g[:, :, :20], beta[:, :, :20], chunk_size=16)
    o2, _ = delta_rule_chunked_scan(q[:, :, 20:], k[:, :, 20:], v[:, :, 20:], g[:, :, 20:], beta[:, :, 20:], chunk_size=16, initial_state=s1)
    torch.testing.assert_close(torch.cat([o1, o2], dim=2), o_full, atol=2e-4, rtol=1e-3)
    v1 = v.clone().requires_grad_()
    v2 = v.clone().requires_grad_()
    delta_rule_chunked_scan(q, k, v1, g, beta, chunk_size=16)[0].square().sum().backward()
    delta_rule_recurrent(q, k, v2, g, beta)[0].square().sum().backward()
    torch.testing.assert_close(v1.grad, v2.grad, atol=5e-4, rtol=1e-3)


def test_model_trains_and_is_causal():
    cfg = GatedDeltaNetConfig(seq_len=32, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, head_k_dim=8, head_v_dim=16,
                              chunk_size=8, gradient_checkpointing=False)
    model = cfg.build(64, seed=0)
    tokens = torch.randint(0, 64, (3, 32), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
    with torch.no_grad():
        a = model.activations(tokens)
        t2 = tokens.clone()
        t2[:, 20:] = (t2[:, 20:] + 1) % 64
        b = model.activations(t2)
    torch.testing.assert_close(a[:, :20], b[:, :20])
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    ex = LmExample.causal(tokens)
    losses = []
    for _ in range(8):
        loss = compute_next_token_loss(model, ex)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
