"""Layer checkpointing that keeps attention outputs: same gradients as no checkpointing, also with dropout and non-tensor arguments."""
import pytest
import torch
import torch.nn as nn

from levanter_b200.layers.attention import AttentionMask
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.utils.remat import ScanCheckpointPolicy, checkpoint_layer, keeps_attention, should_recompute


class _Block(nn.Module):
    def __init__(self, p=0.0):
        super().__init__()
        self.a, self.b, self.drop = nn.Linear(8, 16), nn.Linear(16, 8), nn.Dropout(p)

    def forward(self, x, scale=None, flag=None):
        h = self.drop(torch.tanh(self.a(x)))
        return x + self.b(h) * (1.0 if scale is None else scale)


@pytest.mark.parametrize("p", [0.0, 0.5])
def test_same_gradients_as_plain_autograd(p):
    torch.manual_seed(0)
    blk = _Block(p)
    x = torch.randn(4, 8, requires_grad=True)
    torch.manual_seed(1)
    y = blk(blk(x, 2.0), None, "unused")
    y.square().sum().backward()
    ref = [x.grad.clone()] + [q.grad.clone() for q in blk.parameters()]
    x.grad = None
    blk.zero_grad()
    torch.manual_seed(1)
    y2 = checkpoint_layer(blk, checkpoint_layer(blk, x, 2.0), None, "unused")
    assert torch.allclose(y, y2)
    y2.square().sum().backward()
    got = [x.grad] + [q.grad for q in blk.parameters()]
    for a, b in zip(ref, got):
        assert torch.allclose(a, b, atol=1e-6)


def test_llama_with_and_without_checkpointing_agree():
    torch.manual_seed(0)
    grads = {}
    for gc in (False, True, "full"):
        cfg = LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, gradient_checkpointing=gc)
        m = cfg.build(50, seed=0).train()
        ids = torch.randint(0, 50, (2, 16), generator=torch.Generator().manual_seed(3))
        h = m.activations(ids, AttentionMask.causal())
        h.square().mean().backward()
        grads[gc] = {n: q.grad.clone() for n, q in m.named_parameters() if q.grad is not None}
        assert len(grads[gc]) > 10
    for n in grads[False]:
        assert torch.allclose(grads[False][n], grads[True][n], atol=1e-6), n
        assert torch.allclose(grads[False][n], grads["full"][n], atol=1e-6), n


def test_policy_flags():
    assert should_recompute(True) and keeps_attention(True)
    assert should_recompute("full") and not keeps_attention("full")
    assert not should_recompute(False)
    assert not keeps_attention(ScanCheckpointPolicy(recompute_attention=True))


def test_no_grad_pass_runs_directly():
    blk = _Block()
    with torch.no_grad():
        y = checkpoint_layer(blk, torch.randn(2, 8))
    assert not y.requires_grad


def test_input_without_gradient_but_trainable_parameters_inside():
    """Frozen embeddings (LoRA): the layer input does not require gradients, the parameters inside the layer do."""
    blk = _Block()
    x = torch.randn(4, 8)  # requires_grad False
    y = checkpoint_layer(blk, x)
    assert y.requires_grad
    y.sum().backward()
    assert blk.a.weight.grad is not None
