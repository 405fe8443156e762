"""Hyena operator: the FFT long convolution against a direct causal convolution, causality of the whole operator, and a
training step of the GPT-2/Hyena model."""
import torch

from levanter_b200.models.gpt2_hyena import Gpt2HyenaConfig
from levanter_b200.models.hyena import HyenaConfig, HyenaOperator, fft_conv
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss


def test_fft_conv_matches_direct_causal_convolution():
    torch.manual_seed(0)
    u = torch.randn(2, 3, 17, 5)
    k = torch.randn(17, 5)
    want = torch.zeros_like(u)
    for t in range(17):
        for s in range(t + 1):
            want[..., t, :] += u[..., s, :] * k[t - s]
    torch.testing.assert_close(fft_conv(u, k), want, atol=1e-4, rtol=1e-4)


def test_operator_is_causal_and_blockwise():
    torch.manual_seed(0)
    cfg = HyenaConfig(seq_len=32, hidden_dim=16, num_heads=2, order=3, filter_order=8, num_blocks=2)
    op = HyenaOperator(cfg).eval()
    x = torch.randn(1, 32, 16)
    y = op(x)
    x2 = x.clone()
    x2[:, 20:] += 1.0
    y2 = op(x2)
    torch.testing.assert_close(y[:, :20], y2[:, :20])  # the future does not leak
    assert not torch.allclose(y[:, 20:], y2[:, 20:])
    # the long filter does not cross a block boundary: only the 3-tap input filter reaches two positions into block two
    x3 = x.clone()
    x3[:, :10] += 1.0
    y3 = op(x3)
    torch.testing.assert_close(y[:, 18:], y3[:, 18:])


def test_gpt2_hyena_trains():
    cfg = Gpt2HyenaConfig(num_layers=2, hyena=HyenaConfig(seq_len=32, hidden_dim=32, filter_order=8), gradient_checkpointing=False)
    model = cfg.build(64, seed=0)
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    tokens = torch.randint(0, 64, (4, 32), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
    ex = LmExample.causal(tokens)
    losses = []
    for _ in range(8):
        loss = compute_next_token_loss(model, ex)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
