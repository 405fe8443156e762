"""Next-token losses: vocabulary-blocked cross-entropy against the materialised one (value and gradients), z-loss, soft cap,
reductions and masks (modelled on the reference's tests/test_loss.py)."""
import pytest
import torch
import torch.nn.functional as F

from levanter_b200.models.loss import (cross_entropy_and_logsumexp_penalty, fused_cross_entropy_loss_and_logsumexp_penalty,
                                       maybe_fused_next_token_loss, next_token_loss)


def _setup(B=2, S=7, E=16, V=37, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, S, E, generator=g, requires_grad=True), (torch.randn(V, E, generator=g) * 0.3).requires_grad_(),
            torch.randint(0, V, (B, S), generator=g))


@pytest.mark.parametrize("block", [5, 16, 37, 64])
@pytest.mark.parametrize("z", [None, 1e-2])
def test_blockwise_equals_full(block, z):
    x, w, ids = _setup()
    full = maybe_fused_next_token_loss(x, w, ids, logsumexp_weight=z, block_size=None)
    gx, gw = torch.autograd.grad(full, (x, w))
    blk = maybe_fused_next_token_loss(x, w, ids, logsumexp_weight=z, block_size=block)
    bx, bw = torch.autograd.grad(blk, (x, w))
    assert torch.allclose(full, blk, atol=1e-5) and torch.allclose(gx, bx, atol=1e-5) and torch.allclose(gw, bw, atol=1e-5)


def test_matches_torch_cross_entropy_with_mask_and_last_position_dropped():
    x, w, ids = _setup()
    mask = torch.ones(2, 7)
    mask[0, 2] = 0
    loss = maybe_fused_next_token_loss(x, w, ids, loss_mask=mask)
    logits = x @ w.t()
    per = F.cross_entropy(logits[:, :-1].reshape(-1, 37), ids[:, 1:].reshape(-1), reduction="none").view(2, 6)
    m = mask[:, :-1]
    assert torch.allclose(loss, (per * m).sum() / m.sum(), atol=1e-5)
    assert torch.allclose(next_token_loss(logits, ids, loss_mask=mask), loss, atol=1e-5)


def test_reductions():
    x, w, ids = _setup()
    none = maybe_fused_next_token_loss(x, w, ids, reduction=None)
    assert none.shape == (2, 7) and float(none[:, -1].abs().sum()) == 0.0
    assert torch.allclose(maybe_fused_next_token_loss(x, w, ids, reduction="sum"), none.sum(), atol=1e-5)
    per_row = maybe_fused_next_token_loss(x, w, ids, reduction="mean", reduction_dim=-1)
    assert per_row.shape == (2,) and torch.allclose(per_row, none.sum(-1) / 6, atol=1e-5)


def test_z_loss_and_soft_cap_formulas():
    logits = torch.randn(3, 5, 11)
    tgt = torch.randint(0, 11, (3, 5))
    loss, lse = cross_entropy_and_logsumexp_penalty(logits, tgt, logsumexp_weight=0.1)
    ref_lse = torch.logsumexp(logits, -1)
    ref = F.cross_entropy(logits.reshape(-1, 11), tgt.reshape(-1), reduction="none").view(3, 5) + 0.1 * ref_lse ** 2
    assert torch.allclose(loss, ref, atol=1e-5) and torch.allclose(lse, ref_lse, atol=1e-5)
    capped, _ = cross_entropy_and_logsumexp_penalty(logits * 10, tgt, logit_soft_cap=5.0)
    ref = F.cross_entropy((5.0 * torch.tanh(logits * 10 / 5.0)).reshape(-1, 11), tgt.reshape(-1), reduction="none").view(3, 5)
    assert torch.allclose(capped, ref, atol=1e-5)
    x, w, ids = _setup()
    a = fused_cross_entropy_loss_and_logsumexp_penalty(x, w, torch.roll(ids, -1, -1), block_size=8, logsumexp_weight=None, dtype=torch.float32,
                                                       logit_soft_cap=3.0)
    b, _ = cross_entropy_and_logsumexp_penalty(x @ w.t(), torch.roll(ids, -1, -1), logit_soft_cap=3.0)
    assert torch.allclose(a, b, atol=1e-5)
