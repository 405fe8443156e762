"""Padded expert-sorted layout and the grouped expert MLP against the per-expert loop (CPU: reference path)."""
import torch

from levanter_b200.ops.moe import BLOCK, grouped_mlp, grouped_mlp_padded, padded_layout
from levanter_b200.utils.activation import ActivationFunctionEnum


def test_padded_layout_invariants():
    g = torch.Generator().manual_seed(0)
    E = 5
    idx = torch.randint(0, E, (300,), generator=g)
    idx[idx == 3] = 2  # expert 3 gets nothing
    dest, offsets, tile_group, capacity = padded_layout(idx, E)
    counts = torch.bincount(idx, minlength=E)
    assert capacity % BLOCK == 0 and capacity >= int(offsets[-1])
    assert (offsets % BLOCK == 0).all() and offsets[0] == 0
    assert torch.equal((offsets[1:] - offsets[:-1]).long(), (counts + BLOCK - 1) // BLOCK * BLOCK)
    assert len(torch.unique(dest)) == 300  # a permutation into distinct rows
    for e in range(E):
        rows = dest[idx == e]
        assert ((rows >= offsets[e]) & (rows < offsets[e] + counts[e])).all()
        assert torch.equal(rows, torch.sort(rows).values)  # stable: pair order kept inside an expert
    blocks = capacity // BLOCK
    expect = torch.full((blocks,), -1, dtype=torch.int32)
    for e in range(E):
        expect[int(offsets[e]) // BLOCK:int(offsets[e + 1]) // BLOCK] = e
    assert torch.equal(tile_group, expect)


def test_grouped_mlp_padded_matches_per_expert_loop():
    torch.manual_seed(0)
    T, k, E, H, M = 37, 2, 4, 16, 24
    x = torch.randn(T, H, requires_grad=True)
    w1, w3, w2 = (torch.randn(E, M, H) * 0.2).requires_grad_(), (torch.randn(E, M, H) * 0.2).requires_grad_(), (torch.randn(E, H, M) * 0.2).requires_grad_()
    topk_idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    out = grouped_mlp_padded(x, topk_idx, w1, w3, w2, ActivationFunctionEnum.silu)
    out.square().sum().backward()
    got = [out.detach().clone()] + [t.grad.clone() for t in (x, w1, w3, w2)]
    for t in (x, w1, w3, w2):
        t.grad = None
    flat = topk_idx.reshape(-1)
    sort_idx = torch.argsort(flat, stable=True)
    sizes = torch.bincount(flat, minlength=E)
    ref_sorted = grouped_mlp(x.index_select(0, sort_idx // k), sizes, w1, w3, w2, ActivationFunctionEnum.silu)
    inv = torch.empty_like(sort_idx)
    inv[sort_idx] = torch.arange(sort_idx.numel())
    ref = ref_sorted.index_select(0, inv)
    ref.square().sum().backward()
    want = [ref.detach()] + [t.grad for t in (x, w1, w3, w2)]
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)
