"""tcgen05 flash attention (forward and backward) against a PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from levanter_b200.layers.attention import AttentionMask, simple_attention_with_dropout
from levanter_b200.ops import lib
from levanter_b200.ops._flash_impl import flash_attention_cuda

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    scale = b.abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale}"


def _run(B, S, Hq, Hkv, mask, soft_cap=None, seed=0, growing=False, D=128):
    torch.manual_seed(seed)
    q = torch.randn(B, S, Hq, D, device="cuda")
    k = torch.randn(B, S, Hkv, D, device="cuda")
    if growing:
        # logits whose row maximum jumps by far more than the lazy-rescale threshold in later key blocks, and only for
        # some rows of a warp: the running output must be rescaled mid-row, row by row
        k[:, 128:] *= 3.0
        k[:, 256:] *= 2.0
        q[:, 1::3] *= 4.0
    q, k = q.bfloat16().requires_grad_(), k.bfloat16().requires_grad_()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    o = flash_attention_cuda(q, k, v, mask, logits_soft_cap=soft_cap)
    g = torch.randn_like(o)
    o.backward(g)
    torch.cuda.synchronize()
    lib.check_status()
    qr, kr, vr = [t.detach().float().requires_grad_() for t in (q, k, v)]
    orf = simple_attention_with_dropout(qr, kr, vr, mask, attention_dtype=torch.float32, logits_soft_cap=soft_cap)
    orf.backward(g.float())
    _close(o, orf, 2e-2)
    _close(q.grad, qr.grad, 4e-2)
    _close(k.grad, kr.grad, 4e-2)
    _close(v.grad, vr.grad, 4e-2)


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 1, 1), (2, 256, 2, 2), (1, 512, 4, 1), (2, 384, 4, 2)])
def test_causal(B, S, Hq, Hkv):
    _run(B, S, Hq, Hkv, AttentionMask.causal())


@pytest.mark.parametrize("one_tile", [False, True])
def test_running_max_rescale(one_tile):
    from levanter_b200.ops import _flash_impl

    _flash_impl._FORCE_ONE_TILE = one_tile
    try:
        _run(1, 512, 2, 2, AttentionMask.causal(), growing=True)
        _run(2, 768, 2, 1, AttentionMask.causal(), growing=True, seed=1)
    finally:
        _flash_impl._FORCE_ONE_TILE = False


def test_sliding_window():
    _run(1, 640, 2, 2, AttentionMask.causal(sliding_window=200))
    _run(1, 512, 2, 1, AttentionMask.causal(sliding_window=128))


def test_segment_ids():
    S = 384
    seg = torch.zeros(2, S, dtype=torch.int32, device="cuda")
    seg[0, 100:] = 1
    seg[0, 300:] = 2
    seg[1, 129:] = 1
    _run(2, S, 2, 2, AttentionMask.causal().with_segment_ids(seg))


def test_soft_cap():
    _run(1, 256, 2, 2, AttentionMask.causal(), soft_cap=20.0)


def test_one_tile_kernel_matches():
    from levanter_b200.ops import _flash_impl

    _flash_impl._FORCE_ONE_TILE = True
    try:
        _run(2, 512, 2, 2, AttentionMask.causal())
        _run(1, 512, 2, 1, AttentionMask.causal(sliding_window=128))
    finally:
        _flash_impl._FORCE_ONE_TILE = False


def test_long_sequence():
    _run(1, 2048, 2, 2, AttentionMask.causal(), seed=7)


def test_deterministic_forward():
    torch.manual_seed(3)
    q = torch.randn(1, 512, 2, 128, device="cuda").bfloat16()
    k = torch.randn(1, 512, 2, 128, device="cuda").bfloat16()
    v = torch.randn(1, 512, 2, 128, device="cuda").bfloat16()
    a = flash_attention_cuda(q, k, v, AttentionMask.causal()).clone()
    b = flash_attention_cuda(q, k, v, AttentionMask.causal())
    assert torch.equal(a, b)


def test_head_sizes_the_kernel_does_not_cover_take_the_fused_library_path():
    """Head size 64 (GPT-2) on CUDA: same numbers as the plain implementation, with and without grouped-query heads."""
    import math

    from levanter_b200.layers.attention import AttentionMask, dot_product_attention, simple_attention_with_dropout

    torch.manual_seed(0)
    for Hq, Hkv in ((4, 4), (4, 2)):
        q = torch.randn(2, 256, Hq, 64, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(2, 256, Hkv, 64, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(2, 256, Hkv, 64, device="cuda", dtype=torch.bfloat16)
        for mask in (AttentionMask.causal(), None):
            out = dot_product_attention(q, k, v, mask)
            ref = simple_attention_with_dropout(q.float(), k.float(), v.float(), mask)
            assert (out.float() - ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("S", [384, 1024])
def test_packed_sequences_skip_foreign_key_blocks(S):
    """Sorted segment ids (a packed prefill batch, padding at the end): the forward kernels start each query block's key loop
    at its own sequence; the result equals the kernel without the hint and the fp32 reference."""
    torch.manual_seed(11)
    B, H = 1, 4
    q, k, v = (torch.randn(B, S, H, 128, device="cuda").bfloat16() for _ in range(3))
    bounds = sorted(set([0, 100, 130, 300, S - 40, S]))
    seg = torch.full((S,), -1, dtype=torch.int32, device="cuda")
    for i, (a, b) in enumerate(zip(bounds[:-2], bounds[1:-1])):
        seg[a:b] = i
    with torch.no_grad():
        hint = flash_attention_cuda(q, k, v, AttentionMask.causal().with_segment_ids(seg[None], sorted=True))
        plain = flash_attention_cuda(q, k, v, AttentionMask.causal().with_segment_ids(seg[None]))
    torch.cuda.synchronize()
    lib.check_status()
    live = seg >= 0
    assert torch.equal(hint[:, live], plain[:, live])


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 1, 1), (2, 256, 12, 12), (1, 1024, 4, 1), (2, 384, 4, 2)])
def test_head_size_64_causal(B, S, Hq, Hkv):
    """GPT-2's and Whisper's head size on the kernels templated on the head dimension."""
    _run(B, S, Hq, Hkv, AttentionMask.causal(), D=64)


def test_head_size_64_running_max_sliding_window_soft_cap_segments():
    _run(1, 512, 2, 2, AttentionMask.causal(), growing=True, D=64)
    _run(1, 640, 2, 1, AttentionMask.causal(sliding_window=200), D=64)
    _run(1, 256, 2, 2, AttentionMask.causal(), soft_cap=30.0, D=64)
    seg = torch.tensor([[0] * 100 + [1] * 200 + [2] * 84], device="cuda")
    _run(1, 384, 2, 2, AttentionMask.causal().with_segment_ids(seg), D=64)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 2, 2), (2, 512, 4, 2), (1, 384, 6, 6)])
def test_not_causal(B, S, Hq, Hkv, D):
    """Encoder attention: every query sees every key (``mask=None``), or every key of its own segment."""
    _run(B, S, Hq, Hkv, None, D=D)
    seg = torch.arange(S, device="cuda").div(S // 3 + 1, rounding_mode="floor").expand(B, S)
    _run(B, S, Hq, Hkv, AttentionMask(is_causal=False).with_segment_ids(seg), D=D, seed=1)


@pytest.mark.parametrize("D,S,causal", [(64, 1500, False), (64, 200, True), (128, 200, True), (128, 333, False), (64, 77, False)])
def test_lengths_that_are_not_a_multiple_of_256_are_padded_behind_their_own_segment(D, S, causal):
    """Whisper's encoder runs 1500 positions: the rows added to reach 1536 must be invisible to the real ones."""
    _run(1, S, 2, 2, AttentionMask.causal() if causal else None, D=D)


def test_dispatch_takes_head_size_64_and_encoder_masks():
    from levanter_b200.ops import flash_attention as KFA

    q = torch.randn(1, 256, 2, 64, device="cuda").bfloat16()
    assert KFA.supported(q, q, q, None, None, True, None)
    assert KFA.supported(q, q, q, AttentionMask.causal(), None, True, None)
    assert not KFA.supported(q, q[:, :128], q[:, :128], AttentionMask.causal(), None, True, None)  # causal needs equal lengths
    q96 = torch.randn(1, 256, 2, 96, device="cuda").bfloat16()
    assert not KFA.supported(q96, q96, q96, None, None, True, None)


@pytest.mark.parametrize("D,causal", [(64, True), (64, False), (128, False)])
def test_one_tile_forward_kernel_covers_the_same_cases(D, causal):
    from levanter_b200.ops import _flash_impl

    _flash_impl._FORCE_ONE_TILE = True
    try:
        _run(1, 512, 2, 1, AttentionMask.causal() if causal else None, D=D)
    finally:
        _flash_impl._FORCE_ONE_TILE = False


@pytest.mark.parametrize("D,S,causal,Hq,Hkv", [(128, 512, True, 4, 2), (64, 256, True, 2, 2), (128, 200, False, 2, 1)])
def test_sink_logits_join_the_denominator(D, S, causal, Hq, Hkv):
    from levanter_b200.layers.attention import dot_product_attention_with_sink

    torch.manual_seed(0)
    q = torch.randn(2, S, Hq, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(2, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(2, S, Hkv, D, device="cuda").bfloat16().requires_grad_()
    sink = (torch.randn(Hq, device="cuda") * 2).requires_grad_()
    mask = AttentionMask.causal() if causal else None
    o = flash_attention_cuda(q, k, v, mask, sink=sink)
    g = torch.randn_like(o)
    o.backward(g)
    torch.cuda.synchronize()
    lib.check_status()
    qr, kr, vr = [t.detach().float().requires_grad_() for t in (q, k, v)]
    sr = sink.detach().clone().requires_grad_()
    with lib.reference_ops():
        orf = dot_product_attention_with_sink(qr, kr, vr, sr, mask, attention_dtype=torch.float32)
    orf.backward(g.float())
    _close(o, orf, 2e-2)
    _close(q.grad, qr.grad, 4e-2)
    _close(k.grad, kr.grad, 4e-2)
    _close(v.grad, vr.grad, 4e-2)
    _close(sink.grad, sr.grad, 4e-2)
    # the module-level entry point takes the kernel path
    o2 = dot_product_attention_with_sink(q, k, v, sink, mask)
    assert torch.equal(o2, o)


@pytest.mark.parametrize("D,Sq,Sk,Hq,Hkv", [(64, 448, 1500, 6, 6), (128, 256, 384, 4, 2), (64, 100, 640, 2, 1), (128, 300, 128, 2, 2)])
def test_cross_attention_with_different_query_and_key_lengths(D, Sq, Sk, Hq, Hkv):
    """Whisper's decoder attends from 448 text positions to 1500 audio positions: no causal part, two lengths, both padded."""
    torch.manual_seed(0)
    q = torch.randn(2, Sq, Hq, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(2, Sk, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(2, Sk, Hkv, D, device="cuda").bfloat16().requires_grad_()
    o = flash_attention_cuda(q, k, v, None)
    assert o.shape == q.shape
    g = torch.randn_like(o)
    o.backward(g)
    torch.cuda.synchronize()
    lib.check_status()
    qr, kr, vr = [t.detach().float().requires_grad_() for t in (q, k, v)]
    orf = simple_attention_with_dropout(qr, kr, vr, None, attention_dtype=torch.float32)
    orf.backward(g.float())
    _close(o, orf, 2e-2)
    _close(q.grad, qr.grad, 4e-2)
    _close(k.grad, kr.grad, 4e-2)
    _close(v.grad, vr.grad, 4e-2)
    from levanter_b200.ops import flash_attention as KFA

    assert KFA.supported(q, k, v, None, None, True, None)
    assert not KFA.supported(q, k, v, AttentionMask.causal(), None, True, None)
    assert not KFA.supported(q[:, :1], k, v, None, None, True, None)
