"""Attention masks, the vanilla / blockwise-flash implementations, sinks, MLA, and rotary embeddings (modelled on the reference's
tests/test_attention.py, test_flash_attention.py, test_latent_attention.py, test_rotary.py)."""
import math

import pytest
import torch

from levanter_b200.layers.attention import (Attention, AttentionBackend, AttentionConfig, AttentionMask, AttentionWithSink,
                                            MultiHeadLatentAttention, MultiHeadLatentAttentionConfig, dot_product_attention,
                                            dot_product_attention_with_sink, simple_attention_with_dropout)
from levanter_b200.layers.rotary import (DefaultRotaryEmbeddingsConfig, Llama3RotaryEmbeddingsConfig, YarnRotaryEmbeddingsConfig,
                                         rotate_half)
from levanter_b200.models.flash_attention import flash_attention


def _naive(q, k, v, mask=None, cap=None):
    B, Sq, H, D = q.shape
    KV = k.shape[2]
    k = k.repeat_interleave(H // KV, dim=2)
    v = v.repeat_interleave(H // KV, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(D)
    if cap is not None:
        s = cap * torch.tanh(s / cap)
    if mask is not None:
        s = s.masked_fill(~mask, -1e9)
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), v.float())


def _qkv(B=2, Sq=12, Sk=12, H=4, KV=2, D=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, Sq, H, D, generator=g), torch.randn(B, Sk, KV, D, generator=g), torch.randn(B, Sk, KV, D, generator=g))


# ------------------------------------------------------------------------------------------------ masks
def test_causal_mask_materialize_and_blocks():
    m = AttentionMask.causal()
    full = m.materialize(6, 6)
    assert torch.equal(full.reshape(6, 6), torch.tril(torch.ones(6, 6, dtype=torch.bool)))
    blk = m.materialize(6, 6, q_slice=(2, 2), k_slice=(1, 3))
    assert torch.equal(blk.reshape(2, 3), full.reshape(6, 6)[2:4, 1:4])


def test_causal_offset_scalar_and_per_row():
    m = AttentionMask.causal(offset=2)  # query i sits at absolute position i + 2
    got = m.materialize(2, 4).reshape(2, 4)
    assert got.tolist() == [[True, True, True, False], [True, True, True, True]]
    per_row = AttentionMask.causal(offset=torch.tensor([0, 3])).materialize(1, 4)
    assert per_row.reshape(2, 4).tolist() == [[True, False, False, False], [True, True, True, True]]


def test_sliding_window_and_segments():
    m = AttentionMask.causal(sliding_window=2).materialize(4, 4).reshape(4, 4)
    assert m.tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]]
    seg = torch.tensor([[0, 0, 1, 1]])
    m = AttentionMask.causal().with_segment_ids(seg).materialize(4, 4).reshape(4, 4)
    assert m.tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 0, 1, 0], [0, 0, 1, 1]]


def test_mask_and_or():
    e = torch.zeros(3, 3, dtype=torch.bool)
    e[:, 0] = True
    both = (AttentionMask.causal() & AttentionMask.explicit(e)).materialize(3, 3).reshape(3, 3)
    assert both.tolist() == [[1, 0, 0], [1, 0, 0], [1, 0, 0]]
    # the union is structural (as in the reference): it stays causal only when both sides are, explicit masks are OR-ed
    either = AttentionMask.causal() | AttentionMask.explicit(e)
    assert not either.is_causal and torch.equal(either.materialize(3, 3).reshape(3, 3), e)
    e2 = torch.eye(3, dtype=torch.bool)
    u = AttentionMask(True, None, e) | AttentionMask(True, None, e2)
    assert u.is_causal and torch.equal(u.materialize(3, 3).reshape(3, 3), torch.tril(torch.ones(3, 3, dtype=torch.bool)) & (e | e2))
    assert (AttentionMask.causal(sliding_window=2) | AttentionMask.causal(sliding_window=5)).sliding_window == 5


# ------------------------------------------------------------------------------------------------ implementations
@pytest.mark.parametrize("mask_kind", ["none", "causal", "window", "segments", "explicit"])
def test_vanilla_and_blockwise_flash_match_naive(mask_kind):
    q, k, v = _qkv()
    mask = {"none": None, "causal": AttentionMask.causal(), "window": AttentionMask.causal(sliding_window=3),
            "segments": AttentionMask.causal().with_segment_ids(torch.tensor([[0] * 5 + [1] * 7, [0] * 12])),
            "explicit": AttentionMask.explicit(torch.rand(2, 12, 12, generator=torch.Generator().manual_seed(1)) > 0.3)}[mask_kind]
    if mask_kind == "explicit":
        idx = torch.arange(12)
        mask.explicit_mask[:, idx, idx] = True  # no fully-masked rows
    dense = None if mask is None else mask.materialize(12, 12)
    ref = _naive(q, k, v, dense)
    out_v = simple_attention_with_dropout(q, k, v, mask)
    out_f = flash_attention(q, k, v, mask, block_size=4)
    out_d = dot_product_attention(q, k, v, mask, attn_backend=AttentionBackend.VANILLA)
    for o in (out_v, out_f, out_d):
        assert torch.allclose(o.float(), ref, atol=1e-5, rtol=1e-4)


def test_blockwise_flash_gradients_match_vanilla():
    q, k, v = (t.requires_grad_() for t in _qkv(Sq=9, Sk=9))
    mask = AttentionMask.causal()
    flash_attention(q, k, v, mask, block_size=4).square().sum().backward()
    gf = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    simple_attention_with_dropout(q, k, v, mask).square().sum().backward()
    for a, b in zip(gf, (q.grad, k.grad, v.grad)):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)


def test_soft_cap_and_cross_lengths():
    q, k, v = _qkv(Sq=5, Sk=11)
    ref = _naive(q, k, v, None, cap=5.0)
    assert torch.allclose(flash_attention(q, k, v, None, block_size=4, logits_soft_cap=5.0).float(), ref, atol=1e-5, rtol=1e-4)
    assert torch.allclose(simple_attention_with_dropout(q, k, v, None, logits_soft_cap=5.0).float(), ref, atol=1e-5, rtol=1e-4)


def test_attention_sink_lowers_mass_without_changing_direction():
    q, k, v = _qkv(H=2, KV=2)
    sink = torch.zeros(2, 1)
    out = dot_product_attention_with_sink(q, k, v, sink, AttentionMask.causal())
    ref = _naive(q, k, v, AttentionMask.causal().materialize(12, 12))
    # position 0 attends to one real key with logit s and a sink with logit 0: weight = sigmoid(s)
    s0 = (q[:, 0].float() * k[:, 0].float()).sum(-1) / math.sqrt(8)
    assert torch.allclose(out[:, 0].float(), torch.sigmoid(s0)[..., None] * v[:, 0].float(), atol=1e-5)
    big = dot_product_attention_with_sink(q, k, v, torch.full((2, 1), -1e4), AttentionMask.causal())
    assert torch.allclose(big.float(), ref, atol=1e-5)


def test_attention_module_shapes_gqa_bias_and_qk_norm():
    from levanter_b200.layers.normalization import RmsNormConfig

    cfg = AttentionConfig(hidden_dim=32, num_heads=4, num_kv_heads=2, use_bias=True, qk_norm=RmsNormConfig(),
                          rope=DefaultRotaryEmbeddingsConfig())
    attn = Attention(cfg)
    x = torch.randn(2, 10, 32)
    y = attn(x, AttentionMask.causal())
    assert y.shape == x.shape
    # causality: changing a later token leaves earlier outputs alone
    x2 = x.clone()
    x2[:, 7] += 1.0
    y2 = attn(x2, AttentionMask.causal())
    assert torch.allclose(y[:, :7], y2[:, :7], atol=1e-6) and not torch.allclose(y[:, 7:], y2[:, 7:])


def test_mla_shapes_and_causality():
    cfg = MultiHeadLatentAttentionConfig(hidden_dim=32, num_heads=4, kv_lora_rank=8, q_lora_rank=None, qk_rope_head_dim=4, qk_nope_head_dim=8, v_head_dim=8)
    mla = MultiHeadLatentAttention(cfg)
    x = torch.randn(2, 6, 32)
    y = mla(x, AttentionMask.causal())
    assert y.shape == x.shape
    x2 = x.clone()
    x2[:, 4] += 1.0
    assert torch.allclose(y[:, :4], mla(x2, AttentionMask.causal())[:, :4], atol=1e-6)


# ------------------------------------------------------------------------------------------------ rotary
def test_rotary_is_a_rotation_and_relative():
    rope = DefaultRotaryEmbeddingsConfig(theta=10000.0).build(8)
    q = torch.randn(1, 5, 2, 8)
    pos = torch.arange(5)
    rq = rope(q, pos)
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    assert torch.allclose(rq[:, 0], q[:, 0], atol=1e-6)  # position 0 is the identity
    k = torch.randn(1, 5, 2, 8)
    a = (rope(q, pos)[:, 3] * rope(k, pos)[:, 1]).sum(-1)
    b = (rope(q, pos + 7)[:, 3] * rope(k, pos + 7)[:, 1]).sum(-1)
    assert torch.allclose(a, b, atol=1e-4)  # scores depend on the position difference only
    assert torch.equal(rotate_half(torch.tensor([1.0, 2.0, 3.0, 4.0])), torch.tensor([-3.0, -4.0, 1.0, 2.0]))


def test_llama3_and_yarn_scaling_match_hf():
    transformers = pytest.importorskip("transformers")
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

    hd = 16
    l3 = Llama3RotaryEmbeddingsConfig(theta=500000.0, factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
    hf_cfg = transformers.LlamaConfig(hidden_size=hd * 2, num_attention_heads=2, rope_theta=500000.0, max_position_embeddings=131072,
                                      rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                                    "original_max_position_embeddings": 8192})
    inv, scale = ROPE_INIT_FUNCTIONS["llama3"](hf_cfg, "cpu")
    assert torch.allclose(l3.build(hd).inv_freq, inv.float(), rtol=1e-5, atol=1e-9)


def test_yarn_ramp_follows_the_reference_formula():
    # (the reference's YaRN differs from the Hugging Face one: its ramp bounds use half the head size and it also scales positions)
    hd = 16
    cfg = YarnRotaryEmbeddingsConfig(theta=10000.0, factor=4.0, beta_fast=32.0, beta_slow=1.0, original_max_position_embeddings=2048)
    r = cfg.build(hd)
    base = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    find = lambda n: (hd // 2 * math.log(2048 / (n * 2 * math.pi))) / (2 * math.log(10000.0))
    low, high = max(int(math.floor(find(32.0))), 0), min(int(math.ceil(find(1.0))), hd // 2 - 1)
    ramp = torch.clamp((torch.arange(hd // 2).float() - low) / max(high - low, 1), 0, 1)
    assert torch.allclose(r.inv_freq, base / 4.0 * ramp + base * (1 - ramp))
    assert r.inv_freq[0] == base[0] and torch.allclose(r.inv_freq[-1], base[-1] / 4.0)
    assert r.temperature == pytest.approx(math.sqrt(0.1 * math.log(4.0) + 1.0)) and r.position_scale == 0.25
    theta, d = cfg.to_hf_config()
    assert YarnRotaryEmbeddingsConfig.make_from_hf_config(theta, d) == cfg


def test_attention_with_sink_module_and_window_helper():
    """The module form: zero sinks lower every attention weight by the sink's share; very negative sinks give plain attention
    back.  ``with_sliding_window`` changes only the window of a mask."""
    import dataclasses

    from levanter_b200.layers.attention import Attention, AttentionConfig, AttentionMask, AttentionWithSink

    torch.manual_seed(0)
    cfg = AttentionConfig(hidden_dim=32, num_heads=4, num_kv_heads=2)
    plain = Attention(cfg).eval()
    sink = AttentionWithSink(cfg).eval()
    sink.load_state_dict({**plain.state_dict(), "sinks": torch.zeros(2, 2)})
    assert sink.sinks.shape == (2, 2)  # one logit per query head, grouped by key/value head
    x = torch.randn(2, 10, 32)
    mask = AttentionMask.causal()
    with torch.no_grad():
        base = plain(x, mask)
        with_sink = sink(x, mask)
        assert not torch.allclose(with_sink, base, atol=1e-4)
        sink.sinks.fill_(-1e4)
        assert torch.allclose(sink(x, mask), base, atol=1e-5)
        assert sink(x[0], mask).shape == (10, 32)  # unbatched input
    loss = sink(x, mask).sum()
    sink.sinks.data.zero_()
    sink(x, mask).sum().backward()
    assert sink.sinks.grad is not None and float(sink.sinks.grad.abs().sum()) > 0

    m = AttentionMask.causal().with_sliding_window(3)
    assert m.is_causal and m.sliding_window == 3
    dense = m.materialize(6, 6)
    assert dense.reshape(6, 6)[5].tolist() == [False, False, False, True, True, True]
    assert dataclasses.replace(m, sliding_window=None) == AttentionMask.causal()


def test_passthrough_tokenizer_is_enough_of_a_tokenizer():
    from levanter_b200.data.passthrough_tokenizer import PassthroughTokenizer

    tok = PassthroughTokenizer(100, bos_token_id=1)
    assert len(tok) == tok.vocab_size == 100 and tok.eos_token_id == 99 and tok.eos_token == "99" and tok.bos_token == "1"
    assert PassthroughTokenizer(10).bos_token is None and tok.pad_token_id == 99
    assert tok.encode("3 4 5") == [3, 4, 5] and tok.decode([3, 4, 5]) == "3 4 5"
    assert tok(["1 2", "3"])["input_ids"] == [[1, 2], [3]] and tok("7 8")["input_ids"] == [7, 8]
    assert tok.convert_ids_to_tokens([3, 4]) == ["3", "4"] and tok.convert_tokens_to_ids(["3", "4"]) == [3, 4] and tok.convert_tokens_to_ids("9") == 9
    assert tok.get_vocab()["42"] == 42 and tok.save_vocabulary("/nowhere") == ()
    with pytest.raises(ValueError, match="integers"):
        tok.encode("3 x")
