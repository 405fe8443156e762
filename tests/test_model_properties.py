"""Properties every decoder family must have, on tiny CPU models: the Hugging Face config survives a round trip, parameter
formulas agree with the built model, the position-table size and the length of the input do not change predictions, activation
checkpointing changes neither loss nor gradients, every parameter gets a finite gradient, and the exported names are the names
transformers uses (scenarios after the reference's tests/test_llama.py, test_gemma.py, test_olmo.py, test_mistral.py,
test_mixtral.py, gpt2_test.py)."""
import dataclasses

import pytest
import torch

from levanter_b200.compat.hf_checkpoints import to_hf_state_dict
from levanter_b200.layers.attention import AttentionMask
from levanter_b200.models.gemma import Gemma2Config, Gemma3Config, GemmaConfig
from levanter_b200.models.gpt2 import Gpt2Config
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
from levanter_b200.models.mistral import MistralConfig
from levanter_b200.models.mixtral import MixtralConfig
from levanter_b200.models.olmo import Olmo2Config
from levanter_b200.models.qwen import Qwen3Config, QwenConfig

VOCAB = 200
COMMON = dict(seq_len=64, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=4, num_kv_heads=2, gradient_checkpointing=False)


def _configs():
    return {
        "llama": LlamaConfig(**COMMON),
        "llama_mha": LlamaConfig(**{**COMMON, "num_kv_heads": 4}),
        "llama_mqa": LlamaConfig(**{**COMMON, "num_kv_heads": 1}),
        "mistral": MistralConfig(**COMMON),
        "qwen2": QwenConfig(**COMMON),
        "qwen3": Qwen3Config(**COMMON, head_dim=8),
        "gemma": GemmaConfig(**{**COMMON, "num_kv_heads": 1}, head_dim=8),
        "gemma2": Gemma2Config(**COMMON, head_dim=8),
        "gemma3": Gemma3Config(**COMMON, head_dim=8),
        "olmo2": Olmo2Config(**COMMON),
        "mixtral": MixtralConfig(**COMMON, n_routed_experts=4, num_experts_per_tok=2),
        "gpt2": Gpt2Config(seq_len=64, hidden_dim=32, num_layers=2, num_heads=4, gradient_checkpointing=False),
    }


FAMILIES = list(_configs())


def _cfg(name, **kw):
    c = _configs()[name]
    return dataclasses.replace(c, **kw) if kw else c


@pytest.mark.parametrize("name", FAMILIES)
def test_hf_config_round_trip(name):
    transformers = pytest.importorskip("transformers")
    cfg = _cfg(name)
    hf_dict = cfg.to_hf_config(VOCAB)
    assert hf_dict["vocab_size"] == VOCAB
    hf_cls = transformers.CONFIG_MAPPING[hf_dict["model_type"]]
    hf_cfg = hf_cls(**{k: v for k, v in hf_dict.items() if k not in ("model_type", "architectures")})
    back = type(cfg).from_hf_config(hf_cfg)
    for f in dataclasses.fields(cfg):
        if f.name in ("gradient_checkpointing", "attn_backend", "flash_attention_block_size", "use_flash_attention", "scan_layers",
                      "reference_checkpoint", "tokenizer", "upcast_attn"):
            continue
        a, b = getattr(back, f.name), getattr(cfg, f.name)
        if f.name == "sliding_window":  # "no window" is exported as a window of the whole sequence
            a, b = a or cfg.seq_len, b or cfg.seq_len
        if f.name == "sliding_window_pattern":  # "every layer global" is exported as a pattern of 1
            a, b = a or 1, b or 1
        assert a == b, f.name


@pytest.mark.parametrize("name", FAMILIES)
def test_parameter_formula_matches_the_built_model_whatever_the_sequence_length(name):
    cfg = _cfg(name)
    model = cfg.build(VOCAB, seed=0)
    n = sum(p.numel() for p in model.parameters())
    assert cfg.total_trainable_params(VOCAB) == n
    if name != "gpt2":  # (GPT-2 learns a position table: its size is the sequence length)
        longer = _cfg(name, seq_len=128).build(VOCAB, seed=0)
        assert sum(p.numel() for p in longer.parameters()) == n
    flops = cfg.flops_per_token(VOCAB)
    assert flops is not None and flops > 2 * 0.5 * n  # at least two flops per (active) matrix weight


def test_llama2_7b_parameter_count_and_flops():
    """Llama-2 7B has 6,738,415,616 parameters; its forward pass costs 10 to 20 % more than two flops per parameter and token
    at 4096 tokens of context (the attention products)."""
    cfg = LlamaConfig(seq_len=4096, hidden_dim=4096, intermediate_dim=11008, num_layers=32, num_heads=32, num_kv_heads=32)
    assert cfg.total_trainable_params(32000) == 6_738_415_616
    ratio = cfg.flops_per_token(32000) / (2 * 6.738415616e9)
    assert 1.1 < ratio < 1.2


@pytest.mark.parametrize("name", FAMILIES)
def test_a_shorter_input_gives_the_same_predictions_for_its_positions(name):
    torch.manual_seed(0)
    model = _cfg(name).build(VOCAB, seed=0).eval()
    ids = torch.randint(0, VOCAB, (2, 64))
    with torch.no_grad():
        full = model(ids, AttentionMask.causal())
        short = model(ids[:, :23], AttentionMask.causal())
    assert short.shape == (2, 23, VOCAB)
    assert torch.allclose(short, full[:, :23], atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("name", [f for f in FAMILIES if f != "gpt2"])
def test_the_configured_sequence_length_does_not_change_predictions(name):
    ids = torch.randint(0, VOCAB, (1, 48), generator=torch.Generator().manual_seed(0))
    outs = []
    for seq_len in (64, 256):
        model = _cfg(name, seq_len=seq_len).build(VOCAB, seed=0).eval()
        with torch.no_grad():
            outs.append(model(ids, AttentionMask.causal()))
    assert torch.allclose(outs[0], outs[1], atol=1e-5)


def _loss_and_grads(model, ids):
    ex = LmExample.causal(ids)
    loss = compute_next_token_loss(model, ex)
    model.zero_grad(set_to_none=True)
    loss.backward()
    return float(loss.detach()), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("name", FAMILIES)
def test_every_parameter_gets_a_finite_gradient_and_checkpointing_changes_nothing(name):
    ids = torch.randint(0, VOCAB, (2, 32), generator=torch.Generator().manual_seed(1)).to(torch.int32)
    plain = _cfg(name).build(VOCAB, seed=0).train()
    remat = _cfg(name, gradient_checkpointing=True).build(VOCAB, seed=0).train()
    l0, g0 = _loss_and_grads(plain, ids)
    l1, g1 = _loss_and_grads(remat, ids)
    names = {n for n, _ in plain.named_parameters()}
    missing = names - set(g0)
    if name == "mixtral":  # an expert that no token of this tiny batch was routed to has no gradient: allowed
        missing = {m for m in missing if ".experts." not in m and "block_sparse_moe" not in m}
    assert not missing, sorted(missing)[:5]
    assert all(torch.isfinite(g).all() for g in g0.values())
    assert any(float(g.abs().sum()) > 0 for g in g0.values())
    assert l1 == pytest.approx(l0, rel=1e-6)
    for n in g0:
        assert torch.allclose(g0[n], g1[n], atol=1e-6, rtol=1e-5), n


@pytest.mark.parametrize("name", FAMILIES)
def test_exported_names_and_shapes_are_the_ones_transformers_uses(name):
    transformers = pytest.importorskip("transformers")
    cfg = _cfg(name)
    hf_dict = cfg.to_hf_config(VOCAB)
    hf_cls = transformers.CONFIG_MAPPING[hf_dict["model_type"]]
    hf_model = transformers.AutoModelForCausalLM.from_config(hf_cls(**{k: v for k, v in hf_dict.items() if k not in ("model_type", "architectures")}))
    theirs = {k: tuple(v.shape) for k, v in hf_model.state_dict().items() if not k.endswith((".attn.bias", ".attn.masked_bias", "rotary_emb.inv_freq"))}
    ours = {k: tuple(v.shape) for k, v in to_hf_state_dict(cfg.build(VOCAB, seed=0)).items()}
    if name == "gpt2":  # checkpoints on the hub carry no "transformer." prefix; transformers accepts both
        theirs = {k.removeprefix("transformer."): v for k, v in theirs.items()}
    if name == "mixtral":
        # the export keeps the per-expert names of published checkpoints (block_sparse_moe.experts.N.w1); newer transformers
        # fuses them on load, so only the tensors outside the expert block can be compared by name
        theirs = {k: v for k, v in theirs.items() if ".mlp." not in k}
        ours = {k: v for k, v in ours.items() if ".block_sparse_moe." not in k}
    tied = {"lm_head.weight"} if getattr(hf_model.config, "tie_word_embeddings", False) else set()
    assert set(ours) | tied == set(theirs) | tied, (sorted(set(ours) - set(theirs))[:5], sorted(set(theirs) - set(ours))[:5])
    for k in ours:
        if k in theirs:
            assert ours[k] == theirs[k], k


RESIZABLE = FAMILIES + ["gated_deltanet", "gpt2_hyena"]


def _any_cfg(name):
    if name == "gated_deltanet":
        from levanter_b200.models.gated_deltanet import GatedDeltaNetConfig

        return GatedDeltaNetConfig(seq_len=64, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, head_k_dim=8, head_v_dim=8, chunk_size=16, gradient_checkpointing=False)
    if name == "gpt2_hyena":
        from levanter_b200.models.gpt2_hyena import Gpt2HyenaConfig
        from levanter_b200.models.hyena import HyenaConfig

        return Gpt2HyenaConfig(num_layers=2, gradient_checkpointing=False, hyena=HyenaConfig(seq_len=64, hidden_dim=32, filter_order=8))
    return _cfg(name)


@pytest.mark.parametrize("name", RESIZABLE)
def test_resizing_the_vocabulary_keeps_the_old_rows_and_the_old_predictions(name):
    model = _any_cfg(name).build(VOCAB, seed=0).eval()
    ids = torch.randint(0, VOCAB, (1, 16), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        before = model(ids, AttentionMask.causal())
    bigger = model.resize_vocab(VOCAB + 24)
    assert bigger.vocab_size == VOCAB + 24
    with torch.no_grad():
        after = bigger(ids, AttentionMask.causal())
    assert after.shape == (1, 16, VOCAB + 24)
    assert torch.allclose(after[..., :VOCAB], before, atol=1e-5)  # logits of the old tokens do not move
    assert torch.isfinite(after).all() and float(after[..., VOCAB:].abs().sum()) > 0  # the new rows are initialised, not zeros
    loss = compute_next_token_loss(bigger.train(), LmExample.causal(torch.randint(0, VOCAB + 24, (2, 16)).to(torch.int32)))
    loss.backward()
    assert all(p.grad is None or torch.isfinite(p.grad).all() for p in bigger.parameters())
    smaller = bigger.eval().resize_vocab(VOCAB - 40)
    with torch.no_grad():
        cut = smaller(ids.clamp(max=VOCAB - 41), AttentionMask.causal())
    assert cut.shape[-1] == VOCAB - 40 and smaller.vocab_size == VOCAB - 40


def test_prompt_and_completion_examples_mask_the_prompt():
    tokens = torch.arange(8, dtype=torch.int32)
    ex = LmExample.from_prompt_and_completion(tokens, prompt_length=3)
    assert ex.loss_mask.tolist() == [0, 0, 1, 1, 1, 1, 1, 0] and ex.attn_mask.is_causal  # position 2 predicts the first completion token
    batch = LmExample.from_prompt_and_completion(torch.arange(16, dtype=torch.int32).reshape(2, 8), prompt_length=torch.tensor([1, 6]), ignore_id=15)
    assert batch.loss_mask.tolist() == [[1, 1, 1, 1, 1, 1, 1, 0], [0, 0, 0, 0, 0, 1, 0, 0]]  # the token before an ignored one is not scored
    with pytest.raises(NotImplementedError):
        LmExample.from_prompt_and_completion(tokens, 3, all_causal=False)
