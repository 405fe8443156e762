"""Model numerics against Hugging Face PyTorch implementations: HF model -> save -> load_pretrained -> logits match ->
save_pretrained -> reload in HF -> logits match (the reference's roundtrip tests, tests/test_llama.py:221-286 and siblings)."""
import tempfile

import pytest
import torch

transformers = pytest.importorskip("transformers")

from levanter_b200.compat.hf_checkpoints import HFCheckpointConverter
from levanter_b200.layers.attention import AttentionMask


def _tiny(model_type):
    common = dict(vocab_size=200, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                  max_position_embeddings=64)
    if model_type == "llama":
        return transformers.LlamaConfig(**common, num_key_value_heads=2, rms_norm_eps=1e-5)
    if model_type == "llama3":
        return transformers.LlamaConfig(**common, num_key_value_heads=2, rope_theta=500000.0,
                                        rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 32})
    if model_type == "mistral":
        return transformers.MistralConfig(**common, num_key_value_heads=2, sliding_window=None)
    if model_type == "qwen2":
        return transformers.Qwen2Config(**common, num_key_value_heads=2)
    if model_type == "qwen3":
        return transformers.Qwen3Config(**common, num_key_value_heads=2, head_dim=8)
    if model_type == "gemma":
        return transformers.GemmaConfig(**common, num_key_value_heads=1, head_dim=8)
    if model_type == "gemma2":
        return transformers.Gemma2Config(**common, num_key_value_heads=2, head_dim=8, query_pre_attn_scalar=8,
                                         sliding_window=4096, final_logit_softcapping=None)
    if model_type == "mixtral":
        return transformers.MixtralConfig(**common, num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2,
                                          sliding_window=None)
    if model_type == "olmo2":
        return transformers.Olmo2Config(**common, num_key_value_heads=2)
    if model_type == "gpt2":
        return transformers.GPT2Config(vocab_size=200, n_embd=32, n_layer=2, n_head=4, n_positions=64)
    raise KeyError(model_type)


@pytest.mark.parametrize("model_type", ["llama", "llama3", "mistral", "qwen2", "qwen3", "gemma", "gemma2", "mixtral", "olmo2", "gpt2"])
def test_hf_roundtrip(model_type):
    torch.manual_seed(0)
    hf_cfg = _tiny(model_type)
    hf_cfg._attn_implementation = "eager"
    hf_model = transformers.AutoModelForCausalLM.from_config(hf_cfg).eval().float()
    tokens = torch.randint(0, 200, (2, 32))
    with torch.no_grad():
        ref = hf_model(tokens).logits
    with tempfile.TemporaryDirectory() as tmp:
        hf_model.save_pretrained(f"{tmp}/hf", safe_serialization=True)
        conv = HFCheckpointConverter.from_hf(f"{tmp}/hf")
        model = conv.load_pretrained(ref=f"{tmp}/hf", resize_vocab_to_match_tokenizer=False).eval()
        with torch.no_grad():
            ours = model(tokens, AttentionMask.causal())
        assert torch.allclose(ours, ref, atol=2e-4, rtol=2e-4), (ours - ref).abs().max()
        conv.save_pretrained(model, f"{tmp}/out", save_tokenizer=False)
        back = transformers.AutoModelForCausalLM.from_pretrained(f"{tmp}/out").eval().float()
        with torch.no_grad():
            again = back(tokens).logits
        assert torch.allclose(again, ref, atol=2e-4, rtol=2e-4), (again - ref).abs().max()


def test_sharded_save_and_state_dict_keys():
    from levanter_b200.compat.hf_checkpoints import to_hf_state_dict
    from levanter_b200.models.llama import LlamaConfig

    cfg = LlamaConfig(seq_len=32, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=4, num_kv_heads=2)
    model = cfg.build(100, seed=0)
    sd = to_hf_state_dict(model)
    hf = transformers.AutoModelForCausalLM.from_config(transformers.LlamaConfig(**{k: v for k, v in cfg.to_hf_config(100).items()
                                                                               if k not in ("model_type", "architectures")}))
    assert set(sd.keys()) == set(hf.state_dict().keys())
    with tempfile.TemporaryDirectory() as tmp:
        conv = HFCheckpointConverter(LlamaConfig, reference_checkpoint=None)
        conv.save_pretrained(model, tmp, save_tokenizer=False, max_shard_size=20_000)
        import os

        assert os.path.exists(f"{tmp}/model.safetensors.index.json")
        conv2 = HFCheckpointConverter(LlamaConfig, reference_checkpoint=tmp)
        m2 = conv2.load_pretrained(resize_vocab_to_match_tokenizer=False)
        for (n1, p1), (n2, p2) in zip(model.named_parameters(), m2.named_parameters()):
            assert torch.equal(p1, p2), n1
