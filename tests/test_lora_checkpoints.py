"""LoRA with the trainer's checkpoints and with Hugging Face exports: only adapter weights are written to a training checkpoint,
a run resumes from it, and the merged export loads in transformers with the adapted model's logits
(levanter_b200/lora.py; scenarios after the reference's tests/test_lora.py)."""
import os

import pytest
import torch

from levanter_b200 import config as C
from levanter_b200.checkpoint import discover_latest_checkpoint
from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.layers.attention import AttentionMask
from levanter_b200.lora import LoraConfig, LoraLinear, lora_trainable_params_filter, loraize, save_merged_hf_model
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
from levanter_b200.nn import Linear
from levanter_b200.optim import AdamConfig
from levanter_b200.trainer import Trainer, TrainerConfig

VOCAB = 64


def _llama():
    return LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, gradient_checkpointing=False)


def test_only_the_targets_are_wrapped():
    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.first, self.second = Linear(6, 5), Linear(5, 4)

        def forward(self, x):
            return self.second(self.first(x))

    torch.manual_seed(0)
    base = Two()
    x = torch.randn(3, 6)
    ref = base(x)
    a = loraize(Two(), LoraConfig(r=8, target_modules=["first"]), seed=0)
    assert isinstance(a.first, LoraLinear) and type(a.second) is Linear
    b = loraize(Two(), LoraConfig(r=8, target_modules=["second"]), seed=0)
    assert type(b.first) is Linear and isinstance(b.second, LoraLinear)
    assert b.second.lora.lora_A.weight.shape == (8, 5) and b.second.lora.lora_B.weight.shape == (4, 8)
    everything = loraize(Two(), LoraConfig(r=2, target_modules=None), seed=0)
    assert isinstance(everything.first, LoraLinear) and isinstance(everything.second, LoraLinear)
    assert ref.shape == (3, 4)


def _train(tmp, steps):
    cfg = C.decode(TrainerConfig, {"num_train_steps": steps, "train_batch_size": 8, "require_accelerator": False, "tracker": {"type": "noop"},
                                   "log_dir": f"{tmp}/logs", "id": "lora", "seed": 1,
                                   "checkpointer": {"base_path": f"{tmp}/ckpt", "save_interval": "10h"}})
    g = torch.Generator().manual_seed(0)
    starts = torch.randint(0, VOCAB, (256,), generator=g)
    data = ListAsyncDataset([LmExample.causal(((s + torch.arange(16)) % VOCAB).to(torch.int32)) for s in starts], is_complete=True)
    opt = AdamConfig(learning_rate=1e-2, warmup=0.0, weight_decay=0.0, lr_schedule="constant", min_lr_ratio=1.0)
    losses = {}
    with Trainer(cfg, opt, compute_next_token_loss) as trainer:
        model = loraize(_llama().build(VOCAB, seed=3), LoraConfig(r=4, target_modules=["q_proj", "v_proj"]), seed=5)
        state = trainer.initial_state(0, model=model, is_trainable=lora_trainable_params_filter(model))
        first = int(state.step)
        trainer.add_hook(lambda info: losses.__setitem__(info.step, float(info.loss)), every=1)
        info = trainer.train(state, trainer.data_loader(data).iter_from_step(first))
    return first, losses, info.state.model


def test_training_checkpoints_hold_only_the_adapters_and_resume(tmp_path):
    d = str(tmp_path)
    base = {n: p.detach().clone() for n, p in _llama().build(VOCAB, seed=3).named_parameters()}
    _, full_losses, full_model = _train(d + "/full", 6)
    # base weights did not move, adapters did
    moved = {n: p for n, p in full_model.named_parameters() if "lora" in n}
    assert moved and any(float(p.detach().abs().sum()) > 0 for n, p in moved.items() if "lora_B" in n)
    for n, p in full_model.named_parameters():
        if "lora" not in n:
            assert torch.equal(p, base[n.replace(".wrapped", "")]), n
    assert full_losses[5] < full_losses[0]

    _train(d + "/run", 3)
    ck = discover_latest_checkpoint(d + "/run/ckpt/lora")
    assert ck.endswith("step-2")
    files = [os.path.join(r, f) for r, _, fs in os.walk(os.path.join(ck, "model")) for f in fs]
    assert files and all("lora" in f for f in files), [f for f in files if "lora" not in f][:3]  # no base weight was written
    assert any("lora_A" in f for f in files) and any("lora_B" in f for f in files)
    first, losses, model = _train(d + "/run", 6)
    assert first == 3 and [losses[i] for i in (3, 4, 5)] == pytest.approx([full_losses[i] for i in (3, 4, 5)], abs=1e-5)
    for (n, p), (_, q) in zip(full_model.named_parameters(), model.named_parameters()):
        assert torch.allclose(p, q, atol=1e-5), n


def test_the_merged_export_loads_in_transformers_with_the_adapted_logits(tmp_path):
    transformers = pytest.importorskip("transformers")
    cfg = _llama()
    model = cfg.build(VOCAB, seed=0).eval()
    converter = cfg.hf_checkpoint_converter()
    ids = torch.randint(0, VOCAB, (1, 16), generator=torch.Generator().manual_seed(0))
    converter.save_pretrained(model, str(tmp_path / "base"), save_tokenizer=False)
    with torch.no_grad():
        base_out = model(ids, AttentionMask.causal())
        hf_base = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "base")).eval()(ids.long()).logits
    assert torch.allclose(base_out, hf_base, atol=1e-4)

    lora = loraize(model, LoraConfig(r=8, target_modules=["q_proj", "k_proj", "v_proj"]), seed=0)
    with torch.no_grad():
        for n, p in lora.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.05)
        lora_out = lora(ids, AttentionMask.causal())
    assert not torch.allclose(lora_out, base_out, atol=1e-3)
    save_merged_hf_model(lora, converter, str(tmp_path / "merged"))
    with torch.no_grad():
        hf_merged = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "merged")).eval()(ids.long()).logits
    assert torch.allclose(lora_out, hf_merged, atol=1e-4)
    assert any(isinstance(m, LoraLinear) for m in lora.modules())  # exporting did not merge the live model


def test_adapter_parameters_partition_and_the_export_hooks(tmp_path):
    from types import SimpleNamespace

    from levanter_b200.lora import (combine_lora_params, filter_lora_params, partition_lora_params, save_merged_hf_checkpoint_callback,
                                    save_peft_checkpoint_callback)

    cfg = _llama()
    lora_cfg = LoraConfig(r=2, target_modules=["q_proj"])
    model = loraize(cfg.build(VOCAB, seed=0), lora_cfg, seed=1)
    params = dict(model.named_parameters())
    adapters, base = partition_lora_params(params)
    assert adapters and base and set(adapters) | set(base) == set(params) and not set(adapters) & set(base)
    assert filter_lora_params(params).keys() == adapters.keys() and all("lora" in k for k in adapters)
    new = {k: torch.zeros_like(v) for k, v in adapters.items()}
    combined = combine_lora_params(base, new)
    assert set(combined) == set(params) and all(float(combined[k].abs().sum()) == 0 for k in adapters)
    wrapped = [m for m in model.modules() if isinstance(m, LoraLinear)]
    assert wrapped[0].in_features == 32 and wrapped[0].out_features == 32 and wrapped[0].bias is None and wrapped[0].weight.shape == (32, 32)

    conv = cfg.hf_checkpoint_converter()
    merged_hook = save_merged_hf_checkpoint_callback(str(tmp_path / "merged"), conv, save_tokenizer=False)
    peft_hook = save_peft_checkpoint_callback(str(tmp_path / "peft"), lora_cfg, "org/base")
    for hook in (merged_hook, peft_hook):
        hook(SimpleNamespace(step=0, eval_model=model))  # nothing is exported at step 0
        hook(SimpleNamespace(step=5, eval_model=model))
    assert os.listdir(tmp_path / "merged") == ["step-5"] and os.path.exists(tmp_path / "merged" / "step-5" / "config.json")
    assert os.listdir(tmp_path / "peft") == ["step-5"] and os.path.exists(tmp_path / "peft" / "step-5" / "adapter_config.json")
    assert any(isinstance(m, LoraLinear) for m in model.modules())
