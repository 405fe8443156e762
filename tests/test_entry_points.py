"""Entry points and evaluation on CPU: ``train_lm`` end to end (cache build, training, tagged eval, checkpoint, resume),
``eval_lm`` on the checkpoint it wrote, the harness log-likelihood scorer, and parsing of the reference's YAML configs."""
import glob
import json
import math
import os

import numpy as np
import pytest
import torch

from levanter_b200 import config as C

# directory holding the reference project's YAML configs (its ``config/``); the parse-them-all test is skipped without it
REF_CONFIGS = os.environ.get("LEVANTER_REFERENCE_CONFIGS", "")


def _write_data(d, n=200, vocab=250):
    rng = np.random.default_rng(0)
    for s in range(2):
        with open(f"{d}/shard{s}.jsonl", "w") as f:
            for _ in range(n):
                f.write(json.dumps({"text": " ".join(map(str, rng.integers(0, vocab, size=int(rng.integers(20, 80)))))}) + "\n")


def _train_cfg(d, steps):
    return f"""
data:
  tokenizer: passthrough
  vocab_size: 256
  cache_dir: {d}/cache
  train_urls: ["{d}/shard0.jsonl"]
  validation_urls: ["{d}/shard1.jsonl"]
  tags: [synthetic]
model:
  type: llama
  seq_len: 64
  hidden_dim: 64
  intermediate_dim: 128
  num_layers: 2
  num_heads: 2
  num_kv_heads: 2
trainer:
  id: testrun
  num_train_steps: {steps}
  train_batch_size: 8
  per_device_eval_parallelism: 4
  steps_per_eval: 2
  max_eval_batches: 2
  require_accelerator: false
  tracker:
    type: json_logger
  checkpointer:
    base_path: {d}/ckpt
    save_interval: 1h
  log_dir: {d}/logs
optimizer:
  learning_rate: 3e-3
  warmup: 0.0
"""


@pytest.mark.entry
def test_train_lm_then_resume_then_eval_lm(tmp_path, monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    from levanter_b200.checkpoint import discover_latest_checkpoint
    from levanter_b200.main import eval_lm, train_lm

    d = str(tmp_path)
    _write_data(d)
    cfg = C.decode(train_lm.TrainLmConfig, __import__("yaml").safe_load(_train_cfg(d, 4)))
    train_lm.main(cfg)
    ck = discover_latest_checkpoint(f"{d}/ckpt/testrun")
    assert ck is not None and ck.endswith("step-3") or ck.endswith("step-4"), ck
    # resume: two more steps start from the saved step, not from zero
    cfg2 = C.decode(train_lm.TrainLmConfig, __import__("yaml").safe_load(_train_cfg(d, 6)))
    train_lm.main(cfg2)
    ck2 = discover_latest_checkpoint(f"{d}/ckpt/testrun")
    assert ck2 != ck
    ecfg = C.decode(eval_lm.EvalLmConfig, {"checkpoint_path": ck2, "data": cfg.__dict__ and __import__("yaml").safe_load(_train_cfg(d, 4))["data"],
                                           "model": __import__("yaml").safe_load(_train_cfg(d, 4))["model"],
                                           "trainer": {"require_accelerator": False, "per_device_eval_parallelism": 4, "max_eval_batches": 2,
                                                       "tracker": {"type": "noop"}, "log_dir": f"{d}/logs"}})
    out = eval_lm.main(ecfg)
    assert 0 < out["eval/loss"] < math.log(256) + 0.5


def test_tagged_evaluator_micro_macro():
    from levanter_b200.data.dataset import ListAsyncDataset
    from levanter_b200.eval import TaggedEvaluator
    from levanter_b200.models.llama import LlamaConfig
    from levanter_b200.models.lm_model import LmExample, compute_next_token_loss

    torch.manual_seed(0)
    cfg = LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=1, num_heads=2, num_kv_heads=2)
    model = cfg.build(50, seed=0)
    mk = lambda n, seed: [LmExample.causal(torch.randint(0, 50, (16,), generator=torch.Generator().manual_seed(seed + i), dtype=torch.int32))
                          for i in range(n)]
    a, b = mk(6, 0), mk(3, 100)
    ev = TaggedEvaluator(4, [(ListAsyncDataset(a, is_complete=True), ["web/a"]), (ListAsyncDataset(b, is_complete=True), ["web/b"])])
    r = ev.evaluate(model)
    with torch.no_grad():
        per = lambda exs: torch.stack([(compute_next_token_loss(model, LmExample.stack([e]), reduction=None)[0] * e.loss_mask).sum() for e in exs])
        la, lb = per(a), per(b)
    ta, tb = 6 * 15, 3 * 15
    assert abs(r.tag_micro_losses["web/a"] - la.sum().item() / ta) < 1e-4
    assert abs(r.tag_micro_losses["web/b"] - lb.sum().item() / tb) < 1e-4
    assert abs(r.micro_avg_loss - (la.sum() + lb.sum()).item() / (ta + tb)) < 1e-4
    assert abs(r.macro_avg_loss - 0.5 * (la.sum().item() / ta + lb.sum().item() / tb)) < 1e-4
    assert abs(r.tag_micro_losses["web"] - r.micro_avg_loss) < 1e-4 and abs(r.tag_macro_losses["web"] - r.macro_avg_loss) < 1e-4


def test_harness_scorer_matches_direct_loglikelihood():
    from levanter_b200.eval_harness import LoglikelihoodScorer
    from levanter_b200.layers.attention import AttentionMask
    from levanter_b200.models.llama import LlamaConfig

    cfg = LlamaConfig(seq_len=32, hidden_dim=32, intermediate_dim=64, num_layers=1, num_heads=2, num_kv_heads=2)
    model = cfg.build(40, seed=1).eval()
    rng = np.random.default_rng(0)
    pairs = [(rng.integers(1, 40, size=int(rng.integers(1, 8))).tolist(), rng.integers(1, 40, size=int(rng.integers(1, 5))).tolist())
             for _ in range(9)]
    got = LoglikelihoodScorer(model, 32, 2, pad_token_id=0, max_packed_segments=4).score(pairs)
    for (ctx, cont), (ll, greedy) in zip(pairs, got):
        ids = torch.tensor([ctx + cont], dtype=torch.int32)
        with torch.no_grad():
            acts = model.activations(ids, AttentionMask.causal())
            logits = (acts @ model.get_lm_head().t()).float()[0]
        lp = torch.log_softmax(logits, -1)
        want = sum(lp[len(ctx) - 1 + j, t].item() for j, t in enumerate(cont))
        want_greedy = all(int(logits[len(ctx) - 1 + j].argmax()) == t for j, t in enumerate(cont))
        assert abs(ll - want) < 1e-3, (ll, want)
        assert greedy == want_greedy


def _class_for(name):
    from levanter_b200.main.export_lm_to_hf import ConvertLmConfig
    from levanter_b200.main.lora_lm import LoraLmConfig
    from levanter_b200.main.sft import SFTConfig
    from levanter_b200.main.sft_mixture import SFTMixtureConfig
    from levanter_b200.main.train_lm import TrainLmConfig

    if name.startswith("sft_") or name == "olmo2_sft.yaml":
        return SFTMixtureConfig if ("mixture" in name or name == "olmo2_sft.yaml") else SFTConfig
    if name.startswith("lora"):
        return LoraLmConfig
    if name.startswith("convert"):
        return None  # needs command-line arguments
    if name.startswith("whisper"):
        from levanter_b200.main.train_asr import TrainASRConfig

        return TrainASRConfig
    return TrainLmConfig


@pytest.mark.skipif(not (REF_CONFIGS and os.path.isdir(REF_CONFIGS)), reason="set LEVANTER_REFERENCE_CONFIGS to the reference's config directory")
def test_reference_yaml_configs_parse():
    """Every training/SFT/LoRA config of the reference decodes into the matching config class here.  Exempt: a config whose
    model type the reference itself no longer ships."""
    exempt = {"backpack_nano.yaml"}
    failures = []
    n = 0
    for p in sorted(glob.glob(f"{REF_CONFIGS}/*.yaml")):
        name = os.path.basename(p)
        cls = _class_for(name)
        if cls is None or name in exempt:
            continue
        try:
            C.decode(cls, C.load_yaml(p))
            n += 1
        except Exception as e:  # noqa: BLE001
            failures.append((name, str(e).splitlines()[0][:200]))
    assert not failures, failures
    assert n >= 60
