"""The other entry points, end to end on a CPU with a tokenizer trained in memory: cache_dataset, train_lm with a Hugging Face
export, export_lm_to_hf / export_hf_to_lm, sample_lm, viz_logprobs and lora_lm chained on the artefacts of one tiny run."""
import json
import os

import numpy as np
import pytest
import yaml

from levanter_b200 import config as C

pytestmark = pytest.mark.entry


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    pytest.importorskip("tokenizers")
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    d = tmp_path_factory.mktemp("chain")
    words = "the quick brown fox jumps over the lazy dog while seven small birds sing near a quiet river at dawn".split()
    rng = np.random.default_rng(0)
    docs = [" ".join(rng.choice(words, size=int(rng.integers(12, 40)))) + "." for _ in range(240)]
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(docs, trainers.BpeTrainer(vocab_size=300, special_tokens=["<s>", "</s>", "<pad>"],
                                                      initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", pad_token="<pad>")
    fast.save_pretrained(str(d / "tok"))
    for s in range(2):
        with open(d / f"shard{s}.jsonl", "w") as f:
            for t in docs[s * 120:(s + 1) * 120]:
                f.write(json.dumps({"text": t}) + "\n")
    return d


def _base(d, steps=3):
    return yaml.safe_load(f"""
data:
  tokenizer: {d}/tok
  cache_dir: {d}/cache
  train_urls: ["{d}/shard0.jsonl"]
  validation_urls: ["{d}/shard1.jsonl"]
model:
  type: llama
  seq_len: 32
  hidden_dim: 32
  intermediate_dim: 64
  num_layers: 2
  num_heads: 2
  num_kv_heads: 2
  gradient_checkpointing: false
trainer:
  id: chain
  num_train_steps: {steps}
  train_batch_size: 8
  require_accelerator: false
  tracker: {{type: noop}}
  log_dir: {d}/logs
  steps_per_eval: 100
  max_eval_batches: 1
  checkpointer:
    base_path: {d}/ckpt
    save_interval: 10h
optimizer:
  learning_rate: 1.0e-3
  warmup: 0.0
""")


def test_chain(workdir, monkeypatch, capsys):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    from levanter_b200.checkpoint import discover_latest_checkpoint
    from levanter_b200.main import cache_dataset, export_hf_to_lm, export_lm_to_hf, lora_lm, sample_lm, train_lm, viz_logprobs

    # ---- cache_dataset builds the token cache that training then finds
    ccfg = C.decode(cache_dataset.RayCachedLMDatasetConfig, _base(d)["data"])
    cache_dataset.main(ccfg)
    assert os.path.exists(f"{d}/cache/train/shard_ledger.json") and json.load(open(f"{d}/cache/train/shard_ledger.json"))["is_finished"]

    # ---- train_lm, exporting Hugging Face weights at the end
    tcfg = _base(d)
    tcfg["hf_save_path"] = f"{d}/hf_from_training"
    tcfg["hf_save_steps"] = 3
    train_lm.main(C.decode(train_lm.TrainLmConfig, tcfg))
    ck = discover_latest_checkpoint(f"{d}/ckpt/chain")
    assert ck is not None

    # ---- export_lm_to_hf, then back with export_hf_to_lm
    export_lm_to_hf.main(C.decode(export_lm_to_hf.ConvertLmConfig, {"checkpoint_path": ck, "output_dir": f"{d}/hf", "model": _base(d)["model"],
                                                                    "tokenizer": f"{d}/tok", "use_cpu": True,
                                                                    "trainer": {"require_accelerator": False}}))
    assert os.path.exists(f"{d}/hf/config.json") and any(f.endswith(".safetensors") for f in os.listdir(f"{d}/hf"))
    assert json.load(open(f"{d}/hf/config.json"))["hidden_size"] == 32
    export_hf_to_lm.main(C.decode(export_hf_to_lm.ImportHfConfig, {"hf_checkpoint": f"{d}/hf", "output_path": f"{d}/imported", "dtype": "float32",
                                                                   "tokenizer": f"{d}/tok"}))
    assert os.path.exists(f"{d}/imported/metadata.json")

    # ---- sample_lm from the exported directory
    capsys.readouterr()
    sample_lm.main(C.decode(sample_lm.SampleLmConfig, {"hf_checkpoint": f"{d}/hf", "tokenizer": f"{d}/tok", "model": _base(d)["model"],
                                                       "prompts": ["the quick brown", "seven small"], "max_new_tokens": 6, "n_rounds": 1,
                                                       "stop_sequence": None, "temperature": 0.0,
                                                       "engine": {"max_seqs": 4, "page_size": 8, "max_pages": 32, "max_pages_per_seq": 4, "max_rounds": 4},
                                                       "trainer": {"require_accelerator": False, "tracker": {"type": "noop"}, "log_dir": f"{d}/logs",
                                                                   "mp": "f32"}}))
    out = capsys.readouterr().out
    assert "Generated text for 0" in out and "Generated text for 1" in out

    # ---- viz_logprobs writes the page
    vcfg = {"checkpoint_path": ck, "path": f"{d}/lp.html", "data": _base(d)["data"], "model": _base(d)["model"], "num_docs": 4,
            "trainer": {"require_accelerator": False, "tracker": {"type": "noop"}, "log_dir": f"{d}/logs", "per_device_eval_parallelism": 4}}
    viz_logprobs.main(C.decode(viz_logprobs.VizLmConfig, vcfg))
    assert "<span" in open(f"{d}/lp.html").read()

    # ---- lora_lm on the exported weights, writing an adapter
    lcfg = {"initialize_from_hf": f"{d}/hf", "data": _base(d)["data"], "lora": {"r": 4, "alpha": 8.0},
            "trainer": dict(_base(d, 2)["trainer"], id="lora"), "optimizer": {"learning_rate": 1e-3, "warmup": 0.0},
            "peft_save_path": f"{d}/peft", "hf_save_steps": 2}
    lora_lm.main(C.decode(lora_lm.LoraLmConfig, lcfg))
    saved = [os.path.join(r, f) for r, _, fs in os.walk(f"{d}/peft") for f in fs]
    assert any(f.endswith("adapter_config.json") for f in saved), saved


def test_sft_on_chat_data_from_the_exported_weights(workdir, monkeypatch):
    """Runs after ``test_chain`` (it fine-tunes the Hugging Face directory that test exported)."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    if not os.path.exists(f"{d}/hf/config.json"):
        pytest.skip("needs the export of test_chain")
    from levanter_b200.main import sft

    rng = np.random.default_rng(1)
    words = "the quick brown fox jumps over the lazy dog".split()
    with open(f"{d}/chat.jsonl", "w") as f:
        for _ in range(64):
            q, a = " ".join(rng.choice(words, 5)), " ".join(rng.choice(words, 6))
            f.write(json.dumps({"messages": [{"role": "user", "content": q}, {"role": "assistant", "content": a}]}) + "\n")
    cfg = {"initialize_from_hf": f"{d}/hf", "model_name_or_path": f"{d}/hf", "tokenizer": f"{d}/tok", "max_seq_len": 32,
           "dataset_type": "chat_jsonl", "chat_train_urls": [f"{d}/chat.jsonl"], "supervised_data": {"cache_dir": f"{d}/sft_cache"},
           "trainer": dict(_base(d, 2)["trainer"], id="sft"), "optimizer": {"learning_rate": 1e-4, "warmup": 0.0},
           "hf_save_path": f"{d}/sft_hf", "hf_save_steps": 2}
    sft.train(C.decode(sft.SFTConfig, cfg))
    saved = [os.path.join(r, f) for r, _, fs in os.walk(f"{d}/sft_hf") for f in fs]
    assert any(f.endswith(".safetensors") for f in saved), saved


def test_sft_mixture_of_two_chat_sets(workdir, monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    if not os.path.exists(f"{d}/hf/config.json"):
        pytest.skip("needs the export of test_chain")
    from levanter_b200.main import sft_mixture

    rng = np.random.default_rng(2)
    words = "seven small birds sing near a quiet river at dawn".split()
    for name in ("a", "b"):
        with open(f"{d}/chat_{name}.jsonl", "w") as f:
            for _ in range(40):
                q, a = " ".join(rng.choice(words, 4)), " ".join(rng.choice(words, 5))
                f.write(json.dumps({"messages": [{"role": "user", "content": q}, {"role": "assistant", "content": a}]}) + "\n")
    cfg = {"initialize_from_hf": f"{d}/hf", "model_name_or_path": f"{d}/hf", "tokenizer": f"{d}/tok", "max_seq_len": 32,
           "dataset_type": "chat_jsonl", "mixture_block_size": 16, "mixture_weights": {"a": 0.75, "b": 0.25},
           "supervised_data": {"a": {"cache_dir": f"{d}/mix_cache_a", "train_urls": [f"{d}/chat_a.jsonl"]},
                               "b": {"cache_dir": f"{d}/mix_cache_b", "train_urls": [f"{d}/chat_b.jsonl"]}},
           "trainer": dict(_base(d, 2)["trainer"], id="sftmix"), "optimizer": {"learning_rate": 1e-4, "warmup": 0.0}}
    sft_mixture.train(C.decode(sft_mixture.SFTMixtureConfig, cfg))
    assert os.path.isdir(f"{d}/mix_cache_a") and os.path.isdir(f"{d}/mix_cache_b")


def test_inference_repl_loads_chats_and_runs_a_batch_file(workdir, monkeypatch, capsys):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    if not os.path.exists(f"{d}/hf/config.json"):
        pytest.skip("needs the export of test_chain")
    import transformers

    from levanter_b200.main import inference_repl as R

    # the chat routes need a chat template; give the tiny tokenizer a minimal one
    tok = transformers.AutoTokenizer.from_pretrained(f"{d}/tok")
    tok.chat_template = "{% for m in messages %}{{ m['role'] }}: {{ m['content'] }}\n{% endfor %}{% if add_generation_prompt %}assistant:{% endif %}"
    tok.save_pretrained(f"{d}/tok_chat")
    cfg = C.decode(R.InferenceReplConfig, {"model": _base(d)["model"], "tokenizer": f"{d}/tok_chat", "max_tokens": 5, "temperature": 0.0,
                                          "trainer": {"require_accelerator": False, "tracker": {"type": "noop"}, "log_dir": f"{d}/logs", "mp": "f32"}})
    cfg.trainer.initialize()
    ctx = R.ReplContext(cfg)
    try:
        ctx.execute("load", f"{d}/hf")
        resp = ctx.execute("chat", "the quick brown")
        assert resp["usage"]["completion_tokens"] >= 1 and isinstance(resp["choices"][0]["message"]["content"], str)
        with open(f"{d}/batch.jsonl", "w") as f:
            f.write(json.dumps({"prompt": "seven small birds"}) + "\n")
            f.write(json.dumps({"messages": [{"role": "user", "content": "a quiet river"}]}) + "\n")
        outs = ctx.execute("batch", f"{d}/batch.jsonl")
        assert len(outs) == 2 and all(o["choices"] for o in outs)
        ctx.execute("nonsense")
        assert "Unknown command" in capsys.readouterr().out
    finally:
        ctx.execute("unload")
        if ctx.server is not None:
            ctx.server.shutdown() if hasattr(ctx.server, "shutdown") else None


def test_train_lm_on_a_staged_mixture_with_ema_skip_step_and_gpt2(workdir, monkeypatch):
    """A second training configuration end to end: GPT-2 family, a two-source mixture whose weights change at a step boundary,
    exponential moving average of the weights, the skip-step guard, tagged evaluation during the run."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    from levanter_b200.checkpoint import discover_latest_checkpoint
    from levanter_b200.main import train_lm

    cfg = yaml.safe_load(f"""
data:
  tokenizer: {d}/tok
  cache_dir: {d}/mix_lm_cache
  mixture_block_size: 8
  configs:
    first:
      train_urls: ["{d}/shard0.jsonl"]
      validation_urls: ["{d}/shard1.jsonl"]
      tags: [alpha]
    second:
      train_urls: ["{d}/shard1.jsonl"]
      validation_urls: ["{d}/shard0.jsonl"]
      tags: [beta]
  train_weights:
    - [0, {{first: 1.0, second: 0.0}}]
    - [2, {{first: 0.25, second: 0.75}}]
model:
  type: gpt2
  seq_len: 32
  hidden_dim: 32
  num_layers: 2
  num_heads: 2
  gradient_checkpointing: false
trainer:
  id: mixrun
  num_train_steps: 4
  train_batch_size: 8
  require_accelerator: false
  tracker: {{type: noop}}
  log_dir: {d}/logs
  steps_per_eval: 2
  max_eval_batches: 1
  model_averaging: {{type: ema, beta: 0.9}}
  checkpointer:
    base_path: {d}/ckpt
    save_interval: 10h
optimizer:
  learning_rate: 1.0e-3
  warmup: 0.0
  skip_bad_steps: true
""")
    train_lm.main(C.decode(train_lm.TrainLmConfig, cfg))
    assert discover_latest_checkpoint(f"{d}/ckpt/mixrun") is not None
    assert os.path.isdir(f"{d}/mix_lm_cache/first/train") and os.path.isdir(f"{d}/mix_lm_cache/second/train")


_FAMILIES = {
    "mistral": {"type": "mistral", "seq_len": 32, "hidden_dim": 32, "intermediate_dim": 64, "num_layers": 2, "num_heads": 2, "num_kv_heads": 1},
    "mixtral": {"type": "mixtral", "seq_len": 32, "hidden_dim": 32, "intermediate_dim": 64, "num_layers": 2, "num_heads": 2, "num_kv_heads": 2,
                "n_routed_experts": 4, "num_experts_per_tok": 2},
    "gemma2": {"type": "gemma2", "seq_len": 32, "hidden_dim": 32, "intermediate_dim": 64, "num_layers": 2, "num_heads": 2, "num_kv_heads": 1,
               "head_dim": 16},
    "qwen3": {"type": "qwen3", "seq_len": 32, "hidden_dim": 32, "intermediate_dim": 64, "num_layers": 2, "num_heads": 2, "num_kv_heads": 1,
              "head_dim": 16},
    "olmo2": {"type": "olmo2", "seq_len": 32, "hidden_dim": 32, "intermediate_dim": 64, "num_layers": 2, "num_heads": 2, "num_kv_heads": 2},
    "gated_deltanet": {"type": "gated_deltanet", "seq_len": 32, "hidden_dim": 32, "num_layers": 2, "num_heads": 2, "head_k_dim": 16, "head_v_dim": 16},
    "gpt2_hyena": {"type": "gpt2_hyena", "num_layers": 2, "hyena": {"seq_len": 32, "hidden_dim": 32, "filter_order": 8}},
}


@pytest.mark.parametrize("family", sorted(_FAMILIES))
def test_every_model_family_trains_through_the_entry_point(workdir, monkeypatch, family):
    """Two optimizer steps and an evaluation of each family through ``train_lm`` (configuration decoding, the trainer, the
    sharded engine's single-process path, checkpointing)."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    from levanter_b200.checkpoint import discover_latest_checkpoint
    from levanter_b200.main import train_lm

    cfg = _base(d, 2)
    cfg["model"] = dict(_FAMILIES[family], gradient_checkpointing=False)
    cfg["trainer"]["id"] = f"fam_{family}"
    cfg["trainer"]["steps_per_eval"] = 2
    train_lm.main(C.decode(train_lm.TrainLmConfig, cfg))
    assert discover_latest_checkpoint(f"{d}/ckpt/fam_{family}") is not None


@pytest.mark.parametrize("opt", ["adam", "adopt", "cautious", "kron", "lion", "mars", "mini", "muon", "rmsprop", "scion", "soap", "sophia-h"])
def test_every_optimizer_trains_through_the_entry_point(workdir, monkeypatch, opt):
    """Three steps of a tiny Llama with each registered optimizer, configured the way a YAML file would."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    from levanter_b200.main import train_lm

    cfg = _base(d, 3)
    cfg["trainer"]["id"] = f"opt_{opt.replace('-', '_')}"
    cfg["optimizer"] = {"type": opt, "learning_rate": 1e-3, "warmup": 0.0}
    losses = []
    orig = train_lm.Trainer.train

    def spy(self, state, loader, *a, **k):
        self.add_hook(lambda info: losses.append(float(info.loss)), every=1)
        return orig(self, state, loader, *a, **k)

    monkeypatch.setattr(train_lm.Trainer, "train", spy)
    train_lm.main(C.decode(train_lm.TrainLmConfig, cfg))
    assert len(losses) >= 3 and all(np.isfinite(losses)), losses  # (hooks also run once more, forced, after the last step)


def test_two_process_launch_through_torchrun_and_resume_on_one(workdir):
    """The documented launch line on a CPU host: two processes (gloo), sharded state, one checkpoint; then the same run continues
    as a single process from that checkpoint."""
    import subprocess
    import sys

    d = str(workdir)
    cfg = _base(d, 3)
    cfg["trainer"]["id"] = "launch2"
    path = f"{d}/launch2.yaml"
    yaml.safe_dump(cfg, open(path, "w"))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29611",
           "-m", "levanter_b200.main.train_lm", "--config_path", path]
    r = subprocess.run(cmd, env=env, cwd=d, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    from levanter_b200.checkpoint import discover_latest_checkpoint

    ck = discover_latest_checkpoint(f"{d}/ckpt/launch2")
    assert ck is not None and ck.endswith("step-2"), ck
    r = subprocess.run([sys.executable, "-m", "levanter_b200.main.train_lm", "--config_path", path, "--trainer.num_train_steps", "5"], env=env, cwd=d,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert discover_latest_checkpoint(f"{d}/ckpt/launch2").endswith("step-4")
    assert "Resuming" in r.stderr or "esum" in r.stderr or "step-2" in r.stderr


def test_train_lm_starts_from_hugging_face_weights_and_from_a_checkpoint(workdir, monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    if not os.path.exists(f"{d}/hf/config.json"):
        pytest.skip("needs the export of test_chain")
    from levanter_b200.checkpoint import discover_latest_checkpoint
    from levanter_b200.main import train_lm

    cfg = _base(d, 2)
    cfg["trainer"]["id"] = "from_hf"
    cfg.update(initialize_from_hf=f"{d}/hf", use_hf_model_config=True)
    train_lm.main(C.decode(train_lm.TrainLmConfig, cfg))
    assert discover_latest_checkpoint(f"{d}/ckpt/from_hf") is not None
    cfg = _base(d, 2)
    cfg["trainer"]["id"] = "warm"
    cfg["trainer"]["initialize_from"] = discover_latest_checkpoint(f"{d}/ckpt/chain")
    train_lm.main(C.decode(train_lm.TrainLmConfig, cfg))
    assert discover_latest_checkpoint(f"{d}/ckpt/warm") is not None


@pytest.mark.parametrize("fmt", ["chat", "supervised"])
def test_train_lm_on_chat_and_supervised_formats_with_packing(workdir, monkeypatch, fmt):
    """The two other dataset formats through ``train_lm``: chat transcripts (assistant turns carry the loss, a template with a
    generation block) and prompt / response pairs, both packed several examples to a sequence."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    import transformers

    from levanter_b200.checkpoint import discover_latest_checkpoint
    from levanter_b200.main import train_lm

    tok = transformers.AutoTokenizer.from_pretrained(f"{d}/tok")
    tok.chat_template = ("{% for m in messages %}{% if m['role'] == 'assistant' %}{% generation %}{{ m['content'] }}</s>{% endgeneration %}"
                         "{% else %}{{ m['role'] }}: {{ m['content'] }}\n{% endif %}{% endfor %}")
    tok.save_pretrained(f"{d}/tok_gen")
    rng = np.random.default_rng(3)
    words = "the quick brown fox jumps over the lazy dog".split()
    for split in ("train", "val"):
        with open(f"{d}/{fmt}_{split}.jsonl", "w") as f:
            for _ in range(96):
                q, a = " ".join(rng.choice(words, 4)), " ".join(rng.choice(words, 5))
                row = {"messages": [{"role": "user", "content": q}, {"role": "assistant", "content": a}]} if fmt == "chat" else {"prompt": q, "response": a}
                f.write(json.dumps(row) + "\n")
    cfg = _base(d, 2)
    cfg["trainer"]["id"] = f"fmt_{fmt}"
    cfg["data"] = {"tokenizer": f"{d}/tok_gen", "cache_dir": f"{d}/cache_{fmt}", "train_urls": [f"{d}/{fmt}_train.jsonl"],
                   "validation_urls": [f"{d}/{fmt}_val.jsonl"],
                   "format": {"type": "chat"} if fmt == "chat" else {"type": "supervised", "input_field": "prompt", "output_field": "response"}}
    train_lm.main(C.decode(train_lm.TrainLmConfig, cfg))
    assert discover_latest_checkpoint(f"{d}/ckpt/fmt_{fmt}") is not None


def test_eval_lm_on_the_exported_hugging_face_weights_with_every_analysis(workdir, monkeypatch, capsys):
    """Runs after ``test_chain``: the exported directory gives the same validation loss as the checkpoint it came from, and the
    entropy / top-2 gap / parameter statistics options log their histograms."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    if not os.path.exists(f"{d}/hf/config.json"):
        pytest.skip("needs the export of test_chain")
    import levanter_b200.tracker as T
    from levanter_b200.checkpoint import discover_latest_checkpoint
    from levanter_b200.main import eval_lm
    from levanter_b200.tracker.histogram import Histogram

    class Recorder(T.NoopTracker):
        def __init__(self):
            self.logged = {}

        def log(self, metrics, *, step, commit=None):
            self.logged.update(metrics)

    base = _base(d, 4)
    common = {"data": base["data"], "model": base["model"], "trainer": dict(base["trainer"], id="evalhf", max_eval_batches=2, per_device_eval_parallelism=4)}
    rec = Recorder()
    from levanter_b200.trainer import TrainerConfig

    monkeypatch.setattr(TrainerConfig, "_make_tracker", lambda self: rec)  # the entry point installs the configured tracker
    from_hf = eval_lm.main(C.decode(eval_lm.EvalLmConfig, dict(common, hf_checkpoint=f"{d}/hf", log_entropy=True, log_top2_gap=True, log_param_stats=True)))
    assert from_hf["eval/loss"] > 0 and "Loss:" in capsys.readouterr().out
    assert any(k.startswith("eval/") and k.endswith("bpb") for k in from_hf), sorted(from_hf)
    ent = [v for k, v in rec.logged.items() if k.startswith("analysis/") and k.endswith("/entropy")]
    gap = [v for k, v in rec.logged.items() if k.endswith("/top2_gap")]
    assert ent and gap and all(isinstance(h, Histogram) and float(h.num) > 0 for h in ent + gap)
    assert float(ent[0].min) >= 0 and float(ent[0].max) <= np.log(300) + 1e-3  # an entropy is within [0, log(vocabulary)]
    assert any(k.startswith("params/norm/") for k in rec.logged) and any(k.startswith("params/hist/") for k in rec.logged)

    ck = discover_latest_checkpoint(f"{d}/ckpt/chain")
    from_ckpt = eval_lm.main(C.decode(eval_lm.EvalLmConfig, dict(common, checkpoint_path=ck)))
    assert from_ckpt["eval/loss"] == pytest.approx(from_hf["eval/loss"], rel=1e-4)
    on_train = eval_lm.main(C.decode(eval_lm.EvalLmConfig, dict(common, checkpoint_path=ck, eval_on_train=True)))
    assert on_train["eval/loss"] > 0 and on_train["eval/loss"] != pytest.approx(from_ckpt["eval/loss"], rel=1e-6)


def test_inference_repl_command_line_mode_and_interactive_session(workdir, monkeypatch, capsys):
    """Runs after the REPL test above (it uses the tokenizer with a chat template saved there)."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    if not os.path.exists(f"{d}/hf/config.json") or not os.path.exists(f"{d}/tok_chat"):
        pytest.skip("needs the export of test_chain and the chat tokenizer")
    from levanter_b200.main import inference_repl as R

    base = {"model": _base(d)["model"], "tokenizer": f"{d}/tok_chat", "max_tokens": 4, "temperature": 0.0,
            "trainer": {"require_accelerator": False, "tracker": {"type": "noop"}, "log_dir": f"{d}/logs", "mp": "f32"}}
    # one command from the command line: load the checkpoint, run it, exit
    R.main(C.decode(R.InferenceReplConfig, dict(base, checkpoint=f"{d}/hf", command="chat", args="'the quick brown fox'")))
    out = capsys.readouterr().out
    assert f"Loaded {d}/hf" in out and "tokens]" in out

    # an interactive session: help, a failing command that must not end it, load, a two-turn chat, unload, quit
    lines = iter(["help", "", "load /does/not/exist", f"load {d}/hf", "chat", "the lazy dog", "seven small birds", "", "chat 'a quiet river'",
                  "unload", "chat hello", "quit", "never reached"])
    monkeypatch.setattr("builtins.input", lambda prompt="": next(lines))
    R.main(C.decode(R.InferenceReplConfig, base))
    out = capsys.readouterr().out
    assert out.count("Commands:") >= 2 and "error:" in out and f"Loaded {d}/hf" in out
    assert out.count("tokens]") == 3 and "Model unloaded" in out and "Load a model first" in out
    assert next(lines) == "never reached"

    # end of input ends the session too
    def eof(prompt=""):
        raise EOFError

    monkeypatch.setattr("builtins.input", eof)
    R.main(C.decode(R.InferenceReplConfig, base))


def test_train_lm_for_a_number_of_epochs_stops_when_the_data_ends(workdir, monkeypatch):
    """``epoch: 2`` repeats the training windows twice and no more: the run ends there although ``num_train_steps`` is larger,
    and its last step is checkpointed."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(workdir)
    d = str(workdir)
    from levanter_b200.checkpoint import _load_metadata, discover_latest_checkpoint
    from levanter_b200.main import train_lm

    cfg = _base(d, 10_000)
    cfg["trainer"]["id"] = "epochs"
    cfg["epoch"] = 2
    built = C.decode(train_lm.TrainLmConfig, cfg)
    windows = asyncio_len(built.data.train_set(32, key=0))
    assert windows >= 8
    train_lm.main(built)
    ck = discover_latest_checkpoint(f"{d}/ckpt/epochs")
    assert ck is not None
    steps_run = _load_metadata(ck)["step"] + 1
    assert steps_run == (2 * windows) // 8 or steps_run == -(-(2 * windows) // 8)  # two passes at 8 sequences per step (a short last batch is padded)


def asyncio_len(ds):
    import asyncio

    return asyncio.run(ds.async_len())
