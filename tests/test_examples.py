"""The instruction-tuning example runs end to end on a tiny random model (full and LoRA)."""
import importlib.util
import json
import os
import sys

import pytest

from levanter_b200 import config as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_example():
    spec = importlib.util.spec_from_file_location("instruction_tuning", os.path.join(ROOT, "examples/instruction_tuning/instruction_tuning.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod  # dataclasses resolve string annotations through sys.modules
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.entry
@pytest.mark.parametrize("lora", [False, True])
def test_instruction_tuning_example(tmp_path, monkeypatch, lora):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    ex = _load_example()
    d = str(tmp_path)
    with open(f"{d}/data.jsonl", "w") as f:
        for i in range(24):
            f.write(json.dumps({"instruction": f"{10 + i} {11 + i}", "input": "" if i % 2 else f"{5 + i}", "output": f"{20 + i} {21 + i} {22 + i}"}) + "\n")
    cfg = {
        "data": f"{d}/data.jsonl", "data_cache_dir": f"{d}/cache", "max_tune_length": 32, "tokenizer": "passthrough", "vocab_size": 100,
        "prompts": {"prompt_input": "1 {instruction} 2 {input} 3", "prompt_no_input": "1 {instruction} 3"},
        "model": {"type": "llama", "seq_len": 32, "hidden_dim": 32, "intermediate_dim": 64, "num_layers": 1, "num_heads": 2, "num_kv_heads": 2},
        "trainer": {"num_train_steps": 3, "train_batch_size": 4, "require_accelerator": False, "tracker": {"type": "noop"},
                    "log_dir": f"{d}/logs", "id": "ex", "checkpointer": {"base_path": f"{d}/ckpt", "save_interval": "1h"}},
        "optimizer": {"learning_rate": 1e-3, "warmup": 0.0},
    }
    if lora:
        cfg["lora"] = {"r": 2, "alpha": 2.0, "target_modules": ["q_proj", "v_proj"]}
    info = ex.train(C.decode(ex.TrainArgs, cfg))
    assert info is not None and info.step == 2


def test_example_configs_decode():
    ex = _load_example()
    for name in ("alpaca_llama2.yaml", "alpaca_lora_llama2.yaml"):
        C.decode(ex.TrainArgs, C.load_yaml(os.path.join(ROOT, "examples/instruction_tuning", name)))
