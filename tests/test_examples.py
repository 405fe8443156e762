"""The instruction-tuning example runs end to end on a tiny random model (full and LoRA)."""
import importlib.util
import json
import os
import sys

import pytest

from levanter_b200 import config as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_example(name="instruction_tuning", path="examples/instruction_tuning/instruction_tuning.py"):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, path))
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


@pytest.mark.entry
def test_word_problems_lora_example_trains_and_evaluates_by_generation(tmp_path, monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    ex = _load_example("word_problems_lora", "examples/word_problems_lora/word_problems_lora.py")
    assert ex.final_number("so she has 1,250 apples.\n#### 1,250") == "1250" and ex.final_number("3 then -4.5.") == "-4.5"
    assert ex.final_number("no digits here") is None
    d = str(tmp_path)
    for split, n in (("train", 24), ("test", 6)):
        with open(f"{d}/{split}.jsonl", "w") as f:
            for i in range(n):
                f.write(json.dumps({"question": f"{10 + i} {11 + i}", "answer": f"{20 + i} {21 + i}"}) + "\n")
    cfg = {
        "train_data": f"{d}/train.jsonl", "eval_data": f"{d}/test.jsonl", "data_cache_dir": f"{d}/cache", "prompt": "1 {question} 2",
        "max_tune_length": 32, "max_new_tokens": 4, "tokenizer": "passthrough", "vocab_size": 100,
        "model": {"type": "llama", "seq_len": 32, "hidden_dim": 32, "intermediate_dim": 64, "num_layers": 1, "num_heads": 2, "num_kv_heads": 2},
        "lora": {"r": 2, "alpha": 2.0, "target_modules": ["q_proj", "v_proj"]},
        "engine": {"max_seqs": 4, "page_size": 4, "max_pages_per_seq": 10, "compute_dtype": "float32", "max_rounds": 2},
        "trainer": {"num_train_steps": 3, "train_batch_size": 4, "require_accelerator": False, "tracker": {"type": "noop"},
                    "log_dir": f"{d}/logs", "id": "wp", "checkpointer": {"base_path": f"{d}/ckpt", "save_interval": "1h"}},
        "optimizer": {"learning_rate": 1e-3, "warmup": 0.0},
        "peft_save_path": f"{d}/peft",
    }
    info, report = ex.train(C.decode(ex.TrainArgs, cfg))
    assert info.step == 2
    assert report["eval/num_examples"] == 6 and 0.0 <= report["eval/exact_match"] <= 1.0
    assert len(report["answers"]) == 6 and 6 <= report["eval/generated_tokens"] <= 6 * 4  # more requests than engine slots
    assert os.path.exists(f"{d}/peft/adapter_config.json")
    C.decode(ex.TrainArgs, C.load_yaml(os.path.join(ROOT, "examples/word_problems_lora/gsm8k_llama2.yaml")))
