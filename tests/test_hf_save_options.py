"""Options of the Hugging Face export: the dtype of saved floating-point tensors, shard
sizes, and remote (fsspec) destinations (levanter_b200/compat/hf_checkpoints.py; scenarios after the reference's
tests/test_hf_checkpoints.py)."""
import glob
import json
import os
import uuid

import pytest
import torch

from levanter_b200.compat.hf_checkpoints import to_hf_state_dict
from levanter_b200.models.gpt2 import Gpt2Config

safetensors = pytest.importorskip("safetensors")
from safetensors import safe_open  # noqa: E402


def _tensors(directory):
    out = {}
    for f in glob.glob(os.path.join(directory, "*.safetensors")):
        with safe_open(f, framework="pt", device="cpu") as t:
            for k in t.keys():
                out[k] = t.get_tensor(k)
    return out


def test_floats_are_saved_in_the_requested_dtype(tmp_path):
    cfg = Gpt2Config(seq_len=32, hidden_dim=32, num_layers=1, num_heads=1)
    conv = cfg.hf_checkpoint_converter()
    model = cfg.build(100, seed=0)
    model.register_buffer("an_int_buffer", torch.tensor([-1, 0, 1, 2, 3], dtype=torch.int32))
    assert next(model.parameters()).dtype == torch.float32

    conv.save_pretrained(model, str(tmp_path / "bf16"), save_tokenizer=False, max_shard_size=int(10e9), dtype=torch.bfloat16)
    assert os.path.exists(tmp_path / "bf16" / "model.safetensors")
    t = _tensors(str(tmp_path / "bf16"))
    floats = {k: v for k, v in t.items() if v.is_floating_point()}
    assert floats and all(v.dtype == torch.bfloat16 for v in floats.values())
    assert any(k.endswith("wte.weight") for k in floats)
    assert json.load(open(tmp_path / "bf16" / "config.json"))["torch_dtype"] == "bfloat16"

    conv.save_pretrained(model, str(tmp_path / "plain"), save_tokenizer=False, max_shard_size=int(10e9))
    t32 = _tensors(str(tmp_path / "plain"))
    assert all(v.dtype == torch.float32 for v in t32.values() if v.is_floating_point())
    for k in floats:
        assert torch.allclose(t32[k], floats[k].float(), atol=1e-2, rtol=1e-2)

    # the converter writes exactly what ``to_hf_state_dict`` gives: parameters only, buffers stay behind
    sd = to_hf_state_dict(model, dtype=torch.bfloat16)
    assert set(sd) == set(t) and not any("buffer" in k for k in sd)


def test_save_to_an_fsspec_destination_in_small_shards_and_load_back(tmp_path):
    fsspec = pytest.importorskip("fsspec")
    fs = fsspec.filesystem("memory")
    path = f"memory://lvb/hf-save/{uuid.uuid4().hex}"
    cfg = Gpt2Config(seq_len=32, hidden_dim=32, num_layers=4, num_heads=1)
    conv = cfg.hf_checkpoint_converter()
    model = cfg.build(100, seed=4)
    conv.save_pretrained(model, path, max_shard_size=20_000, save_tokenizer=False)
    base = fs._strip_protocol(path)
    stored = {fs._strip_protocol(f) for f in fs.find(path)}
    shards = {f for f in stored if f.endswith(".safetensors")}
    assert len(shards) > 1 and f"{base}/config.json" in stored and f"{base}/model.safetensors.index.json" in stored
    for f in shards:
        assert fs.size(f) > 0
    index = json.loads(fs.cat(f"{base}/model.safetensors.index.json"))
    assert set(index["weight_map"].values()) == {os.path.basename(f) for f in shards}

    local = str(tmp_path / "model")
    fs.get(f"{base}/", local, recursive=True)
    back = type(conv)(type(cfg), reference_checkpoint=local).load_pretrained(resize_vocab_to_match_tokenizer=False)
    for (n, p), (_, q) in zip(model.named_parameters(), back.named_parameters()):
        assert torch.equal(p, q), n
    fs.rm(base, recursive=True)
