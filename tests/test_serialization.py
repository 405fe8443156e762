"""Checkpoint leaves on disk: tree round trips with scalars / None / named tuples, missing leaves, the zarr layout, corruption
(modelled on the reference's test_tensorstore_serialization.py and the fault tests: a removed or damaged leaf is an error, or is
skipped when partial checkpoints are allowed)."""
import json
import os
import shutil
from typing import NamedTuple

import numpy as np
import pytest
import torch

from levanter_b200 import tensorstore_serialization as tss
from levanter_b200.store.zarr_array import ZarrArray


class _Pair(NamedTuple):
    mu: dict
    count: int


def _tree():
    g = torch.Generator().manual_seed(0)
    return {"model": {"a.weight": torch.randn(5, 3, generator=g), "a.bias": torch.randn(3, generator=g).bfloat16()},
            "opt": _Pair({"a.weight": torch.randn(5, 3, generator=g)}, 7), "step": 12, "lr": 0.25, "flag": True, "nothing": None,
            "arr": np.arange(6, dtype=np.int64).reshape(2, 3)}


def test_tree_round_trip_with_scalars_none_and_named_tuples(tmp_path):
    tree = _tree()
    tss.tree_serialize_leaves_tensorstore(str(tmp_path), tree)
    like = {"model": {"a.weight": torch.zeros(5, 3), "a.bias": torch.zeros(3, dtype=torch.bfloat16)}, "opt": _Pair({"a.weight": torch.zeros(5, 3)}, 0),
            "step": 0, "lr": 0.0, "flag": False, "nothing": None, "arr": np.zeros((2, 3), dtype=np.int64)}
    back = tss.tree_deserialize_leaves_tensorstore(str(tmp_path), like)
    assert torch.equal(back["model"]["a.weight"], tree["model"]["a.weight"]) and back["model"]["a.bias"].dtype == torch.bfloat16
    assert torch.equal(back["model"]["a.bias"], tree["model"]["a.bias"])
    assert isinstance(back["opt"], _Pair) and back["opt"].count == 7 and torch.equal(back["opt"].mu["a.weight"], tree["opt"].mu["a.weight"])
    assert back["step"] == 12 and back["lr"] == 0.25 and back["flag"] is True and back["nothing"] is None
    assert np.array_equal(back["arr"], tree["arr"])


def test_leaf_is_a_zarr_v2_array_with_dot_separated_chunks(tmp_path):
    tss.tree_serialize_leaves_tensorstore(str(tmp_path), {"w": torch.arange(12, dtype=torch.float32).reshape(3, 4)})
    leaf = [os.path.join(r, d) for r, ds, _ in os.walk(tmp_path) for d in ds if os.path.exists(os.path.join(r, d, ".zarray"))]
    assert len(leaf) == 1
    meta = json.load(open(os.path.join(leaf[0], ".zarray")))
    assert meta["zarr_format"] == 2 and meta["shape"] == [3, 4] and meta["dtype"] in ("<f4", "float32") and meta.get("dimension_separator", ".") == "."
    assert any(f.replace(".", "").isdigit() for f in os.listdir(leaf[0]))  # chunk files named like 0.0
    assert torch.equal(ZarrArray.open(leaf[0]).read_tensor(), torch.arange(12, dtype=torch.float32).reshape(3, 4))
    part = ZarrArray.open(leaf[0]).read_tensor([1, 1], [3, 3])
    assert torch.equal(part, torch.tensor([[5.0, 6.0], [9.0, 10.0]]))


def test_missing_leaf_is_an_error_unless_allowed(tmp_path):
    tss.tree_serialize_leaves_tensorstore(str(tmp_path), {"a": torch.ones(2), "b": torch.zeros(2)})
    victim = next(os.path.join(r, d) for r, ds, _ in os.walk(tmp_path) for d in ds if d == "b")
    shutil.rmtree(victim)
    like = {"a": torch.zeros(2), "b": torch.full((2,), 5.0)}
    with pytest.raises(FileNotFoundError, match="b"):
        tss.tree_deserialize_leaves_tensorstore(str(tmp_path), like)
    back = tss.tree_deserialize_leaves_tensorstore(str(tmp_path), like, allow_missing=True)
    assert torch.equal(back["a"], torch.ones(2)) and torch.equal(back["b"], torch.full((2,), 5.0))


def test_damaged_chunk_is_detected(tmp_path):
    tss.tree_serialize_leaves_tensorstore(str(tmp_path), {"w": torch.randn(64, 64)})
    leaf = next(os.path.join(r, d) for r, ds, _ in os.walk(tmp_path) for d in ds if os.path.exists(os.path.join(r, d, ".zarray")))
    chunk = next(os.path.join(leaf, f) for f in os.listdir(leaf) if not f.startswith("."))
    data = bytearray(open(chunk, "rb").read())
    open(chunk, "wb").write(bytes(data[: len(data) // 2]))  # truncated file
    with pytest.raises(Exception):
        ZarrArray.open(leaf).read_tensor()


def test_stacked_reference_layout_for_layer_parameters(tmp_path):
    """Per-layer torch parameters are stored as one array stacked over layers, under the reference's key names."""
    from levanter_b200.models.llama import LlamaConfig

    m = LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=3, num_heads=2, num_kv_heads=2).build(50, seed=0)
    layouts = tss.layouts_of(m)
    params = {n: p.detach() for n, p in m.named_parameters()}
    tss.tree_serialize_leaves_tensorstore(str(tmp_path), {"model": params}, layouts=layouts)
    name = "transformer.layers.1.mlp.gate_proj.weight"
    key, layer = tss.reference_key_for(name)
    assert layer == 1 and "layers" in key
    got = tss.read_param(str(tmp_path), "model", name, layouts.get(name), tuple(params[name].shape))
    assert torch.equal(got, params[name])
    stacked = ZarrArray.open(tss._fs_path(str(tmp_path), f"model.{key}"))
    assert stacked.shape[0] == 3


def test_model_optimizer_state_key_and_step_after_a_few_updates(tmp_path):
    """A tuple of (parameters, optimizer state, key, step) after three Adam steps comes back exactly, into a tree built from
    another seed."""
    from levanter_b200.optim import transforms as T

    def make(seed):
        g = torch.Generator().manual_seed(seed)
        params = {"l1.weight": torch.randn(4, 2, generator=g), "l1.bias": torch.randn(4, generator=g), "l2.weight": torch.randn(1, 4, generator=g)}
        opt = T.chain(T.scale_by_adam(0.9, 0.95, 1e-8), T.scale(-1e-2))
        return params, opt, opt.init(params), torch.tensor([0, seed], dtype=torch.int64)

    params, opt, state, key = make(0)
    first = {k: v.clone() for k, v in params.items()}
    for i in range(3):
        grads = {k: torch.full_like(v, 0.1 * (i + 1)) for k, v in params.items()}
        updates, state = opt.update(grads, state, params)
        params = {k: params[k] + updates[k] for k in params}
    assert not torch.equal(params["l1.weight"], first["l1.weight"])
    tss.tree_serialize_leaves_tensorstore(str(tmp_path), (params, state, key, 3))
    other_params, _, other_state, other_key = make(1)
    r_params, r_state, r_key, r_step = tss.tree_deserialize_leaves_tensorstore(str(tmp_path), (other_params, other_state, other_key, 0))
    assert r_step == 3 and torch.equal(r_key, key)
    for k in params:
        assert torch.equal(r_params[k], params[k])
    for (pa, a), (pb, b) in zip(tss.leaf_key_paths(r_state), tss.leaf_key_paths(state)):
        assert pa == pb and torch.equal(torch.as_tensor(a), torch.as_tensor(b))
    assert type(r_state) is type(state)


def test_dataclass_nodes_none_leaves_and_leaves_missing_on_disk(tmp_path):
    import dataclasses
    from typing import Any

    @dataclasses.dataclass
    class Module:
        a: Any
        b: Any

    tss.tree_serialize_leaves_tensorstore(str(tmp_path / "m"), Module(a=None, b=torch.zeros(10)))
    assert sorted(os.listdir(tmp_path / "m")) == ["b"]  # nothing is written for a None leaf
    back = tss.tree_deserialize_leaves_tensorstore(str(tmp_path / "m"), Module(a=None, b=torch.ones(10)))
    assert isinstance(back, Module) and back.a is None and torch.equal(back.b, torch.zeros(10))
    wants_a = Module(a=torch.full((10,), 4.0), b=torch.ones(10))
    with pytest.raises(FileNotFoundError):
        tss.tree_deserialize_leaves_tensorstore(str(tmp_path / "m"), wants_a)
    partial = tss.tree_deserialize_leaves_tensorstore(str(tmp_path / "m"), wants_a, allow_missing=True)
    assert torch.equal(partial.a, torch.full((10,), 4.0)) and torch.equal(partial.b, torch.zeros(10))


def test_saves_into_the_same_directory_do_not_overlap(tmp_path):
    """The same step saved again while the first save is still being written: the second waits for the first (it starts by clearing
    each leaf's directory), saves into other directories go on side by side, and the last values win."""
    manager = tss.AsyncSerializer(max_workers=8)
    commits = []
    for i in range(12):
        tree = {f"w{j}": torch.full((64, 64), float(i)) for j in range(6)}
        tss.tree_serialize_leaves_tensorstore(str(tmp_path / "same"), tree, manager, commit_callback=lambda i=i: commits.append(i))
        tss.tree_serialize_leaves_tensorstore(str(tmp_path / f"other-{i}"), {"w": torch.full((8,), float(i))}, manager)
    manager.wait_until_finished()
    assert commits == list(range(12))
    back = tss.tree_deserialize_leaves_tensorstore(str(tmp_path / "same"), {f"w{j}": torch.zeros(64, 64) for j in range(6)})
    assert all(float(v.min()) == float(v.max()) == 11.0 for v in back.values())
    assert float(tss.tree_deserialize_leaves_tensorstore(str(tmp_path / "other-3"), {"w": torch.zeros(8)})["w"][0]) == 3.0
