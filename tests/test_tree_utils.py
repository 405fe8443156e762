import os

import torch
import torch.nn as nn

from levanter_b200.utils.cloud_utils import temp_dir_before_upload
from levanter_b200.utils.torch_utils import parameter_count, tree_broadcast_to, zeros_like_tree
from levanter_b200.utils.tree_utils import inference_mode, key_path_to_str, leaf_key_paths, pack_pytree, unpack_pytree


def test_pack_unpack_round_trip():
    tree = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b": [torch.ones(4, dtype=torch.int32), 7], "c": ()}
    offsets, flat = pack_pytree(tree)
    assert flat.shape == (10,)
    back = unpack_pytree(offsets, flat)
    assert torch.equal(back["a"], tree["a"]) and back["b"][0].dtype == torch.int32 and back["b"][1] == 7


def test_leaf_paths_and_inference_mode():
    m = nn.Sequential(nn.Linear(3, 4), nn.Dropout(0.5))
    paths = leaf_key_paths({"model": m, "step": 3})
    assert "model.0.weight" in paths and paths["step"] == 3
    assert key_path_to_str(("layers", 3, "weight")) == "layers.3.weight"
    inference_mode({"model": m}, True)
    assert not m[1].training
    inference_mode({"model": m}, False)
    assert m[1].training


def test_parameter_count_ties_counted_once():
    emb = nn.Embedding(10, 4)
    head = nn.Linear(4, 10, bias=False)
    head.weight = emb.weight
    assert parameter_count(nn.ModuleList([emb, head])) == 40


def test_zeros_and_broadcast():
    t = {"x": torch.ones(2), "y": (torch.ones(3), 1)}
    z = zeros_like_tree(t)
    assert float(z["x"].sum()) == 0 and z["y"][1] == 1
    assert tree_broadcast_to(True, t) == {"x": True, "y": (True, True)}


def test_temp_dir_before_upload(tmp_path):
    dest = str(tmp_path / "out")
    with temp_dir_before_upload(dest) as d:
        open(os.path.join(d, "f.txt"), "w").write("hi")
    assert open(os.path.join(dest, "f.txt")).read() == "hi"
