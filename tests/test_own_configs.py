"""Every YAML file shipped under config/ decodes into the config class of the entry point it is written for."""
import glob
import os

import pytest

from levanter_b200 import config as C

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "config")


def _class_for(name):
    if name.startswith("whisper"):
        from levanter_b200.main.train_asr import TrainASRConfig as T
    elif name.startswith("lora"):
        from levanter_b200.main.lora_lm import LoraLmConfig as T
    elif name.startswith("sft"):
        from levanter_b200.main.sft import SFTConfig as T
    elif name.startswith("sample"):
        from levanter_b200.main.sample_lm import SampleLmConfig as T
    elif name.startswith("eval_harness"):
        from levanter_b200.eval_harness import EvalHarnessMainConfig as T
    else:
        from levanter_b200.main.train_lm import TrainLmConfig as T
    return T


@pytest.mark.parametrize("path", sorted(glob.glob(f"{ROOT}/*.yaml")), ids=os.path.basename)
def test_config_decodes(path):
    cfg = C.decode(_class_for(os.path.basename(path)), C.load_yaml(path))
    assert cfg is not None


def test_there_are_configs():
    assert len(glob.glob(f"{ROOT}/*.yaml")) >= 15


def test_flagship_config_is_llama2_7b():
    from levanter_b200.main.train_lm import TrainLmConfig

    cfg = C.decode(TrainLmConfig, C.load_yaml(f"{ROOT}/llama2_7b_b200.yaml"))
    m = cfg.model
    assert (m.hidden_dim, m.intermediate_dim, m.num_layers, m.num_heads, m.seq_len) == (4096, 11008, 32, 32, 4096)
    assert abs(m.total_trainable_params(32000) - 6.74e9) / 6.74e9 < 0.01


def test_packaging_metadata_names_real_packages_scripts_and_sources():
    """``pyproject.toml`` builds the package that is in the tree: the version attribute, the console scripts' targets and the
    kernel sources it ships all exist."""
    import glob
    import importlib
    import os
    import tomllib

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    meta = tomllib.load(open(os.path.join(root, "pyproject.toml"), "rb"))
    assert meta["project"]["name"] == "levanter_b200"
    mod, attr = meta["tool"]["setuptools"]["dynamic"]["version"]["attr"].rsplit(".", 1)
    assert isinstance(getattr(importlib.import_module(mod), attr), str)
    for target in meta["project"]["scripts"].values():
        module, func = target.split(":")
        assert callable(getattr(importlib.import_module(module), func)), target
    for pkg, patterns in meta["tool"]["setuptools"]["package-data"].items():
        base = os.path.join(root, *pkg.split("."))
        for pattern in patterns:
            assert glob.glob(os.path.join(base, pattern)), (pkg, pattern)
    from setuptools import find_packages

    found = set(find_packages(root, include=meta["tool"]["setuptools"]["packages"]["find"]["include"]))
    on_disk = {os.path.relpath(d, root).replace(os.sep, ".") for d, _, files in os.walk(os.path.join(root, "levanter_b200")) if "__init__.py" in files}
    assert found == on_disk and "levanter_b200.ops" in found and "levanter_b200.main" in found
