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
