"""Convert a checkpoint of this framework into a Hugging Face directory (src/levanter/main/export_lm_to_hf.py:26-94)."""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Optional

import torch

from levanter_b200 import config as lev_config
from levanter_b200.checkpoint import load_checkpoint
from levanter_b200.compat.hf_checkpoints import HFCompatConfig, RepoRef, load_tokenizer
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig
from levanter_b200.parallel.mesh import local_device
from levanter_b200.trainer import TrainerConfig
from levanter_b200.utils.logging import init_logging

logger = logging.getLogger(__name__)


@dataclass
class ConvertLmConfig:
    checkpoint_path: str
    output_dir: str
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    upload_to_hf: Optional[RepoRef] = None
    model: LmConfig = field(default_factory=LlamaConfig)
    save_tokenizer: bool = True
    tokenizer: Optional[str] = None  # default: the tokenizer of the model's reference checkpoint
    override_vocab_size: Optional[int] = None
    config_overrides: Optional[dict] = None
    use_cpu: bool = False


def main(config: ConvertLmConfig):
    init_logging("logs", "export")
    assert isinstance(config.model, HFCompatConfig), "the model must have a Hugging Face converter"
    converter = config.model.hf_checkpoint_converter()
    tokenizer = converter.tokenizer if config.tokenizer is None else load_tokenizer(config.tokenizer)
    vocab_size = config.override_vocab_size or len(tokenizer)
    device = torch.device("cpu") if config.use_cpu else local_device()
    model = config.model.build(vocab_size, seed=0, device=device)
    model = load_checkpoint(model, config.checkpoint_path, subpath="model")
    if config.override_vocab_size:
        model = model.resize_vocab(len(tokenizer))
    converter = converter.replaced(tokenizer=tokenizer)
    if config.config_overrides:
        converter = converter.with_config_overrides(config.config_overrides)
    converter.save_pretrained(model, config.output_dir, upload_to_hf=config.upload_to_hf or False, save_tokenizer=config.save_tokenizer)
    logger.info(f"wrote {config.output_dir}")


if __name__ == "__main__":
    lev_config.main(main)()
