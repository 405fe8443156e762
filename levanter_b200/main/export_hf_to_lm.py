"""Import a Hugging Face checkpoint and save it as a checkpoint of this framework
(src/levanter/main/export_hf_to_lm.py:26-121)."""
from __future__ import annotations

import logging
import time
from dataclasses import dataclass, field
from typing import Optional, Union

import torch

from levanter_b200 import config as lev_config
from levanter_b200.checkpoint import save_checkpoint
from levanter_b200.compat.hf_checkpoints import HFCompatConfig, RepoRef, load_tokenizer
from levanter_b200.config import parse_dtype
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig
from levanter_b200 import tensorstore_serialization as tss

logger = logging.getLogger(__name__)


@dataclass
class ImportHfConfig:
    hf_checkpoint: Union[str, RepoRef]
    output_path: str
    model: LmConfig = field(default_factory=LlamaConfig)
    use_hf_model_config: bool = True
    tokenizer: Optional[str] = None
    dtype: Optional[str] = "bfloat16"
    resize_vocab_to_match_tokenizer: bool = True


def main(config: ImportHfConfig):
    logging.basicConfig(level=logging.INFO)
    t0 = time.time()
    ref = config.hf_checkpoint if isinstance(config.hf_checkpoint, RepoRef) else RepoRef.from_string(str(config.hf_checkpoint))
    assert isinstance(config.model, HFCompatConfig), "the model must have a Hugging Face converter"
    converter = config.model.hf_checkpoint_converter().replaced(reference_checkpoint=ref)
    if config.tokenizer is not None:
        converter = converter.replaced(tokenizer=load_tokenizer(config.tokenizer))
    dtype = parse_dtype(config.dtype) if config.dtype else None
    model = converter.load_pretrained(ref=ref, config=None if config.use_hf_model_config else config.model, dtype=dtype,
                                      resize_vocab_to_match_tokenizer=config.resize_vocab_to_match_tokenizer, device="cpu")
    n = sum(p.numel() for p in model.parameters())
    logger.info(f"loaded {n / 1e6:.1f}M parameters in {time.time() - t0:.1f}s; saving to {config.output_path}")
    tree = {"model": {k: v.detach() for k, v in model.named_parameters()}}
    save_checkpoint(tree, step=0, checkpoint_path=config.output_path, layouts=tss.layouts_of(model))
    logger.info(f"done in {time.time() - t0:.1f}s")


if __name__ == "__main__":
    lev_config.main(main)()
