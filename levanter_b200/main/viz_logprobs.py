"""Write an HTML page colouring validation tokens by their log-probability under a checkpoint, optionally against a second
model (src/levanter/main/viz_logprobs.py:34-183)."""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Optional, Union

import torch

import levanter_b200 as lev
from levanter_b200 import config as lev_config
from levanter_b200.analysis.visualization import compute_and_diff_log_probs, compute_and_visualize_log_probs
from levanter_b200.data.loader import DataLoader
from levanter_b200.data.text import LMMixtureDatasetConfig, SingleDatasetLMConfig, UrlSingleDatasetLMConfig
from levanter_b200.main._common import compute_logits, load_model
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig
from levanter_b200.parallel.mesh import local_device
from levanter_b200.trainer import TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class VizLmConfig:
    checkpoint_path: str
    path: str = "logprobs.html"
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    data: Union[SingleDatasetLMConfig, LMMixtureDatasetConfig] = field(default_factory=UrlSingleDatasetLMConfig)
    model: LmConfig = field(default_factory=LlamaConfig)
    num_docs: int = 32
    checkpoint_is_hf: bool = False
    data_seed: Optional[int] = 0
    comparison_model_path: Optional[str] = None
    comparison_is_hf: bool = False


def _log_probs_and_argmax(model, batch):
    logits = compute_logits(model, batch).float()
    logp = torch.log_softmax(logits, dim=-1)
    targets = torch.roll(batch.tokens, -1, dims=-1).long()
    lp = logp.gather(-1, targets.unsqueeze(-1)).squeeze(-1) * batch.loss_mask.to(logp.dtype)
    return lp, logits.argmax(-1)


def main(config: VizLmConfig):
    lev.initialize(config)
    tokenizer = config.data.the_tokenizer
    Pos = config.model.seq_len
    validation_sets = config.data.validation_sets(Pos)
    if not validation_sets:
        raise ValueError("no validation set")
    device = local_device()
    dtype = config.trainer.mp.compute_dtype

    def load(path, is_hf):
        return load_model(config.model, tokenizer, checkpoint_path=None if is_hf else path, hf_checkpoint=path if is_hf else None,
                          dtype=dtype, device=device).eval()

    model = load(config.checkpoint_path, config.checkpoint_is_hf)
    comparison = load(config.comparison_model_path, config.comparison_is_hf) if config.comparison_model_path else None
    for name, ds in validation_sets.items():
        if config.data_seed is not None:
            ds = ds.shuffle(config.data_seed)
        loader = DataLoader(ds.take(config.num_docs), config.trainer.eval_batch_size, max_buffered_batches=0)
        path = config.path if not name else config.path.replace(".html", f".{name}.html")
        if comparison is None:
            compute_and_visualize_log_probs(path, model, tokenizer, _log_probs_and_argmax, loader, max_docs=config.num_docs)
        else:
            compute_and_diff_log_probs(path, model, comparison, tokenizer, lambda m, b: _log_probs_and_argmax(m, b)[0], loader,
                                       max_docs=config.num_docs)
        logger.info(f"wrote {path}")


if __name__ == "__main__":
    lev_config.main(main)()
