"""Evaluate a checkpoint on the validation sets of a data config (src/levanter/main/eval_lm.py:33-191)."""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Optional, Union

import levanter_b200 as lev
from levanter_b200 import config as lev_config
from levanter_b200.analysis import compute_entropy_histogram, compute_top2_gap_histogram, summary_statistics_for_tree
from levanter_b200.compat.hf_checkpoints import RepoRef
from levanter_b200.data.loader import DataLoader
from levanter_b200.data.text import LMMixtureDatasetConfig, SingleDatasetLMConfig, UrlSingleDatasetLMConfig
from levanter_b200.eval import TaggedEvaluator, eval_model
from levanter_b200.main._common import compute_logits, load_model
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig
from levanter_b200.parallel.mesh import local_device
from levanter_b200.trainer import TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class EvalLmConfig:
    checkpoint_path: Optional[str] = None
    hf_checkpoint: Optional[RepoRef] = None
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    data: Union[SingleDatasetLMConfig, LMMixtureDatasetConfig] = field(default_factory=UrlSingleDatasetLMConfig)
    model: LmConfig = field(default_factory=LlamaConfig)
    eval_on_train: bool = False
    log_entropy: bool = False
    log_top2_gap: bool = False
    log_param_stats: bool = False


def main(config: EvalLmConfig):
    lev.initialize(config)
    tokenizer = config.data.the_tokenizer
    Batch = config.trainer.eval_batch_size
    Pos = config.model.seq_len

    if config.eval_on_train:
        datasets = [(ds, [name]) for name, ds in config.data.train_sets(Pos, key=0).items()]
    else:
        datasets = config.data.tagged_eval_sets(Pos)
    if not datasets:
        raise ValueError("no dataset found!")
    max_examples = None
    if config.trainer.max_eval_batches is not None:
        max_examples = config.trainer.max_eval_batches * config.trainer.eval_batch_size
        datasets = [(ds.take(max_examples), tags) for ds, tags in datasets]

    mesh = config.trainer.device_mesh if config.trainer.num_devices > 1 else None
    evaluator = TaggedEvaluator(Batch, datasets, tokenizer, device_mesh=mesh, max_examples_per_dataset=max_examples)
    model = load_model(config.model, tokenizer, checkpoint_path=config.checkpoint_path, hf_checkpoint=config.hf_checkpoint,
                       dtype=config.trainer.mp.compute_dtype, device=local_device())

    log_dict = eval_model(evaluator, model, prefix="eval")
    lev.tracker.log(log_dict, step=0)
    print("Loss:", log_dict["eval/loss"])

    def _sets():
        for name, ds in config.data.validation_sets(Pos).items():
            if max_examples is not None:
                ds = ds.take(max_examples)
            yield name, DataLoader(ds, Batch, max_buffered_batches=0)

    if config.log_entropy:
        for name, loader in _sets():
            lev.tracker.log({f"analysis/{name}/entropy": compute_entropy_histogram(model, None, compute_logits, loader)}, step=0)
    if config.log_top2_gap:
        for name, loader in _sets():
            lev.tracker.log({f"analysis/{name}/top2_gap": compute_top2_gap_histogram(model, None, compute_logits, loader)}, step=0)
    if config.log_param_stats:
        lev.tracker.log(summary_statistics_for_tree("params", dict(model.named_parameters()), split_scan_layers=True,
                                                    include_histogram=True), step=0)
    lev.tracker.current_tracker().finish()
    return log_dict


if __name__ == "__main__":
    lev_config.main(main)()
