"""Pre-train or continue training a causal language model (src/levanter/main/train_lm.py:37-281).

Launch one process per GPU: ``torchrun --nproc-per-node 8 -m levanter_b200.main.train_lm --config_path llama2_7b.yaml``."""
from __future__ import annotations

import functools
import gc
import logging
import os
from dataclasses import dataclass, field
from typing import Optional, Union

import torch

import levanter_b200 as lev
from levanter_b200 import callbacks
from levanter_b200 import config as lev_config
from levanter_b200.checkpoint import load_checkpoint
from levanter_b200.compat.hf_checkpoints import HFCompatConfig, save_hf_checkpoint_callback
from levanter_b200.data.dataset import _fold_in
from levanter_b200.data.text import LMMixtureDatasetConfig, SingleDatasetLMConfig, UrlSingleDatasetLMConfig
from levanter_b200.eval_harness import LmEvalHarnessConfig
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig, compute_next_token_loss
from levanter_b200.optim import AdamConfig, OptimizerConfig
from levanter_b200.trainer import Trainer, TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class TrainLmConfig:
    data: Union[SingleDatasetLMConfig, LMMixtureDatasetConfig] = field(default_factory=UrlSingleDatasetLMConfig)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    model: LmConfig = field(default_factory=LlamaConfig)
    optimizer: OptimizerConfig = field(default_factory=AdamConfig)

    initialize_from_hf: Union[bool, str] = False
    """a checkpoint id/path, or True for the model class's default reference checkpoint"""
    use_hf_model_config: bool = False  # replace ``model`` by the config stored with the HF checkpoint

    z_loss_weight: float = 0.0

    hf_save_path: Optional[str] = None
    hf_upload: Optional[str] = None
    hf_save_steps: int = 10000
    hf_save_dtype: Optional[str] = None

    data_seed: Optional[int] = None  # overrides the data key derived from trainer.seed
    initialize_from_checkpoint_path: Optional[str] = None
    """start from this checkpoint's weights at step 0 (the data loader starts over, unlike trainer.initialize_from)"""
    epoch: int = 0
    eval_harness: Optional[LmEvalHarnessConfig] = None
    eval_harness_steps: int = 10000

    log_entropy: bool = False


def main(config: TrainLmConfig):
    tokenizer = config.data.the_tokenizer

    converter = None
    if config.initialize_from_hf:
        if config.trainer.initialize_from is not None:
            raise ValueError("Cannot specify both initialize_from_hf and initialize_from")
        assert isinstance(config.model, HFCompatConfig)
        converter = config.model.hf_checkpoint_converter()
        if isinstance(config.initialize_from_hf, str):
            converter = converter.replaced(reference_checkpoint=config.initialize_from_hf, tokenizer=tokenizer)
        else:
            converter = converter.replaced(tokenizer=tokenizer)
        if config.use_hf_model_config:
            config.model = converter.config_from_hf_config(converter.default_hf_config)
    elif isinstance(config.model, HFCompatConfig):
        converter = config.model.hf_checkpoint_converter().replaced(tokenizer=tokenizer)

    lev.initialize(config)
    loss_function = functools.partial(compute_next_token_loss, logsumexp_weight=config.z_loss_weight or None)

    with Trainer(config.trainer, config.optimizer, loss_function) as trainer:
        seed = config.trainer.seed
        data_key, loader_key, model_key, training_key = (_fold_in(seed, i) for i in range(4))
        if config.data_seed is not None:
            logger.info(f"Overriding data seed with {config.data_seed}")
            data_key = config.data_seed

        Pos = config.model.seq_len
        vocab_size = len(tokenizer)
        # the vocabulary axis is split over the model (tensor-parallel) axis: round it up to a multiple of its size
        tp_size = config.trainer.device_mesh.model_size if hasattr(config.trainer.device_mesh, "model_size") else 1
        Vocab = -(-vocab_size // tp_size) * tp_size
        if Vocab != vocab_size:
            logger.info(f"Rounding vocab size from {vocab_size} to {Vocab} for partitioning")

        train_dataset = config.data.train_set(Pos, config.trainer.batch_schedule, key=data_key, epochs=config.epoch)
        tagged_eval_datasets = config.data.tagged_eval_sets(Pos)

        def model_init():
            tp = trainer.tensor_parallel
            if tp is None:
                return config.model.build(Vocab, seed=model_key, device=trainer.device)
            # model axis > 1 (tensor_parallel_axes): heads and MLP columns are split over the model axis; every rank takes its
            # slices of the weights an unsharded run with this seed would start from
            from levanter_b200.parallel.tp import build_sharded_from_seed

            return build_sharded_from_seed(lambda tp: config.model.build(Vocab, seed=model_key, device=trainer.device, tp=tp), tp)

        state = trainer.initial_state(training_key, model_init=model_init)

        if int(state.step) == 0 and config.initialize_from_checkpoint_path is not None:
            state = load_checkpoint(state, config.initialize_from_checkpoint_path)
            state.step = 0

        if int(state.step) == 0:
            if config.initialize_from_hf:
                logger.info(f"No training checkpoint found. Initializing model from HF checkpoint '{converter.reference_checkpoint}'")
                gc.collect()
                hf_model = converter.load_pretrained(config=config.model if not config.use_hf_model_config else None, device="cpu")
                state.engine.load_full_params({k: v.detach() for k, v in hf_model.named_parameters()})
                del hf_model
            else:
                logger.info("No checkpoint found. Starting from scratch.")

        lev.tracker.log_summary({"parameter_count": sum(p.numel() for p in state.model.parameters())})

        max_eval_examples_per_ds = config.trainer.max_eval_batches
        if max_eval_examples_per_ds is not None:
            max_eval_examples_per_ds *= config.trainer.eval_batch_size

        if len(tagged_eval_datasets) == 0:
            logger.warning("No evaluation datasets provided.")
        else:
            from levanter_b200.eval import cb_tagged_lm_evaluate

            cb = cb_tagged_lm_evaluate(config.trainer.eval_batch_size, tagged_eval_datasets, tokenizer,
                                       trainer.device_mesh if config.trainer.num_devices > 1 else None, None,
                                       max_eval_examples_per_ds, mp=config.trainer.mp)
            trainer.add_hook(cb, every=config.trainer.steps_per_eval)

        flops_per_token = config.model.flops_per_token(vocab_size)
        flops_per_example = 3 * flops_per_token * Pos if flops_per_token is not None else None
        trainer.add_hook(callbacks.log_performance_stats(Pos, config.trainer.batch_schedule, flops_per_example), every=1)

        if config.hf_save_path is not None and converter is not None:
            full_save_path = os.path.join(config.hf_save_path, trainer.run_id) \
                if config.trainer.checkpointer.append_run_id_to_base_path else config.hf_save_path
            save_dtype = None
            if config.hf_save_dtype is not None:
                save_dtype = getattr(torch, config.hf_save_dtype.replace("bf16", "bfloat16").replace("fp32", "float32"), None)
                if save_dtype is None:
                    logger.warning(f"Invalid hf_save_dtype: {config.hf_save_dtype}. Defaulting to None.")
            trainer.add_hook(save_hf_checkpoint_callback(full_save_path, converter, upload_to_hf=config.hf_upload or False,
                                                         save_dtype=save_dtype), every=config.hf_save_steps)

        if config.eval_harness is not None:
            from levanter_b200.eval_harness import lm_eval_harness

            trainer.add_hook(lm_eval_harness(config.eval_harness, tokenizer, config.trainer.eval_batch_size, None, config.trainer.mp),
                             every=config.eval_harness_steps)

        if config.log_entropy:
            from levanter_b200.analysis import cb_compute_entropies

            def compute_logits(model, example):
                acts = model.activations(example.tokens, example.attn_mask)
                acts = acts[0] if isinstance(acts, tuple) else acts
                return acts @ model.get_lm_head().to(acts.dtype).t()

            for name, dataset in config.data.validation_sets(Pos).items():
                trainer.add_hook(cb_compute_entropies(compute_logits, Vocab, dataset, prefix=os.path.join("analysis", name) if name else "analysis",
                                                      batch_size=config.trainer.eval_batch_size, mapping=None),
                                 every=config.trainer.steps_per_eval)

        train_loader = trainer.data_loader(train_dataset)
        if int(state.step) > 0:
            logger.info(f"Resuming training from step {state.step}")
        train_iter = train_loader.iter_from_step(int(state.step))

        last_info = trainer.train(state, train_iter)

        if config.trainer.checkpointer is not None and config.epoch > 0 and last_info is not None:
            trainer.hooks.run_hooks(last_info, force=True)
            trainer.checkpointer.wait_until_finished()

    if trainer.tracker is not None:
        trainer.tracker.finish()


if __name__ == "__main__":
    lev_config.main(main)()
