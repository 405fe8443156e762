"""Train an encoder-decoder speech recognition model (src/levanter/main/train_asr.py:31-204); mirrors ``train_lm``.

``torchrun --nproc-per-node 8 -m levanter_b200.main.train_asr --config_path whisper_tiny_librispeech.yaml``."""
from __future__ import annotations

import gc
import logging
import os
from dataclasses import dataclass, field
from typing import Optional, Union

import levanter_b200 as lev
from levanter_b200 import callbacks
from levanter_b200 import config as lev_config
from levanter_b200.compat.hf_checkpoints import HFCompatConfig, save_hf_checkpoint_callback
from levanter_b200.data.audio import AudioIODatasetConfig, AudioMixtureDatasetConfig, AudioTextDataset
from levanter_b200.data.dataset import _fold_in
from levanter_b200.models.asr_model import ASRConfig, compute_asr_loss
from levanter_b200.models.whisper import WhisperConfig
from levanter_b200.optim import AdamConfig, OptimizerConfig
from levanter_b200.trainer import Trainer, TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class TrainASRConfig:
    data: Union[AudioIODatasetConfig, AudioMixtureDatasetConfig] = field(default_factory=AudioIODatasetConfig)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    model: ASRConfig = field(default_factory=WhisperConfig)
    optimizer: OptimizerConfig = field(default_factory=AdamConfig)
    batch_size: int = 16  # kept for config compatibility; the trainer's train_batch_size is what is used

    initialize_from_hf: Union[bool, str] = False
    use_hf_model_config: bool = False

    hf_save_path: Optional[str] = None
    hf_upload: Optional[str] = None
    hf_save_steps: int = 10000
    data_seed: Optional[int] = None


def main(config: TrainASRConfig):
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

    with Trainer(config.trainer, config.optimizer, compute_asr_loss) as trainer:
        seed = config.trainer.seed
        data_key, loader_key, model_key, training_key = (_fold_in(seed, i) for i in range(4))
        if config.data_seed is not None:
            logger.info(f"Overriding data seed with {config.data_seed}")
            data_key = config.data_seed

        vocab_size = len(tokenizer)
        tp_size = config.trainer.device_mesh.model_size if hasattr(config.trainer.device_mesh, "model_size") else 1
        Vocab = -(-vocab_size // tp_size) * tp_size
        if Vocab != vocab_size:
            logger.info(f"Rounding vocab size from {vocab_size} to {Vocab} for partitioning")

        pad_id = config.data.pad_token_id
        train_cache = config.data.train_set(key=data_key)
        if train_cache is None:
            raise ValueError("No training data: set data.train_urls or data.id")
        train_dataset = AudioTextDataset(train_cache, ignore_index=pad_id)
        eval_datasets = config.data.validation_sets()

        state = trainer.initial_state(training_key, model_init=lambda: config.model.build_asr(Vocab, seed=model_key, device=trainer.device))

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

        if len(eval_datasets) == 0:
            logger.warning("No evaluation datasets provided.")
        for name, eval_cache in eval_datasets.items():
            trainer.add_eval_hook(AudioTextDataset(eval_cache, ignore_index=pad_id), name=name or None)

        trainer.add_hook(callbacks.log_performance_stats(config.model.max_length, config.trainer.batch_schedule), every=1)

        if config.hf_save_path is not None and converter is not None:
            full_save_path = os.path.join(config.hf_save_path, trainer.run_id)
            trainer.add_hook(save_hf_checkpoint_callback(full_save_path, converter, upload_to_hf=config.hf_upload or False,
                                                         save_feature_extractor=True), every=config.hf_save_steps)

        train_loader = trainer.data_loader(train_dataset)
        if int(state.step) > 0:
            logger.info(f"Resuming training from step {state.step}")
        train_iter = train_loader.iter_from_step(int(state.step))
        trainer.train(state, train_iter)

    if trainer.tracker is not None:
        trainer.tracker.finish()


if __name__ == "__main__":
    lev_config.main(main)()
