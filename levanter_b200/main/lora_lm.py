"""LoRA fine-tuning of a Hugging Face checkpoint (src/levanter/main/lora_lm.py:33-177): the base weights are frozen (they
never get gradient, master or optimizer storage in the engine), only the low-rank factors train; adapters are exported in
PEFT format and/or merged into a full HF checkpoint."""
from __future__ import annotations

import dataclasses
import logging
from dataclasses import dataclass, field
from typing import Optional

import levanter_b200 as lev
from levanter_b200 import callbacks
from levanter_b200 import config as lev_config
from levanter_b200.compat.hf_checkpoints import HFCheckpointConverter
from levanter_b200.data.dataset import _fold_in
from levanter_b200.data.text import SingleDatasetLMConfig, UrlSingleDatasetLMConfig
from levanter_b200.lora import (LoraConfig, lora_trainable_params_filter, loraize, save_merged_hf_checkpoint_callback,
                                save_peft_checkpoint_callback)
from levanter_b200.models.lm_model import compute_next_token_loss
from levanter_b200.optim import AdamConfig, OptimizerConfig
from levanter_b200.trainer import Trainer, TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class LoraLmConfig:
    initialize_from_hf: str
    lora: LoraConfig = field(default_factory=LoraConfig)
    data: SingleDatasetLMConfig = field(default_factory=UrlSingleDatasetLMConfig)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    optimizer: OptimizerConfig = field(default_factory=AdamConfig)
    peft_save_path: Optional[str] = None
    peft_hf_upload: Optional[str] = None
    hf_save_steps: int = 1000
    merged_hf_save_path: Optional[str] = None
    merged_hf_upload: Optional[str] = None
    trust_remote_code: bool = False
    max_train_length: Optional[int] = None


def main(config: LoraLmConfig):
    lev.initialize(config)
    tokenizer = config.data.the_tokenizer
    converter = HFCheckpointConverter.from_hf(config.initialize_from_hf, trust_remote_code=config.trust_remote_code)
    converter = converter.replaced(tokenizer=tokenizer)
    model_config = converter.default_config
    seed = config.trainer.seed
    data_key, loader_key, model_key, lora_key, training_key = (_fold_in(seed, i) for i in range(5))
    Pos = model_config.seq_len
    if config.max_train_length is not None:
        logger.info(f"Setting max tune length to {config.max_train_length}")
        Pos = config.max_train_length
        model_config = dataclasses.replace(model_config, seq_len=Pos)

    with Trainer(config.trainer, config.optimizer, loss_fn=compute_next_token_loss) as trainer:
        train_dataset = config.data.train_set(Pos, config.trainer.batch_schedule, key=data_key)
        eval_datasets = config.data.validation_sets(Pos)

        base = converter.load_pretrained(config=model_config, dtype=config.trainer.mp.compute_dtype, device=trainer.device)
        model = loraize(base, config.lora, seed=lora_key)
        state = trainer.initial_state(training_key, model=model, is_trainable=lora_trainable_params_filter(model))
        n_all = sum(p.numel() for p in state.model.parameters())
        n_train = sum(p.numel() for n, p in state.model.named_parameters() if state.is_trainable(n))
        lev.tracker.log_summary({"parameter_count": n_all, "trainable_parameter_count": n_train,
                                 "fraction_trainable": n_train / max(n_all, 1)})
        logger.info(f"Total parameter count: {n_all}; trainable: {n_train} ({n_train * 100.0 / max(n_all, 1):.3f}%)")

        for name, ds in eval_datasets.items():
            trainer.add_eval_hook(ds, name=name or None)
        trainer.add_hook(callbacks.log_performance_stats(Pos, config.trainer.batch_schedule), every=1)
        if config.peft_save_path is not None:
            trainer.add_hook(save_peft_checkpoint_callback(f"{config.peft_save_path}/{trainer.run_id}", config.lora,
                                                           config.initialize_from_hf, upload_to_hf=config.peft_hf_upload),
                             every=config.hf_save_steps)
        if config.merged_hf_save_path is not None:
            trainer.add_hook(save_merged_hf_checkpoint_callback(f"{config.merged_hf_save_path}/{trainer.run_id}", converter,
                                                                upload_to_hf=config.merged_hf_upload or False),
                             every=config.hf_save_steps)
        loader = trainer.data_loader(train_dataset).iter_from_step(int(state.step))
        trainer.train(state, loader)


if __name__ == "__main__":
    lev_config.main(main)()
