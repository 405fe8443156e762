"""Instruction tuning written against the public API only (the counterpart of the reference's examples/alpaca/alpaca.py and
examples/alpaca-lora/alpaca_lora.py): read instruction/input/output records, render the prompt, tokenize prompt and response
together, cache, put the loss on the response tokens, and train; with ``lora:`` set only low-rank adapters are trained.

    python examples/instruction_tuning/instruction_tuning.py --config_path examples/instruction_tuning/alpaca_llama2.yaml
"""
from __future__ import annotations

import dataclasses
import logging
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

import levanter_b200 as lev
from levanter_b200 import callbacks
from levanter_b200 import config as lev_config
from levanter_b200.compat.hf_checkpoints import HFCheckpointConverter, save_hf_checkpoint_callback
from levanter_b200.data.dataset import MappedAsyncDataset, _fold_in
from levanter_b200.data.sharded_datasource import datasource_from_json, datasource_from_jsonl
from levanter_b200.lora import LoraConfig, lora_trainable_params_filter, loraize, save_peft_checkpoint_callback
from levanter_b200.models.lm_model import LmConfig, LmExample, compute_next_token_loss
from levanter_b200.optim import AdamConfig, OptimizerConfig
from levanter_b200.trainer import Trainer, TrainerConfig

logger = logging.getLogger(__name__)

DEFAULT_PROMPTS = {
    "prompt_input": ("Below is an instruction that describes a task, paired with an input that provides further context. "
                     "Write a response that appropriately completes the request.\n\n"
                     "### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:"),
    "prompt_no_input": ("Below is an instruction that describes a task. "
                        "Write a response that appropriately completes the request.\n\n"
                        "### Instruction:\n{instruction}\n\n### Response:"),
}


@dataclass
class TrainArgs:
    optimizer: OptimizerConfig = field(default_factory=AdamConfig)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    data: str = "alpaca_data.json"  # a .json (one list) or .jsonl file/url of {instruction, input, output} records
    data_cache_dir: str = "cache/instruction_tuning"
    max_tune_length: int = 2048
    prompts: Optional[Dict[str, str]] = None
    mask_inputs: bool = True  # no loss on the prompt tokens

    model_name_or_path: Optional[str] = None  # a Hugging Face checkpoint to start from ...
    model: Optional[LmConfig] = None          # ... or a model config to initialise randomly (smoke tests)
    tokenizer: Optional[str] = None
    vocab_size: Optional[int] = None  # for the passthrough tokenizer
    trust_remote_code: bool = False

    lora: Optional[LoraConfig] = None
    hf_save_path: Optional[str] = None
    hf_save_steps: int = 1000


def _records(path: str):
    return datasource_from_json([path]) if path.endswith(".json") else datasource_from_jsonl([path])


def mk_dataset(config: TrainArgs, tokenizer, seq_len: int):
    prompts = config.prompts or DEFAULT_PROMPTS
    eos = tokenizer.eos_token or ""

    def render(batch: Sequence[dict]) -> List[dict]:
        sources = [prompts["prompt_input" if ex.get("input") else "prompt_no_input"].format_map(ex) for ex in batch]
        targets = [f" {ex['output']} {eos}".rstrip() for ex in batch]
        full = tokenizer([s + t for s, t in zip(sources, targets)], truncation=True, max_length=seq_len)["input_ids"]
        src = tokenizer(sources, truncation=True, max_length=seq_len)["input_ids"]
        return [{"input_ids": np.asarray(f, dtype=np.int32), "source_len": np.asarray(len(s), dtype=np.int32)} for f, s in zip(full, src)]

    exemplar = {"input_ids": np.zeros((0,), dtype=np.int32), "source_len": np.zeros((), dtype=np.int32)}
    cache = _records(config.data).map_batches(render, batch_size=256, output_exemplar=exemplar).build_or_load_cache(config.data_cache_dir)
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else tokenizer.eos_token_id

    def to_example(row) -> LmExample:
        ids = np.asarray(row["input_ids"])[:seq_len]
        n = len(ids)
        tokens = np.full((seq_len,), pad, dtype=np.int64)
        tokens[:n] = ids
        loss_mask = np.zeros((seq_len,), dtype=np.float32)
        start = int(np.asarray(row["source_len"]).reshape(-1)[0]) - 1 if config.mask_inputs else 0  # position i predicts token i + 1
        loss_mask[max(start, 0):max(n - 1, 0)] = 1.0
        return LmExample.causal(torch.from_numpy(tokens), loss_mask=torch.from_numpy(loss_mask))

    return MappedAsyncDataset(cache, to_example)


def train(config: TrainArgs):
    lev.initialize(config)
    converter = None
    if config.model_name_or_path is not None:
        converter = HFCheckpointConverter.from_hf(config.model_name_or_path, trust_remote_code=config.trust_remote_code)
        tokenizer = converter.tokenizer if config.tokenizer is None else lev.compat.hf_checkpoints.load_tokenizer(config.tokenizer)
        model_config = converter.default_config
    else:
        assert config.model is not None, "give model_name_or_path or model"
        model_config = config.model
        if config.tokenizer == "passthrough":
            from levanter_b200.data.passthrough_tokenizer import PassthroughTokenizer

            tokenizer = PassthroughTokenizer(config.vocab_size or 1000)
        else:
            tokenizer = lev.compat.hf_checkpoints.load_tokenizer(config.tokenizer)
    seq_len = min(config.max_tune_length, model_config.seq_len)
    model_config = dataclasses.replace(model_config, seq_len=seq_len)
    seed = config.trainer.seed
    model_key, lora_key, training_key = (_fold_in(seed, i) for i in range(3))

    with Trainer(config.trainer, config.optimizer, loss_fn=compute_next_token_loss) as trainer:
        dataset = mk_dataset(config, tokenizer, seq_len)
        if converter is not None:
            model = converter.load_pretrained(config=model_config, dtype=config.trainer.mp.compute_dtype, device=trainer.device)
            if len(tokenizer) != model.vocab_size:
                model = model.resize_vocab(len(tokenizer))
        else:
            model = model_config.build(len(tokenizer), seed=model_key, device=trainer.device)
        if config.lora is not None:
            model = loraize(model, config.lora, seed=lora_key)
            state = trainer.initial_state(training_key, model=model, is_trainable=lora_trainable_params_filter(model))
        else:
            state = trainer.initial_state(training_key, model=model)
        trainer.add_hook(callbacks.log_performance_stats(seq_len, config.trainer.batch_schedule), every=1)
        if config.hf_save_path is not None:
            path = os.path.join(config.hf_save_path, trainer.run_id)
            if config.lora is not None:
                trainer.add_hook(save_peft_checkpoint_callback(path, config.lora, config.model_name_or_path), every=config.hf_save_steps)
            elif converter is not None:
                trainer.add_hook(save_hf_checkpoint_callback(path, converter.replaced(tokenizer=tokenizer)), every=config.hf_save_steps)
        loader = trainer.data_loader(dataset).iter_from_step(int(state.step))
        return trainer.train(state, loader)


if __name__ == "__main__":
    lev_config.main(train)()
