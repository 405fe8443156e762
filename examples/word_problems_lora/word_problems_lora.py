"""LoRA fine-tuning on question / answer records followed by an evaluation that *generates* answers (the counterpart of the
reference's examples/gsm8k-lora/gsm8k_lora.py): read ``{"question", "answer"}`` rows, train low-rank adapters with the loss on
the answer only, then answer held-out questions with the paged-KV generation engine and report exact-match accuracy of the
final number.  Written against the public API only.

    python examples/word_problems_lora/word_problems_lora.py --config_path examples/word_problems_lora/gsm8k_llama2.yaml
"""
from __future__ import annotations

import dataclasses
import logging
import os
import re
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch

import levanter_b200 as lev
from levanter_b200 import callbacks
from levanter_b200 import config as lev_config
from levanter_b200.compat.hf_checkpoints import HFCheckpointConverter, load_tokenizer
from levanter_b200.data.dataset import MappedAsyncDataset, _fold_in
from levanter_b200.data.sharded_datasource import datasource_from_jsonl
from levanter_b200.inference.engine import InferenceEngine, InferenceEngineConfig, Request
from levanter_b200.inference.jit_scheduler import SeqDecodingParams
from levanter_b200.lora import LoraConfig, lora_trainable_params_filter, loraize, save_merged_hf_model, save_peft_pretrained
from levanter_b200.models.lm_model import LmConfig, LmExample, compute_next_token_loss
from levanter_b200.optim import AdamConfig, OptimizerConfig
from levanter_b200.trainer import Trainer, TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class TrainArgs:
    optimizer: OptimizerConfig = field(default_factory=AdamConfig)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    lora: LoraConfig = field(default_factory=LoraConfig)
    train_data: str = "gsm8k_train.jsonl"
    eval_data: Optional[str] = "gsm8k_test.jsonl"
    data_cache_dir: str = "cache/word_problems"
    prompt: str = "Question: {question}\nAnswer:"
    max_tune_length: int = 512
    max_new_tokens: int = 256
    max_eval_examples: int = 200
    engine: InferenceEngineConfig = field(default_factory=lambda: InferenceEngineConfig(max_seqs=32, page_size=16, max_pages_per_seq=64))

    model_name_or_path: Optional[str] = None  # a Hugging Face checkpoint to start from ...
    model: Optional[LmConfig] = None          # ... or a model config to initialise randomly (smoke tests)
    tokenizer: Optional[str] = None
    vocab_size: Optional[int] = None  # for the passthrough tokenizer
    peft_save_path: Optional[str] = None
    merged_hf_save_path: Optional[str] = None


def final_number(text: str) -> Optional[str]:
    """The last number of an answer (GSM8K answers end in ``#### <number>``); commas are dropped."""
    found = re.findall(r"-?\d[\d,]*\.?\d*", text.split("####")[-1] if "####" in text else text)
    return found[-1].replace(",", "").rstrip(".") if found else None


def mk_dataset(config: TrainArgs, tokenizer, seq_len: int):
    eos = tokenizer.eos_token or ""

    def render(batch) -> List[dict]:
        prompts = [config.prompt.format_map(ex) for ex in batch]
        full = tokenizer([f"{p} {ex['answer']} {eos}".rstrip() for p, ex in zip(prompts, batch)], truncation=True, max_length=seq_len)["input_ids"]
        src = tokenizer(prompts, truncation=True, max_length=seq_len)["input_ids"]
        return [{"input_ids": np.asarray(f, dtype=np.int32), "source_len": np.asarray(len(s), dtype=np.int32)} for f, s in zip(full, src)]

    exemplar = {"input_ids": np.zeros((0,), dtype=np.int32), "source_len": np.zeros((), dtype=np.int32)}
    cache = datasource_from_jsonl([config.train_data]).map_batches(render, batch_size=256, output_exemplar=exemplar) \
        .build_or_load_cache(os.path.join(config.data_cache_dir, "train"))
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else tokenizer.eos_token_id

    def to_example(row) -> LmExample:
        ids = np.asarray(row["input_ids"])[:seq_len]
        tokens = np.full((seq_len,), pad, dtype=np.int64)
        tokens[:len(ids)] = ids
        loss_mask = np.zeros((seq_len,), dtype=np.float32)
        start = int(np.asarray(row["source_len"]).reshape(-1)[0]) - 1  # position i predicts token i + 1
        loss_mask[max(start, 0):max(len(ids) - 1, 0)] = 1.0
        return LmExample.causal(torch.from_numpy(tokens), loss_mask=torch.from_numpy(loss_mask))

    return MappedAsyncDataset(cache, to_example)


@torch.no_grad()
def evaluate_by_generation(model, tokenizer, config: TrainArgs) -> dict:
    """Greedy answers to the held-out questions; exact match of the final number."""
    rows = list(datasource_from_jsonl([config.eval_data]))[:config.max_eval_examples]
    prompts = [config.prompt.format_map(r) for r in rows]
    prompt_ids = tokenizer(prompts)["input_ids"]
    stop = None
    if tokenizer.eos_token_id is not None:
        stop = np.asarray([[tokenizer.eos_token_id]], dtype=np.int32)
    engine = InferenceEngine.from_model_with_config(model=model.eval(), tokenizer=tokenizer, config=config.engine)
    requests = [Request(prompt_tokens=[int(t) for t in ids], request_id=i,
                        decode_params=SeqDecodingParams(len(ids) + config.max_new_tokens, stop, 0.0, _fold_in(config.engine.seed, i)),
                        n_generations=1) for i, ids in enumerate(prompt_ids)]
    result = engine.generate(requests)
    correct, answers = 0, []
    for row, out in zip(rows, result.tokens):
        out = [t for t in out if t >= 0 and t != tokenizer.pad_token_id]
        text = tokenizer.decode(out, skip_special_tokens=True)
        answers.append(text)
        correct += int(final_number(text) is not None and final_number(text) == final_number(str(row["answer"])))
    return {"eval/exact_match": correct / max(len(rows), 1), "eval/num_examples": len(rows), "eval/generated_tokens": result.total_generated,
            "answers": answers}


def train(config: TrainArgs):
    lev.initialize(config)
    converter = None
    if config.model_name_or_path is not None:
        converter = HFCheckpointConverter.from_hf(config.model_name_or_path)
        tokenizer = converter.tokenizer if config.tokenizer is None else load_tokenizer(config.tokenizer)
        model_config = converter.default_config
    else:
        assert config.model is not None, "give model_name_or_path or model"
        model_config = config.model
        if config.tokenizer == "passthrough":
            from levanter_b200.data.passthrough_tokenizer import PassthroughTokenizer

            tokenizer = PassthroughTokenizer(config.vocab_size or 1000)
        else:
            tokenizer = load_tokenizer(config.tokenizer)
    seq_len = min(config.max_tune_length, model_config.seq_len)
    seed = config.trainer.seed
    model_key, lora_key, training_key = (_fold_in(seed, i) for i in range(3))

    with Trainer(config.trainer, config.optimizer, loss_fn=compute_next_token_loss) as trainer:
        dataset = mk_dataset(config, tokenizer, seq_len)
        if converter is not None:
            model = converter.load_pretrained(config=dataclasses.replace(model_config, seq_len=seq_len),
                                              dtype=config.trainer.mp.compute_dtype, device=trainer.device)
        else:
            model = model_config.build(len(tokenizer), seed=model_key, device=trainer.device)
        model = loraize(model, config.lora, seed=lora_key)
        state = trainer.initial_state(training_key, model=model, is_trainable=lora_trainable_params_filter(model))
        trainer.add_hook(callbacks.log_performance_stats(seq_len, config.trainer.batch_schedule), every=1)
        info = trainer.train(state, trainer.data_loader(dataset).iter_from_step(int(state.step)))

        report = None
        if config.eval_data is not None:
            report = evaluate_by_generation(info.state.model, tokenizer, config)
            lev.tracker.log_summary({k: v for k, v in report.items() if k != "answers"})
            logger.info(f"exact match {report['eval/exact_match']:.3f} over {report['eval/num_examples']} questions")
        if config.peft_save_path is not None:
            save_peft_pretrained(info.state.model, config.lora, config.model_name_or_path, config.peft_save_path)
        if config.merged_hf_save_path is not None and converter is not None:
            save_merged_hf_model(info.state.model, converter.replaced(tokenizer=tokenizer), config.merged_hf_save_path)
        return info, report


if __name__ == "__main__":
    lev_config.main(train)()
