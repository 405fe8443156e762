"""Supervised fine-tuning on prompt/response data, with online packing of several examples per row
(src/levanter/main/sft.py:55-428)."""
from __future__ import annotations

import dataclasses
import logging
import os
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, Iterator, List, Optional, Union

import torch

import levanter_b200 as lev
from levanter_b200 import callbacks
from levanter_b200 import config as lev_config
from levanter_b200.compat.hf_checkpoints import HFCheckpointConverter, HFCompatConfig, save_hf_checkpoint_callback
from levanter_b200.data.dataset import AsyncDataset, EpochDataset, _fold_in
from levanter_b200.data.loader import stack_batches
from levanter_b200.data.packing import PromptCompletion, pack_prompt_completions
from levanter_b200.data.permutation import PermutationDataset
from levanter_b200.data.text import (ChatUrlDataSourceConfig, SupervisedHfSourceConfig, SupervisedUrlSourceConfig,
                                     mk_single_turn_cached_sft_dataset, mk_supervised_dataset)
from levanter_b200.data.utils import batched
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig, compute_next_token_loss
from levanter_b200.optim import AdamConfig, OptimizerConfig
from levanter_b200.trainer import Trainer, TrainerConfig
from levanter_b200.utils.background_iterable import BackgroundIterator

logger = logging.getLogger(__name__)

DEFAULT_PAD_TOKEN = "[PAD]"
DEFAULT_EOS_TOKEN = "</s>"
DEFAULT_BOS_TOKEN = "<s>"
DEFAULT_UNK_TOKEN = "<unk>"
SupervisedSourceConfig = Union[SupervisedUrlSourceConfig, SupervisedHfSourceConfig]


class DatasetType(str, Enum):
    HUGGINGFACE = "huggingface"
    CHAT_JSONL = "chat_jsonl"


@dataclass
class SFTConfig:
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    model: LmConfig = field(default_factory=LlamaConfig)
    optimizer: OptimizerConfig = field(default_factory=AdamConfig)
    supervised_data: Union[None, SupervisedSourceConfig, Dict[str, SupervisedSourceConfig]] = None
    initialize_from_hf: Union[bool, str] = False
    hf_save_path: Optional[str] = None
    hf_upload: Optional[str] = None
    hf_save_steps: int = 0
    max_seq_len: int = 2048
    model_name_or_path: str = "NousResearch/Llama-2-7b-hf"
    tokenizer: str = "NousResearch/Llama-2-7b-hf"
    dataset_type: DatasetType = DatasetType.CHAT_JSONL
    chat_train_urls: Optional[List[str]] = None
    messages_field: str = "messages"
    input_role: str = "user"
    output_role: str = "assistant"
    data_seed: Optional[int] = None
    epoch: int = 0
    reinit_tokens: Union[List[str], bool] = False
    """re-draw the embedding rows of these tokens from the distribution of the trained rows (tokens never seen in
    pre-training have much smaller norms); True = the Llama-3 chat control tokens"""
    reinit_lm_head: bool = True
    reinit_embeddings: bool = True


def load_sft_tokenizer(name: str, max_seq_len: int):
    from levanter_b200.compat.hf_checkpoints import load_tokenizer

    tok = load_tokenizer(name)
    tok.model_max_length = max_seq_len
    tok.padding_side = "right"
    return tok


def resolve_model_and_converter(config, tokenizer):
    converter = None
    if config.initialize_from_hf:
        if config.trainer.initialize_from is not None:
            raise ValueError("Cannot use both --initialize_from_hf and --initialize_from")
        assert isinstance(config.model, HFCompatConfig)
        converter = HFCheckpointConverter.from_hf(config.model_name_or_path, trust_remote_code=True)
        if isinstance(config.initialize_from_hf, str):
            converter = converter.replaced(reference_checkpoint=config.initialize_from_hf, tokenizer=tokenizer)
        else:
            converter = converter.replaced(tokenizer=tokenizer)
        model_config = dataclasses.replace(converter.default_config, seq_len=config.max_seq_len)
    elif config.trainer.initialize_from is None:
        raise ValueError("Must specify either --initialize_from_hf or --initialize_from")
    else:
        if config.hf_save_steps:
            converter = HFCheckpointConverter.from_hf(config.model_name_or_path, trust_remote_code=True).replaced(tokenizer=tokenizer)
        model_config = config.model
    return model_config, converter


def train(config: SFTConfig):
    tokenizer = load_sft_tokenizer(config.tokenizer, config.max_seq_len)
    model_config, converter = resolve_model_and_converter(config, tokenizer)
    config = dataclasses.replace(config, model=model_config)
    lev.initialize(config)
    logger.info(f"Added {add_special_tokens(tokenizer)} new tokens")

    seed = config.trainer.seed
    data_key, _, model_key, training_key = (_fold_in(seed, i) for i in range(4))
    if config.data_seed is not None:
        data_key = config.data_seed
    Pos = model_config.seq_len

    if config.dataset_type == DatasetType.CHAT_JSONL:
        assert config.chat_train_urls is not None and config.supervised_data is not None
        sd = config.supervised_data
        cache_dir = sd.cache_dir if not isinstance(sd, dict) else next(iter(sd.values())).cache_dir
        chat_config = ChatUrlDataSourceConfig(cache_dir=cache_dir, train_urls=config.chat_train_urls, messages_field=config.messages_field,
                                              input_role=config.input_role, output_role=config.output_role)
        train_dataset = mk_single_turn_cached_sft_dataset(chat_config, tokenizer, Pos)
    else:
        assert config.supervised_data is not None
        sd = next(iter(config.supervised_data.values())) if isinstance(config.supervised_data, dict) else config.supervised_data
        train_dataset = _cached_supervised(sd, tokenizer)
    train_dataset = PermutationDataset(train_dataset, data_key)
    if config.epoch > 0:
        train_dataset = EpochDataset(train_dataset, max_epochs=config.epoch)
    run_sft(config, tokenizer, converter, train_dataset, model_key, training_key)


def _cached_supervised(sd, tokenizer) -> AsyncDataset:
    """The tokenised ``{"input_ids", "sources_len"}`` cache of a supervised source (no padding: packing happens online)."""
    import numpy as np

    from levanter_b200.data.text import _preprocess_supervised_example
    from levanter_b200.utils.hf_utils import num_cpus_used_by_tokenizer

    source = sd.get_shard_source("train")
    exemplar = {"input_ids": np.zeros((0,), dtype=np.int32), "sources_len": np.zeros((0,), dtype=np.int32)}
    ds = source.map_batches(lambda ex: _preprocess_supervised_example(ex, tokenizer, sd.input_field, sd.output_field), batch_size=128,
                            num_cpus=num_cpus_used_by_tokenizer(tokenizer), output_exemplar=exemplar)
    return ds.build_or_load_cache(os.path.join(sd.cache_dir, "train"), await_finished=True)


def run_sft(config, tokenizer, converter, train_dataset: AsyncDataset, model_key, training_key):
    """Shared by ``sft`` and ``sft_mixture``: build the state, pack prompt/completions online, train."""
    Pos = config.model.seq_len
    with Trainer(config.trainer, config.optimizer, loss_fn=compute_next_token_loss) as trainer:
        vocab_size = len(tokenizer)
        if config.initialize_from_hf:
            logger.info(f"Loading pretrained model from {converter.reference_checkpoint}")
            model = converter.load_pretrained(config=config.model, dtype=trainer.config.mp.param_dtype, device=trainer.device)
            model = model.resize_vocab(vocab_size)
            state = trainer.initial_state(training_key, model=model)
        else:
            state = trainer.initial_state(training_key, model_init=lambda: config.model.build(vocab_size, seed=model_key, device=trainer.device))

        fpt = config.model.flops_per_token(vocab_size)
        trainer.add_hook(callbacks.log_performance_stats(Pos, config.trainer.batch_schedule, 3 * fpt * Pos if fpt else None), every=1)

        current_step = int(state.step)
        it = create_prompt_completion_iterator(train_dataset, Pos)
        if current_step > 0:
            logger.info(f"Resuming training from step {current_step}")
            for _ in range(current_step * config.trainer.train_batch_size):
                try:
                    next(it)
                except StopIteration:
                    logger.warning("Ran out of examples while seeking - restarting from beginning")
                    it = create_prompt_completion_iterator(train_dataset, Pos)
        elif config.reinit_tokens:
            toks = ["<|finetune_right_pad_id|>", "<|start_header_id|>", "<|end_header_id|>", "<|eom_id|>", "<|eot_id|>"] \
                if config.reinit_tokens is True else list(config.reinit_tokens)
            logger.info(f"Reinitializing tokens: {toks}")
            reinitialize_some_tokens(state, tokenizer, toks, _fold_in(int(training_key[0]) if hasattr(training_key, "__len__") else training_key, 7),
                                     reinit_lm_head=config.reinit_lm_head, reinit_embeddings=config.reinit_embeddings)

        pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else tokenizer.eos_token_id
        packed = pack_prompt_completions(Pos, it, max_segments_per_example=4, pad_token=pad, max_buffered_examples=16)
        mesh = trainer.device_mesh if config.trainer.num_devices > 1 else None
        shard = (mesh.batch_index, mesh.batch_size_divisor) if mesh is not None else None
        loader = BackgroundIterator(lambda: stack_batches(packed, Pos, config.trainer.train_batch_size, shard=shard), max_capacity=1024)

        if config.hf_save_path is not None and converter is not None and config.hf_save_steps:
            path = os.path.join(config.hf_save_path, trainer.run_id) if config.trainer.checkpointer.append_run_id_to_base_path else config.hf_save_path
            trainer.add_hook(save_hf_checkpoint_callback(path, converter, upload_to_hf=config.hf_upload or False), every=config.hf_save_steps)
        trainer.train(state, loader)


def reinitialize_some_tokens(state, tokenizer, tokens_to_reinit: List[str], key, reinit_lm_head=True, reinit_embeddings=True):
    """Overwrite the embedding (and lm_head) rows of ``tokens_to_reinit`` with draws from a truncated normal that has the
    per-dimension mean and standard deviation of the whole matrix; the change goes through the engine so master and compute
    copies agree."""
    ids = [tokenizer.convert_tokens_to_ids(t) for t in tokens_to_reinit]
    if not ids:
        raise ValueError("No tokens to reinitialize")
    if any(i is None or tokenizer.convert_ids_to_tokens(i) != t for i, t in zip(ids, tokens_to_reinit)):
        raise ValueError("One or more tokens are not in the tokenizer vocabulary")
    gen = torch.Generator().manual_seed(int(key) & 0x7FFFFFFF)
    full = state.engine.full_master()
    changed = {}
    for name, w in full.items():
        is_emb = name.endswith("token_embeddings.weight") and reinit_embeddings
        is_head = name.startswith("lm_head") and name.endswith("weight") and reinit_lm_head
        if not (is_emb or is_head):
            continue
        w = w.detach().float().cpu().clone()
        mu, std = w.mean(dim=0), w.std(dim=0)
        draw = torch.nn.init.trunc_normal_(torch.empty(len(ids), w.shape[1]), 0.0, 1.0, -3.0, 3.0, generator=gen)
        w[torch.tensor(ids)] = draw * std + mu
        changed[name] = w
    if changed:
        full.update(changed)
        state.engine.load_full_params(full)
    return state


def create_prompt_completion_iterator(cached_dataset: AsyncDataset, Pos) -> Iterator[PromptCompletion]:
    """Examples whose prompt alone fills the window, or that have no response token left after truncation, are skipped."""
    S = int(getattr(Pos, "size", Pos))
    sync = cached_dataset.as_sync_dataset()
    n = len(sync)
    for idxs in batched(range(n), 4096):
        for i, ex in zip(idxs, sync.get_batch(list(idxs))):
            src = int(ex["sources_len"].reshape(-1)[0])
            if src > S - 1:
                continue
            ids = ex["input_ids"].tolist()[:S]
            if len(ids) <= src:
                continue
            yield PromptCompletion(ids=ids, prompt_length=src, segment_id=i)


def add_special_tokens(tokenizer, use_unk_instead_of_adding: bool = False) -> int:
    if use_unk_instead_of_adding and tokenizer.unk_token is None:
        raise ValueError("use_unk_instead_of_add is True but tokenizer doesn't have an unk token")
    unk = tokenizer.unk_token if use_unk_instead_of_adding else None
    special = {}
    if tokenizer.pad_token is None:
        special["pad_token"] = unk or DEFAULT_PAD_TOKEN
    if tokenizer.eos_token is None:
        special["eos_token"] = unk or DEFAULT_EOS_TOKEN
    if tokenizer.bos_token is None:
        special["bos_token"] = unk or DEFAULT_BOS_TOKEN
    if tokenizer.unk_token is None:
        special["unk_token"] = DEFAULT_UNK_TOKEN
    return tokenizer.add_special_tokens(special) if special else 0


if __name__ == "__main__":
    lev_config.main(train)()
