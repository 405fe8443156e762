"""Supervised fine-tuning on a weighted mixture of prompt/response datasets (src/levanter/main/sft_mixture.py:58-406)."""
from __future__ import annotations

import dataclasses
import logging
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Union

import levanter_b200 as lev
from levanter_b200 import config as lev_config
from levanter_b200.data.dataset import _fold_in
from levanter_b200.data.mixture import MixtureDataset, StopStrategy
from levanter_b200.data.permutation import PermutationDataset
from levanter_b200.data.text import ChatUrlDataSourceConfig, mk_single_turn_cached_sft_dataset
from levanter_b200.main.sft import (DatasetType, SupervisedSourceConfig, _cached_supervised, add_special_tokens, load_sft_tokenizer,
                                    resolve_model_and_converter, run_sft)
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig
from levanter_b200.optim import AdamConfig, OptimizerConfig
from levanter_b200.trainer import TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class SFTMixtureConfig:
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    model: LmConfig = field(default_factory=LlamaConfig)
    optimizer: OptimizerConfig = field(default_factory=AdamConfig)
    supervised_data: Dict[str, SupervisedSourceConfig] = field(default_factory=dict)
    mixture_weights: Dict[str, float] = field(default_factory=dict)
    mixture_block_size: int = 2048
    stop_strategy: str = StopStrategy.RESTART_STRATEGY
    initialize_from_hf: Union[bool, str] = False
    hf_save_path: Optional[str] = None
    hf_upload: Optional[str] = None
    hf_save_steps: int = 0
    max_seq_len: int = 2048
    model_name_or_path: str = "marin-community/marin-8b-base"
    tokenizer: str = "marin-community/marin-8b-base"
    dataset_type: DatasetType = DatasetType.CHAT_JSONL
    messages_field: str = "messages"
    input_role: str = "user"
    output_role: str = "assistant"
    data_seed: Optional[int] = None
    reinit_tokens: Union[List[str], bool] = False
    reinit_lm_head: bool = True
    reinit_embeddings: bool = True
    epoch: int = 0


def train(config: SFTMixtureConfig):
    tokenizer = load_sft_tokenizer(config.tokenizer, config.max_seq_len)
    model_config, converter = resolve_model_and_converter(config, tokenizer)
    config = dataclasses.replace(config, model=model_config)
    lev.initialize(config)
    logger.info(f"Added {add_special_tokens(tokenizer)} new tokens")
    seed = config.trainer.seed
    data_key, mix_key, model_key, training_key = (_fold_in(seed, i) for i in range(4))
    if config.data_seed is not None:
        data_key = config.data_seed
    if not config.supervised_data:
        raise ValueError("supervised_data must name at least one dataset")
    datasets = {}
    for i, (name, sd) in enumerate(config.supervised_data.items()):
        if config.dataset_type == DatasetType.CHAT_JSONL:
            chat = ChatUrlDataSourceConfig(cache_dir=sd.cache_dir, train_urls=list(sd.train_urls), messages_field=config.messages_field,
                                           input_role=config.input_role, output_role=config.output_role)
            ds = mk_single_turn_cached_sft_dataset(chat, tokenizer, model_config.seq_len)
        else:
            ds = _cached_supervised(sd, tokenizer)
        datasets[name] = PermutationDataset(ds, _fold_in(data_key, i))
    weights = config.mixture_weights or {n: 1.0 for n in datasets}
    mixture = MixtureDataset(datasets, weights, block_size=config.mixture_block_size, key=mix_key, stop_strategy=config.stop_strategy)
    run_sft(config, tokenizer, converter, _FiniteView(mixture, sum(len(d.as_sync_dataset()) for d in datasets.values())), model_key, training_key)


class _FiniteView:
    """One pass over a restart-strategy mixture: as many examples as the component datasets hold together."""

    def __init__(self, ds, n: int):
        self._ds, self._n = ds, n

    def as_sync_dataset(self):
        sync, n = self._ds.as_sync_dataset(), self._n

        class _V:
            def __len__(self_inner):
                return n

            def get_batch(self_inner, idx):
                return sync.get_batch(idx)

        return _V()


if __name__ == "__main__":
    lev_config.main(train)()
