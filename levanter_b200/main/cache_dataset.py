"""Tokenise and cache the train and validation splits of a dataset ahead of training
(src/levanter/main/cache_dataset.py:21-61)."""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field

from levanter_b200 import config as lev_config
from levanter_b200.data.metrics_monitor import LoggingMetricsMonitor
from levanter_b200.data.text import UrlSingleDatasetLMConfig, preprocessor_for_format
from levanter_b200.distributed import RayConfig
from levanter_b200.store.cache import build_or_load_cache
from levanter_b200.tracker import NoopConfig, TrackerConfig
from levanter_b200.utils.logging import init_logging

logger = logging.getLogger(__name__)


@dataclass(frozen=True)
class RayCachedLMDatasetConfig(UrlSingleDatasetLMConfig, RayConfig):
    tracker: TrackerConfig = field(default_factory=NoopConfig)


@lev_config.main()
def main(args: RayCachedLMDatasetConfig):
    init_logging(".", "cache_dataset.log")
    args.initialize()
    tokenizer = args.the_tokenizer
    for split in ["train", "validation"]:
        print(f"Caching {split} to {args.cache_dir}.")
        processor = preprocessor_for_format(args.format, tokenizer, enforce_bos=True, enforce_eos=args.enforce_eos)
        split_cache_dir = os.path.join(args.cache_dir, split)
        source = args.get_shard_source(split)
        if source is None:
            logger.warning(f"Skipping {split} because it is empty.")
            continue
        monitors = [] if isinstance(args.tracker, NoopConfig) else [LoggingMetricsMonitor("preprocess/" + split, commit=True)]
        cache = build_or_load_cache(split_cache_dir, source, processor, await_finished=False, monitors=monitors, options=args.cache_options)
        cache.await_finished()
        print(f"Finished caching {split} to {split_cache_dir}.")


if __name__ == "__main__":
    main()
