"""Sample continuations of a few prompts with the paged-KV generation engine (src/levanter/main/sample_lm.py:31-199)."""
from __future__ import annotations

import logging
import time
from dataclasses import dataclass, field
from typing import List, Optional, Tuple, Union

import numpy as np

import levanter_b200 as lev
from levanter_b200 import config as lev_config
from levanter_b200.callbacks import profile_ctx
from levanter_b200.compat.hf_checkpoints import RepoRef, load_tokenizer
from levanter_b200.data.dataset import _fold_in
from levanter_b200.inference.engine import InferenceEngine, InferenceEngineConfig, Request
from levanter_b200.inference.jit_scheduler import SeqDecodingParams
from levanter_b200.inference.utils import INVALID
from levanter_b200.main._common import load_model
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmConfig
from levanter_b200.parallel.mesh import local_device
from levanter_b200.trainer import TrainerConfig

logger = logging.getLogger(__name__)


@dataclass
class SampleLmConfig:
    checkpoint_path: Optional[str] = None
    hf_checkpoint: Optional[RepoRef] = None
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    model: LmConfig = field(default_factory=LlamaConfig)
    tokenizer: Optional[str] = None
    engine: InferenceEngineConfig = field(default_factory=InferenceEngineConfig)
    prompts: Union[List[str], str, Tuple[str, ...]] = ("Four score and seven years ago, our",
                                                       "In a hole in the ground there lived a hobbit, not a nasty, dirty, wet hole") * 5
    stop_sequence: Optional[str] = "."  # whole-token match
    max_new_tokens: int = 192
    temperature: float = 0.7
    seed: int = 2
    n_generations: int = 1
    n_rounds: int = 4
    profile: bool = False


def main(config: SampleLmConfig):
    lev.initialize(config)
    tok_name = config.tokenizer or (str(config.hf_checkpoint) if config.hf_checkpoint is not None else None)
    if tok_name is None:
        raise ValueError("Must specify a tokenizer or an HF checkpoint with a tokenizer")
    tokenizer = load_tokenizer(tok_name)
    model = load_model(config.model, tokenizer, checkpoint_path=config.checkpoint_path, hf_checkpoint=config.hf_checkpoint,
                       dtype=config.trainer.mp.compute_dtype, device=local_device()).eval()
    prompts = [config.prompts] if isinstance(config.prompts, str) else list(config.prompts)
    prompt_ids = tokenizer(prompts, add_special_tokens=False)["input_ids"]
    service = InferenceEngine.from_model_with_config(model=model, tokenizer=tokenizer, config=config.engine)
    stop_ids = None
    if config.stop_sequence is not None:
        ids = tokenizer(config.stop_sequence, add_special_tokens=False)["input_ids"]
        if len(ids) == 0:
            raise ValueError("Stop sequence must be non-empty")
        stop_ids = np.asarray([ids], dtype=np.int32)

    for r in range(config.n_rounds):
        ctx = None
        if config.profile and (config.n_rounds == 1 or r == 1):
            ctx = profile_ctx(str(config.trainer.log_dir / str(config.trainer.id) / "profiler"), create_perfetto_link=False)
            ctx.__enter__()
        t0 = time.time()
        reqs = [Request(prompt_tokens=list(map(int, toks)), request_id=i,
                        decode_params=SeqDecodingParams(len(toks) + config.max_new_tokens, stop_ids, config.temperature,
                                                        _fold_in(config.engine.seed, i)), n_generations=config.n_generations)
                for i, toks in enumerate(prompt_ids)]
        result = service.generate(reqs)
        dt = time.time() - t0
        if ctx is not None:
            ctx.__exit__(None, None, None)
        print(f"Round {r} took {dt:.2f} seconds, generated {result.total_generated} tokens in {len(result.tokens)} sequences "
              f"({result.total_generated / max(dt, 1e-9):.1f} tokens/s).")
        lev.tracker.log({"sample/round_time": dt, "sample/tokens_per_second": result.total_generated / max(dt, 1e-9)}, step=r)
        for sid, out in enumerate(result.tokens):
            out = [t for t in out if t != tokenizer.pad_token_id and t != INVALID]
            print(f"Generated text for {sid} (len {len(out)}): {tokenizer.decode(out, skip_special_tokens=True)}")
    lev.current_tracker().finish()


if __name__ == "__main__":
    lev_config.main(main)()
