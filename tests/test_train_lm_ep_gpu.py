"""``train_lm`` end to end on two GPUs with an expert-parallel Mixtral: cache build, bf16 training through the sharded engine
(rank-local expert buckets next to the sharded ones) with the token exchange on peer memory, evaluation, a checkpoint written
by both ranks, and a resume of the same command."""
import json
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _write_data(d, n=400, vocab=250):
    rng = np.random.default_rng(0)
    for s in range(2):
        with open(f"{d}/shard{s}.jsonl", "w") as f:
            for _ in range(n):
                f.write(json.dumps({"text": " ".join(map(str, rng.integers(0, vocab, size=int(rng.integers(40, 160)))))}) + "\n")


def _cfg(d, steps):
    return f"""
data:
  tokenizer: passthrough
  vocab_size: 256
  cache_dir: {d}/cache
  train_urls: ["{d}/shard0.jsonl"]
  validation_urls: ["{d}/shard1.jsonl"]
model:
  type: mixtral
  seq_len: 128
  hidden_dim: 256
  intermediate_dim: 512
  num_layers: 2
  num_heads: 2
  num_kv_heads: 2
  n_routed_experts: 8
  num_experts_per_tok: 2
  expert_parallel: true
  gradient_checkpointing: false
trainer:
  id: eprun
  mp: p=f32,c=bfloat16
  num_train_steps: {steps}
  train_batch_size: 16
  per_device_eval_parallelism: 4
  steps_per_eval: 4
  max_eval_batches: 2
  tracker:
    type: json_logger
  checkpointer:
    base_path: {d}/ckpt
    save_interval: 1h
  log_dir: {d}/logs
optimizer:
  learning_rate: 3e-3
  warmup: 0.0
"""


def _worker(rank, world, port, d, steps):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import yaml

    from levanter_b200 import config as C
    from levanter_b200.main import train_lm
    from levanter_b200.ops import lib

    torch.cuda.set_device(rank)
    cfg = C.decode(train_lm.TrainLmConfig, yaml.safe_load(_cfg(d, steps)))
    n0 = lib.launch_count
    train_lm.main(cfg)
    lib.check_status()
    assert lib.launch_count > n0
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_train_lm_expert_parallel_two_gpus_then_resume(tmp_path):
    import torch.multiprocessing as mp

    from levanter_b200.checkpoint import discover_latest_checkpoint

    d = str(tmp_path)
    _write_data(d)
    mp.spawn(_worker, args=(2, 29751, d, 4), nprocs=2, join=True)
    ck = discover_latest_checkpoint(f"{d}/ckpt/eprun")
    assert ck is not None and (ck.endswith("step-3") or ck.endswith("step-4")), ck
    mp.spawn(_worker, args=(2, 29753, d, 8), nprocs=2, join=True)  # the same command continues from the saved step
    ck2 = discover_latest_checkpoint(f"{d}/ckpt/eprun")
    assert ck2 != ck and (ck2.endswith("step-7") or ck2.endswith("step-8")), ck2
