"""Tensor-parallel inference over two gloo ranks: a model whose heads and MLP columns are split over the model axis, filled from
the unsharded weights, generates exactly the tokens of the unsharded model; every rank runs the same engine loop."""
import datetime
import json
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROMPTS = [[5, 9, 2, 11], [7, 8, 9, 10, 11, 12, 13], [40]]


def _generate(model):
    from levanter_b200.inference.engine import InferenceEngine, InferenceEngineConfig, Request
    from levanter_b200.inference.jit_scheduler import SeqDecodingParams

    ecfg = InferenceEngineConfig(max_seqs=4, page_size=4, max_pages_per_seq=8, compute_dtype=torch.float32, max_rounds=4, enable_logprobs=True)
    eng = InferenceEngine.from_model_with_config(model, None, ecfg)
    reqs = [Request(p, i, SeqDecodingParams(len(p) + 8, None, 0.0 if i != 1 else 0.7, 100 + i), 1) for i, p in enumerate(PROMPTS)]
    out = eng.generate(reqs)
    return out.tokens, out.logprobs


def _cfg():
    from levanter_b200.models.llama import LlamaConfig

    return LlamaConfig(seq_len=64, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=4, num_kv_heads=2, gradient_checkpointing=False)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      CUDA_VISIBLE_DEVICES="")
    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        from levanter_b200.parallel.mesh import DeviceMesh
        from levanter_b200.parallel.tp import TensorParallel, shard_full_state_

        mesh = DeviceMesh(1, 1, world)
        tp = TensorParallel.from_mesh(mesh)
        assert tp is not None and tp.size == world
        full = _cfg().build(60, seed=0).eval()
        model = _cfg().build(60, seed=1, tp=tp).eval()
        shard_full_state_(model, {n: p.detach() for n, p in full.named_parameters()}, tp)
        q = dict(model.named_parameters())["transformer.layers.0.self_attn.q_proj.weight"]
        assert q.shape[0] == dict(full.named_parameters())["transformer.layers.0.self_attn.q_proj.weight"].shape[0] // world
        with torch.no_grad():
            tokens, lps = _generate(model)
        json.dump({"tokens": tokens, "lps": lps}, open(f"{tmp}/r{rank}.json", "w"))
    finally:
        dist.destroy_process_group()


def test_two_way_tensor_parallel_generation_matches_the_unsharded_model(tmp_path):
    sys.path.insert(0, ROOT)
    with torch.no_grad():
        ref_tokens, ref_lps = _generate(_cfg().build(60, seed=0).eval())
    mp.spawn(_worker, args=(2, 29741, str(tmp_path)), nprocs=2, join=True)
    outs = [json.load(open(tmp_path / f"r{r}.json")) for r in range(2)]
    assert outs[0]["tokens"] == outs[1]["tokens"] == ref_tokens
    for a, b in zip(outs[0]["lps"], ref_lps):
        assert a == pytest.approx(b, abs=1e-4)
