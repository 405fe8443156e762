"""Prefill and decode throughput of the inference engine on one GPU:
``python -m levanter_b200.inference.bench_decode --model llama3_8b --seqs 64 --prompt-len 512 --new-tokens 128 [--cuda-graph]``,
or tensor-parallel over the GPUs of one node (one rank per GPU, heads / KV heads / MLP columns split over the ranks):
``python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m levanter_b200.inference.bench_decode --tp 8 --seqs 256
--prompt-min 128 --prompt-max 2048 --new-tokens 256 --cuda-graph``.

Random-init weights of the named architecture in bf16, synthetic uniform-random prompts, greedy decoding with stop tokens
disabled, so that every request produces exactly ``--new-tokens`` tokens.  The engine's own public entry point
(``InferenceEngine.generate``) is what is timed; phase times come from ``engine.stats`` (host clock after a device
synchronisation at the phase boundaries).  Prints one JSON line."""
from __future__ import annotations

import argparse
import json
import time

import numpy as np
import torch

MODELS = {
    "llama3_8b": dict(hidden_dim=4096, intermediate_dim=14336, num_layers=32, num_heads=32, num_kv_heads=8, vocab=128256),
    "llama2_7b": dict(hidden_dim=4096, intermediate_dim=11008, num_layers=32, num_heads=32, num_kv_heads=32, vocab=32000),
    "llama_1b": dict(hidden_dim=2048, intermediate_dim=8192, num_layers=16, num_heads=32, num_kv_heads=8, vocab=128256),
    "tiny": dict(hidden_dim=256, intermediate_dim=512, num_layers=2, num_heads=4, num_kv_heads=2, vocab=1024),
}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", choices=sorted(MODELS), default="llama3_8b")
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-rounds", type=int, default=16)
    ap.add_argument("--cuda-graph", action="store_true")
    ap.add_argument("--layers", type=int, default=None, help="override the number of layers (short profiler captures)")
    ap.add_argument("--repeats", type=int, default=2, help="timed generate() calls after one warm-up call")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (launch with torchrun, one rank per GPU)")
    ap.add_argument("--prompt-min", type=int, default=0, help="with --prompt-max: prompt lengths uniform in [min, max]")
    ap.add_argument("--prompt-max", type=int, default=0)
    ap.add_argument("--quiet", action="store_true", help="return the result without printing it")
    a = ap.parse_args(argv)
    return run(a)


def run(a):
    import os

    from ..data.passthrough_tokenizer import PassthroughTokenizer
    from ..models.llama import LlamaConfig
    from .engine import InferenceEngine, InferenceEngineConfig, Request
    from .jit_scheduler import SeqDecodingParams

    m = dict(MODELS[a.model])
    vocab = m.pop("vocab")
    if a.layers is not None:
        m["num_layers"] = a.layers
    prompt_max = a.prompt_max or a.prompt_len
    prompt_min = a.prompt_min or prompt_max
    total_len = prompt_max + a.new_tokens
    cfg = LlamaConfig(seq_len=max(total_len, 128), gradient_checkpointing=False, **m)
    rank, local_rank = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    tp = None
    if a.tp > 1:
        import torch.distributed as dist

        from ..parallel.mesh import DeviceMesh
        from ..parallel.tp import TensorParallel, shard_full_state_

        if not dist.is_initialized():
            dist.init_process_group("nccl" if dev.type == "cuda" else "gloo")
        assert dist.get_world_size() == a.tp, "launch one rank per tensor-parallel shard"
        tp = TensorParallel.from_mesh(DeviceMesh(1, 1, a.tp))
        # every rank builds the same unsharded random weights, keeps its shard and drops the rest
        full = cfg.build(vocab, seed=0, device=dev, dtype=dtype).eval()
        model = cfg.build(vocab, seed=1, device=dev, dtype=dtype, tp=tp).eval()
        shard_full_state_(model, {n: p.detach() for n, p in full.named_parameters()}, tp)
        del full
        if dev.type == "cuda":
            torch.cuda.empty_cache()
    else:
        model = cfg.build(vocab, seed=0, device=dev, dtype=dtype).eval()
    pages_per_seq = -(-total_len // a.page_size) + 1
    ecfg = InferenceEngineConfig(max_pages=a.seqs * pages_per_seq + 8, max_seqs=a.seqs, page_size=a.page_size, max_pages_per_seq=pages_per_seq,
                                 compute_dtype=dtype, max_seqs_in_prefill=min(a.seqs, 16), max_prefill_size=16 * prompt_max,
                                 max_rounds=a.max_rounds, use_cuda_graph=a.cuda_graph)
    engine = InferenceEngine.from_model_with_config(model, PassthroughTokenizer(vocab), ecfg)
    rng = np.random.default_rng(0)

    def requests():
        out = []
        for i in range(a.seqs):
            n = int(rng.integers(prompt_min, prompt_max + 1))
            out.append(Request(prompt_tokens=rng.integers(1, vocab - 1, n).tolist(), request_id=i,
                               decode_params=SeqDecodingParams(max_num_tokens=n + a.new_tokens, stop_tokens=None, temperature=0.0, key=i),
                               n_generations=1))
        return out

    with torch.no_grad():
        engine.generate(requests())  # warm-up (kernel attributes, graph capture, allocator)
        runs = []
        for _ in range(a.repeats):
            engine.reset()
            for k in engine.stats:
                engine.stats[k] = 0
            if dev.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = engine.generate(requests())
            if dev.type == "cuda":
                torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            st = dict(engine.stats)
            runs.append({"wall_s": wall, "generated": res.total_generated,
                         **st})
    device_round_ms = None
    if a.cuda_graph and engine._graph is not None:
        # the captured round alone, replayed back to back with no host work in between: pure device time per round
        # (the tables left in its static inputs are those of the last real round; token destinations are rewritten in place)
        g = engine._graph.graph
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(20):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        device_round_ms = e0.elapsed_time(e1) / 20
    if tp is not None:
        # a phase lasts as long as its slowest rank
        import torch.distributed as dist

        for r in runs:
            t = torch.tensor([r["wall_s"], r["prefill_seconds"], r["decode_seconds"]], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            r["wall_s"], r["prefill_seconds"], r["decode_seconds"] = (float(x) for x in t)
    best = min(runs, key=lambda r: r["wall_s"])
    out = {"metric": f"decode tokens/s (engine.generate, {a.tp} GPU{'s, tensor parallel' if a.tp > 1 else ''})", "model": a.model, "seqs": a.seqs,
           "prompt_len": a.prompt_len if not a.prompt_max else [prompt_min, prompt_max], "tp": a.tp,
           "kernel_all_reduces": None if tp is None else tp.kernel_all_reduces,
           "new_tokens": a.new_tokens, "page_size": a.page_size, "cuda_graph": bool(a.cuda_graph), "max_rounds": a.max_rounds, "dtype": str(dtype),
           "prefill_tokens_per_s": round(best["prefill_tokens"] / max(best["prefill_seconds"], 1e-9), 1),
           "decode_tokens_per_s": round(best["decode_tokens"] / max(best["decode_seconds"], 1e-9), 1),
           "end_to_end_generated_tokens_per_s": round(best["generated"] / best["wall_s"], 1),
           "ms_per_decode_round": round(1e3 * best["decode_seconds"] / max(best.get("decode_rounds", 0), 1), 3),
           "device_ms_per_round_graph_only": None if device_round_ms is None else round(device_round_ms, 3), "runs": runs}
    if rank == 0 and not a.quiet:
        print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
