"""Prefill and decode throughput of the inference engine on one GPU:
``python -m levanter_b200.inference.bench_decode --model llama3_8b --seqs 64 --prompt-len 512 --new-tokens 128 [--cuda-graph]``.

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
    a = ap.parse_args(argv)

    from ..data.passthrough_tokenizer import PassthroughTokenizer
    from ..models.llama import LlamaConfig
    from .engine import InferenceEngine, InferenceEngineConfig, Request
    from .jit_scheduler import SeqDecodingParams

    m = dict(MODELS[a.model])
    vocab = m.pop("vocab")
    if a.layers is not None:
        m["num_layers"] = a.layers
    total_len = a.prompt_len + a.new_tokens
    cfg = LlamaConfig(seq_len=max(total_len, 128), gradient_checkpointing=False, **m)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = cfg.build(vocab, seed=0, device=dev, dtype=dtype).eval()
    pages_per_seq = -(-total_len // a.page_size) + 1
    ecfg = InferenceEngineConfig(max_pages=a.seqs * pages_per_seq + 8, max_seqs=a.seqs, page_size=a.page_size, max_pages_per_seq=pages_per_seq,
                                 compute_dtype=dtype, max_seqs_in_prefill=min(a.seqs, 16), max_prefill_size=16 * a.prompt_len,
                                 max_rounds=a.max_rounds, use_cuda_graph=a.cuda_graph)
    engine = InferenceEngine.from_model_with_config(model, PassthroughTokenizer(vocab), ecfg)
    rng = np.random.default_rng(0)

    def requests():
        return [Request(prompt_tokens=rng.integers(1, vocab - 1, a.prompt_len).tolist(), request_id=i,
                        decode_params=SeqDecodingParams(max_num_tokens=total_len, stop_tokens=None, temperature=0.0, key=i),
                        n_generations=1) for i in range(a.seqs)]

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
    best = min(runs, key=lambda r: r["wall_s"])
    out = {"metric": "decode tokens/s (engine.generate, 1 GPU)", "model": a.model, "seqs": a.seqs, "prompt_len": a.prompt_len,
           "new_tokens": a.new_tokens, "page_size": a.page_size, "cuda_graph": bool(a.cuda_graph), "max_rounds": a.max_rounds, "dtype": str(dtype),
           "prefill_tokens_per_s": round(best["prefill_tokens"] / max(best["prefill_seconds"], 1e-9), 1),
           "decode_tokens_per_s": round(best["decode_tokens"] / max(best["decode_seconds"], 1e-9), 1),
           "end_to_end_generated_tokens_per_s": round(best["generated"] / best["wall_s"], 1),
           "ms_per_decode_round": round(1e3 * best["decode_seconds"] / max(best.get("decode_rounds", 0), 1), 3),
           "device_ms_per_round_graph_only": None if device_round_ms is None else round(device_round_ms, 3), "runs": runs}
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
