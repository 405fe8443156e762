"""Micro-benchmarks of this library's kernels: ``python -m levanter_b200.ops.bench_kernels <kernel> [options]``.

Each kernel is timed with CUDA events on the launching stream after warm-up iterations, with a buffer larger than the L2
cache rewritten between timed iterations (``--no-flush`` turns that off), and reported as achieved TFLOP/s or GB/s and as a
fraction of the measured peaks in ``MEASURED_PEAKS.json`` at the repository root (falling back to 1.59 PFLOP/s and
6.65 TB/s when the file is absent).  ``--once`` runs warm-up plus a single launch, which is the shape of run a profiler
capture wants."""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics

import torch


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        p = json.load(open(path))
        return p.get("bf16_tflops", 1590.0), p.get("hbm_gbs", 6650.0), "measured"
    except Exception:  # noqa: BLE001
        return 1590.0, 6650.0, "fallback"


def _time(fn, iters: int, warmup: int, flush: bool):
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if scratch is not None:
            scratch.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times), min(times)


def _report(name, cfg, ms, ms_min, flops=None, nbytes=None):
    tf_peak, bw_peak, how = _peaks()
    out = {"kernel": name, "config": cfg, "ms_median": round(ms, 4), "ms_min": round(ms_min, 4)}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out[f"frac_of_{how}_bf16_peak"] = round(flops / ms / 1e9 / tf_peak, 3)
    if nbytes:
        out["gbs"] = round(nbytes / ms / 1e6, 1)
        out[f"frac_of_{how}_hbm_peak"] = round(nbytes / ms / 1e6 / bw_peak, 3)
    print(json.dumps(out))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm", "gemm_fp8", "gemm_mxfp8", "mxfp8_quant", "flash_fwd", "flash_bwd", "rmsnorm", "cross_entropy", "adamw", "paged_attention", "sampler", "moe_mlp", "delta_rule", "rmsnorm_bwd", "rope", "dwconv", "entropy", "histogram", "gdn_layer"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=None)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--context", type=int, default=4096, help="paged attention: tokens already in the cache per sequence")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--head-dim", type=int, default=128, help="flash attention: 64 or 128")
    ap.add_argument("--not-causal", action="store_true", help="flash attention: every key visible (encoder attention)")
    ap.add_argument("--sdpa", action="store_true", help="flash attention: time the library's fused attention instead (comparison row)")
    ap.add_argument("--bn", type=int, default=0, help="gemm_mxfp8: tile width 128 or 256 (0: chosen by the launcher)")
    ap.add_argument("--once", action="store_true", help="warm-up plus one launch (for profiler captures)")
    a = ap.parse_args(argv)
    from . import lib

    assert lib.available(), "needs a B200 and the built kernel library"
    if a.once:
        a.iters = 1
    torch.manual_seed(0)
    dev = "cuda"
    flush = not a.no_flush
    bf = torch.bfloat16

    if a.kernel == "gemm":
        from .gemm import gemm

        A = torch.randn(a.m, a.k, device=dev, dtype=bf)
        B = torch.randn(a.n, a.k, device=dev, dtype=bf)
        C = torch.empty(a.m, a.n, device=dev, dtype=bf)
        ms, mn = _time(lambda: gemm(A, B, out=C), a.iters, a.warmup, flush)
        return _report("gemm_bf16", {"m": a.m, "n": a.n, "k": a.k}, ms, mn, flops=2.0 * a.m * a.n * a.k)

    if a.kernel == "gemm_fp8":
        from .fp8 import E4M3, fp8_gemm, quantize

        A, sa = quantize(torch.randn(a.m, a.k, device=dev), E4M3)
        B, sb = quantize(torch.randn(a.n, a.k, device=dev), E4M3)
        C = torch.empty(a.m, a.n, device=dev, dtype=bf)
        sc = sa * sb
        ms, mn = _time(lambda: fp8_gemm(A, B, sc, out=C), a.iters, a.warmup, flush)
        return _report("gemm_fp8_e4m3", {"m": a.m, "n": a.n, "k": a.k}, ms, mn, flops=2.0 * a.m * a.n * a.k)

    if a.kernel == "gemm_mxfp8":
        from .fp8 import E4M3, mx_gemm, mx_quantize

        A, sa, _, _ = mx_quantize(torch.randn(a.m, a.k, device=dev, dtype=bf), E4M3)
        B, sb, _, _ = mx_quantize(torch.randn(a.n, a.k, device=dev, dtype=bf), E4M3)
        C = torch.empty(a.m, a.n, device=dev, dtype=bf)
        ms, mn = _time(lambda: mx_gemm(A, sa, B, sb, out=C, bn=a.bn), a.iters, a.warmup, flush)
        return _report("gemm_mxfp8_e4m3_block32", {"m": a.m, "n": a.n, "k": a.k, "bn": a.bn}, ms, mn, flops=2.0 * a.m * a.n * a.k)

    if a.kernel == "mxfp8_quant":
        from .fp8 import E4M3, mx_quantize

        X = torch.randn(a.m, a.k, device=dev, dtype=bf)
        ms, mn = _time(lambda: mx_quantize(X, E4M3, True, True), a.iters, a.warmup, flush)
        # read bf16 once, write the fp8 tensor and its transpose (+ 1/16 of that in scales)
        return _report("mxfp8_quantize_both_directions", {"rows": a.m, "cols": a.k}, ms, mn, nbytes=a.m * a.k * (2 + 2 + 2 / 32))

    if a.kernel in ("flash_fwd", "flash_bwd"):
        from ..layers.attention import AttentionMask
        from ._flash_impl import flash_attention_cuda

        kvh = a.kv_heads or a.heads
        hd = a.head_dim
        q = torch.randn(a.batch, a.seq, a.heads, hd, device=dev, dtype=bf, requires_grad=True)
        k = torch.randn(a.batch, a.seq, kvh, hd, device=dev, dtype=bf, requires_grad=True)
        v = torch.randn(a.batch, a.seq, kvh, hd, device=dev, dtype=bf, requires_grad=True)
        causal = not a.not_causal
        mask = AttentionMask.causal() if causal else None
        causal_flops = 4.0 * a.batch * a.heads * a.seq * a.seq * hd / (2 if causal else 1)
        cfg = {"batch": a.batch, "seq": a.seq, "heads": a.heads, "kv_heads": kvh, "head_dim": hd, "causal": causal, "impl": "library sdpa" if a.sdpa else "own"}
        if a.sdpa:
            # the library's fused attention on the same tensors (the comparison row; not this framework's kernel)
            import torch.nn.functional as F

            rep = a.heads // kvh

            def attn(q, k, v):
                kk, vv = (k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)) if rep > 1 else (k, v)
                return F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=causal).transpose(1, 2)
        else:
            def attn(q, k, v):
                return flash_attention_cuda(q, k, v, mask)
        if a.kernel == "flash_fwd":
            with torch.no_grad():
                ms, mn = _time(lambda: attn(q, k, v), a.iters, a.warmup, flush)
            return _report("flash_attention_fwd", cfg, ms, mn, flops=causal_flops)
        o = attn(q, k, v)
        g = torch.randn_like(o)
        ms, mn = _time(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True), a.iters, a.warmup, flush)
        return _report("flash_attention_bwd", cfg, ms, mn, flops=2.5 * causal_flops)

    if a.kernel == "rmsnorm":
        from .norm import rms_norm

        rows = a.batch * a.seq
        x = torch.randn(rows, a.hidden, device=dev, dtype=bf)
        w = torch.ones(a.hidden, device=dev, dtype=torch.float32)
        with torch.no_grad():
            ms, mn = _time(lambda: rms_norm(x, w, None, 1e-5), a.iters, a.warmup, flush)
        return _report("rmsnorm_fwd", {"rows": rows, "hidden": a.hidden}, ms, mn, nbytes=2.0 * rows * a.hidden * 2)

    if a.kernel == "cross_entropy":
        from .cross_entropy import fused_linear_cross_entropy

        rows = a.batch * a.seq
        x = torch.randn(rows, a.hidden, device=dev, dtype=bf, requires_grad=True)
        w = (torch.randn(a.vocab, a.hidden, device=dev, dtype=bf) * 0.02).requires_grad_()
        y = torch.randint(0, a.vocab, (rows,), device=dev)

        def step():
            loss, _ = fused_linear_cross_entropy(x, w, y)
            loss.mean().backward()

        ms, mn = _time(step, a.iters, a.warmup, flush)
        return _report("fused_linear_cross_entropy_fwd_bwd", {"rows": rows, "hidden": a.hidden, "vocab": a.vocab}, ms, mn,
                       flops=(2.0 + 2.0 + 4.0) * rows * a.hidden * a.vocab)

    if a.kernel == "adamw":
        from .optim_kernels import adamw

        n = a.m * a.n
        p = torch.randn(n, device=dev)
        m = torch.zeros(n, device=dev)
        v = torch.zeros(n, device=dev)
        g = torch.randn(n, device=dev)
        pb = torch.empty(n, device=dev, dtype=bf)
        ms, mn = _time(lambda: adamw(p, m, v, g, pb, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** 3, 1 - 0.95 ** 3, None), a.iters, a.warmup, flush)
        return _report("fused_adamw", {"n": n}, ms, mn, nbytes=n * (4 * 4 + 3 * 4 + 2.0))

    if a.kernel == "paged_attention":
        from . import paged_attention as PA

        kvh = a.kv_heads or a.heads
        S, ps = a.batch, 16
        pps = (a.context + ps) // ps + 1
        P = S * pps
        kv = torch.randn(P, ps, 2 * kvh, 128, device=dev, dtype=bf)
        pages = torch.arange(P, device=dev, dtype=torch.int32).reshape(S, pps)
        lens = torch.full((S,), a.context + 1, device=dev, dtype=torch.int32)
        cu = torch.arange(S + 1, device=dev, dtype=torch.int32)
        q = torch.randn(S, a.heads, 128, device=dev, dtype=bf)
        n = torch.tensor(S, device=dev, dtype=torch.int32)
        ms, mn = _time(lambda: PA.ragged_paged_attention(q, kv, lens, pages, cu, n, sm_scale=1 / math.sqrt(128)), a.iters, a.warmup, flush)
        return _report("paged_attention_decode", {"seqs": S, "context": a.context, "heads": a.heads, "kv_heads": kvh}, ms, mn,
                       nbytes=2.0 * S * (a.context + 1) * kvh * 128 * 2)

    if a.kernel == "moe_mlp":
        # Mixtral-style expert MLP, forward + backward: one grouped launch per projection against a launch per expert
        from ..utils.activation import ActivationFunctionEnum
        from .moe import grouped_mlp, grouped_mlp_padded

        T, E, k, H, M = a.batch * a.seq, 8, 2, a.hidden, a.n if a.n != 8192 else 14336
        x = (torch.randn(T, H, device=dev) * 0.5).to(bf).requires_grad_()
        w1, w3 = ((torch.randn(E, M, H, device=dev) * 0.02).to(bf).requires_grad_() for _ in range(2))
        w2 = (torch.randn(E, H, M, device=dev) * 0.02).to(bf).requires_grad_()
        idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)])
        act = ActivationFunctionEnum.silu

        def grouped():
            grouped_mlp_padded(x, idx, w1, w3, w2, act).sum().backward()

        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)

        def looped():
            sizes = torch.bincount(flat, minlength=E)  # read back by the loop: one host synchronisation per call
            grouped_mlp(x.index_select(0, order // k), sizes, w1, w3, w2, act).sum().backward()

        flops = 3 * 3 * 2.0 * T * k * H * M  # three projections, forward + two backward GEMMs each
        ms_g, mn_g = _time(grouped, a.iters, a.warmup, flush)
        ms_l, mn_l = _time(looped, a.iters, a.warmup, flush)
        cfg = {"tokens": T, "experts": E, "top_k": k, "hidden": H, "mlp": M}
        _report("moe_mlp_grouped_fwd_bwd", cfg, ms_g, mn_g, flops=flops)
        return _report("moe_mlp_per_expert_loop_fwd_bwd", cfg, ms_l, mn_l, flops=flops)

    if a.kernel == "delta_rule":
        # the carried-state loop of the gated delta rule: one launch per direction against the same loop on framework ops
        from .delta_rule import chunk_state_scan, chunk_state_scan_reference

        B, H, N, C, dk, dv = a.batch, a.heads, a.seq // 64, 64, 128, 128
        w, qg, kd = ((torch.randn(B, H, N, C, dk, device=dev) * 0.02).requires_grad_() for _ in range(3))
        P = (torch.randn(B, H, N, C, C, device=dev) * 0.1).tril().requires_grad_()
        u = torch.randn(B, H, N, C, dv, device=dev).requires_grad_()
        dec = torch.rand(B, H, N, device=dev).mul(0.4).add(0.4).requires_grad_()  # contraction: the state stays bounded
        cfg = {"batch": B, "heads": H, "seq": N * C, "d_k": dk, "d_v": dv}
        per_chunk = 2.0 * C * dk * dv * 3 + 2.0 * C * C * dv  # w S, qg S, kd^T v_new, P v_new
        flops = B * H * N * per_chunk
        tile_bytes = 4.0 * B * H * N * (3 * C * dk + C * C + 2 * C * dv)

        def fwd():
            with torch.no_grad():
                chunk_state_scan(w, qg, kd, P, u, dec)

        def fwd_ops():
            with torch.no_grad():
                chunk_state_scan_reference(w, qg, kd, P, u, dec)

        def fwd_bwd():
            chunk_state_scan(w, qg, kd, P, u, dec)[0].sum().backward()

        def fwd_bwd_ops():
            chunk_state_scan_reference(w, qg, kd, P, u, dec)[0].sum().backward()

        if a.once:
            fwd(); fwd_bwd(); torch.cuda.synchronize()
            return None
        ms, mn = _time(fwd, a.iters, a.warmup, flush)
        _report("delta_rule_scan_fwd", cfg, ms, mn, flops=flops, nbytes=tile_bytes)
        ms, mn = _time(fwd_ops, max(a.iters // 4, 2), 2, flush)
        _report("delta_rule_scan_fwd_framework_ops", cfg, ms, mn, flops=flops)
        ms, mn = _time(fwd_bwd, a.iters, a.warmup, flush)
        _report("delta_rule_scan_fwd_bwd", cfg, ms, mn, flops=3 * flops)
        ms, mn = _time(fwd_bwd_ops, max(a.iters // 4, 2), 2, flush)
        return _report("delta_rule_scan_fwd_bwd_framework_ops", cfg, ms, mn, flops=3 * flops)

    if a.kernel == "rmsnorm_bwd":
        from .norm import rms_norm

        rows = a.batch * a.seq
        x = torch.randn(rows, a.hidden, device=dev, dtype=bf, requires_grad=True)
        w = torch.ones(a.hidden, device=dev, dtype=torch.float32, requires_grad=True)
        gy = torch.randn(rows, a.hidden, device=dev, dtype=bf)

        def step():
            x.grad = None
            rms_norm(x, w, None, 1e-5).backward(gy)

        ms, mn = _time(step, a.iters, a.warmup, flush)
        # forward reads x, writes y; backward reads x, dy, writes dx
        return _report("rmsnorm_fwd_bwd", {"rows": rows, "hidden": a.hidden}, ms, mn, nbytes=5.0 * rows * a.hidden * 2)

    if a.kernel == "rope":
        from ..layers.rotary import DefaultRotaryEmbeddingsConfig
        from .rope import apply_rope

        kv = a.kv_heads or a.heads
        q = torch.randn(a.batch, a.seq, a.heads, 128, device=dev, dtype=bf)
        k = torch.randn(a.batch, a.seq, kv, 128, device=dev, dtype=bf)
        rot = DefaultRotaryEmbeddingsConfig().build(128)
        with torch.no_grad():
            ms, mn = _time(lambda: apply_rope(q, k, rot), a.iters, a.warmup, flush)
        return _report("rope_q_and_k", {"batch": a.batch, "seq": a.seq, "heads": a.heads, "kv_heads": kv}, ms, mn,
                       nbytes=2.0 * 2 * a.batch * a.seq * (a.heads + kv) * 128)

    if a.kernel == "dwconv":
        from .dwconv import causal_dwconv, causal_dwconv_reference

        x = torch.randn(a.batch, a.seq, a.hidden, device=dev, dtype=bf, requires_grad=True)
        w = (torch.randn(a.hidden, 1, 4, device=dev) * 0.5).requires_grad_()
        gy = torch.randn(a.batch, a.seq, a.hidden, device=dev, dtype=bf)
        cfg = {"batch": a.batch, "seq": a.seq, "channels": a.hidden, "k": 4, "act": "silu"}
        nb = 2.0 * a.batch * a.seq * a.hidden
        with torch.no_grad():
            ms, mn = _time(lambda: causal_dwconv(x, w, None, True), a.iters, a.warmup, flush)
        _report("dwconv_silu_fwd", cfg, ms, mn, nbytes=2 * nb)
        if a.once:
            causal_dwconv(x, w, None, True).backward(gy)
            return None
        wb = w.detach().to(bf).requires_grad_()
        with torch.no_grad():
            ms, mn = _time(lambda: causal_dwconv_reference(x, wb, None, True), a.iters, a.warmup, flush)
        _report("dwconv_silu_fwd_library_conv1d", cfg, ms, mn, nbytes=2 * nb)

        def step(fn, weight):
            x.grad = None
            fn(x, weight, None, True).backward(gy)

        ms, mn = _time(lambda: step(causal_dwconv, w), a.iters, a.warmup, flush)
        # forward: x, y; gradient prologue: x, dy, dpre; input gradient: dpre, dx
        _report("dwconv_silu_fwd_bwd", cfg, ms, mn, nbytes=7 * nb)
        ms, mn = _time(lambda: step(causal_dwconv_reference, wb), a.iters, a.warmup, flush)
        return _report("dwconv_silu_fwd_bwd_library_conv1d", cfg, ms, mn, nbytes=7 * nb)

    if a.kernel == "entropy":
        from .analysis_kernels import entropy_top2, entropy_top2_reference

        rows = a.batch * a.seq
        z = torch.randn(rows, a.vocab, device=dev, dtype=bf)
        cfg = {"rows": rows, "vocab": a.vocab}
        ms, mn = _time(lambda: entropy_top2(z), a.iters, a.warmup, flush)
        _report("entropy_top2_lse", cfg, ms, mn, nbytes=2.0 * rows * a.vocab)
        if a.once:
            return None
        ms, mn = _time(lambda: entropy_top2_reference(z), max(a.iters // 4, 2), 2, flush)
        return _report("entropy_top2_lse_framework_ops", cfg, ms, mn, nbytes=2.0 * rows * a.vocab)

    if a.kernel == "histogram":
        from ..tracker.histogram import Histogram

        n = a.m * a.n
        x = torch.randn(n, device=dev)
        ms, mn = _time(lambda: Histogram.from_array(x), a.iters, a.warmup, flush)  # includes the read-back of the result
        return _report("summary_and_histogram_31_bins", {"elements": n}, ms, mn, nbytes=2 * 4.0 * n)

    if a.kernel == "gdn_layer":
        # one gated delta-rule token mixer (projections, short convolutions, scan, gated norm), forward + backward, with the
        # scan and convolution kernels against the same layer on framework ops
        from ..models import gated_deltanet as G
        from .delta_rule import chunk_state_scan_reference
        from .dwconv import causal_dwconv_reference

        cfg = G.GatedDeltaNetConfig(seq_len=a.seq, hidden_dim=a.hidden, num_heads=a.heads, head_k_dim=128, head_v_dim=128, num_layers=1)
        with torch.device(dev):
            layer = G.GatedDeltaNetLayer(cfg).bfloat16()
        x = torch.randn(a.batch, a.seq, a.hidden, device=dev, dtype=bf, requires_grad=True)
        gy = torch.randn(a.batch, a.seq, a.hidden, device=dev, dtype=bf)

        def step():
            x.grad = None
            layer(x).backward(gy)

        shape = {"batch": a.batch, "seq": a.seq, "hidden": a.hidden, "heads": a.heads}
        ms, mn = _time(step, a.iters, a.warmup, flush)
        _report("gated_deltanet_layer_fwd_bwd", shape, ms, mn)
        kernels = (G.chunk_state_scan, G.causal_dwconv)
        G.chunk_state_scan, G.causal_dwconv = chunk_state_scan_reference, causal_dwconv_reference
        try:
            ms, mn = _time(step, max(a.iters // 4, 2), 2, flush)
        finally:
            G.chunk_state_scan, G.causal_dwconv = kernels
        return _report("gated_deltanet_layer_fwd_bwd_framework_ops", shape, ms, mn)

    if a.kernel == "sampler":
        from ..layers.sampler import Sampler

        z = torch.randn(a.batch, a.vocab, device=dev, dtype=bf)
        t = torch.full((a.batch,), 0.7, device=dev)
        seeds = torch.arange(a.batch, device=dev, dtype=torch.int64)
        s = Sampler()
        ms, mn = _time(lambda: s._cuda(z, t, seeds), a.iters, a.warmup, flush)
        return _report("sampler", {"rows": a.batch, "vocab": a.vocab}, ms, mn, nbytes=2.0 * a.batch * a.vocab)


if __name__ == "__main__":
    main()
