"""The comparison arm of ``bench.py``: the same Llama-2 7B training step on stock PyTorch.

Nothing of ``levanter_b200`` is imported here.  The model is written with ``torch.nn`` modules only: ``nn.Embedding``,
``nn.Linear`` (cuBLAS), ``nn.RMSNorm``, rotary embedding as tensor ops, ``F.scaled_dot_product_attention`` (the library's
fused causal attention), SwiGLU, ``F.cross_entropy``.  Parallelism is ``torch.distributed.fsdp.fully_shard`` (per-layer
parameter sharding over NCCL, bf16 compute / fp32 parameters, gradients reduced in fp32), the optimizer is
``torch.optim.AdamW(fused=True)`` on the fp32 shards with global-norm clipping at 1.0, i.e. the same dtype policy, batch,
sequence length and optimizer as the framework's own arm.  The model runs eagerly (no ``torch.compile``).

The reference project itself (JAX) cannot be installed offline, so this is the "same mathematics on the vendor libraries"
baseline that the framework's numbers are divided by.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LlamaShape:
    vocab: int = 32000
    hidden: int = 4096
    intermediate: int = 11008
    layers: int = 32
    heads: int = 32
    kv_heads: int = 32
    seq_len: int = 4096
    rope_theta: float = 1e4
    eps: float = 1e-5
    init_std: float = 0.02


def _rope_tables(S: int, D: int, theta: float, device):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
    ang = torch.arange(S, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang), torch.sin(ang)


def _apply_rope(x, cos, sin):
    # x: [B, H, S, D]; rotate-half convention
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[None, None].to(x.dtype), sin[None, None].to(x.dtype)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


class Block(nn.Module):
    def __init__(self, c: LlamaShape):
        super().__init__()
        D = c.hidden // c.heads
        self.c = c
        self.ln1 = nn.RMSNorm(c.hidden, eps=c.eps)
        self.q = nn.Linear(c.hidden, c.heads * D, bias=False)
        self.k = nn.Linear(c.hidden, c.kv_heads * D, bias=False)
        self.v = nn.Linear(c.hidden, c.kv_heads * D, bias=False)
        self.o = nn.Linear(c.heads * D, c.hidden, bias=False)
        self.ln2 = nn.RMSNorm(c.hidden, eps=c.eps)
        self.gate = nn.Linear(c.hidden, c.intermediate, bias=False)
        self.up = nn.Linear(c.hidden, c.intermediate, bias=False)
        self.down = nn.Linear(c.intermediate, c.hidden, bias=False)

    def forward(self, x, cos, sin):
        c = self.c
        B, S, _ = x.shape
        D = c.hidden // c.heads
        h = self.ln1(x)
        q = self.q(h).view(B, S, c.heads, D).transpose(1, 2)
        k = self.k(h).view(B, S, c.kv_heads, D).transpose(1, 2)
        v = self.v(h).view(B, S, c.kv_heads, D).transpose(1, 2)
        q, k = _apply_rope(q, cos, sin), _apply_rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=c.kv_heads != c.heads)
        x = x + self.o(a.transpose(1, 2).reshape(B, S, c.heads * D))
        h = self.ln2(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


class Llama(nn.Module):
    def __init__(self, c: LlamaShape):
        super().__init__()
        self.c = c
        self.embed = nn.Embedding(c.vocab, c.hidden)
        self.blocks = nn.ModuleList([Block(c) for _ in range(c.layers)])
        self.norm = nn.RMSNorm(c.hidden, eps=c.eps)
        self.lm_head = nn.Linear(c.hidden, c.vocab, bias=False)

    def forward(self, tokens):
        c = self.c
        S = tokens.shape[1]
        cos, sin = _rope_tables(S, c.hidden // c.heads, c.rope_theta, tokens.device)
        x = self.embed(tokens)
        for b in self.blocks:
            x = b(x, cos, sin)
        return self.lm_head(self.norm(x))


def next_token_loss(model, tokens, loss_mask):
    logits = model(tokens)
    tgt = torch.roll(tokens, -1, dims=1).long()
    per = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), tgt.view(-1), reduction="none").view_as(tokens)
    m = loss_mask.to(per.dtype)
    return (per * m).sum() / m.sum().clamp_min(1.0)


def run(shape: LlamaShape, *, world: int, rank: int, device, per_gpu_batch: int, micro: int, steps: int, warmup: int,
        seed: int = 0, clock_sampler=None) -> dict:
    """W warm-up steps, then two timed regions of ``steps`` steps each (device-resident batch timed with CUDA events; pinned
    host batch copied in and loss read back every step, timed on the wall clock), both bracketed by barrier + synchronize and
    reduced with MAX over ranks.  The process group (NCCL) must be initialised, also for one rank."""
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    torch.manual_seed(seed)
    with torch.device("meta"):
        model = Llama(shape)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for blk in model.blocks:
        fully_shard(blk, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    model.to_empty(device=device)
    with torch.no_grad():
        g = torch.Generator(device=device)
        g.manual_seed(seed + 1 + rank)
        for name, p in model.named_parameters():
            local = p.to_local() if hasattr(p, "to_local") else p
            if "ln" in name or name.startswith("norm"):
                local.fill_(1.0)
            else:
                local.normal_(0.0, shape.init_std, generator=g)
    n_params = sum(p.numel() for p in model.parameters())
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: min(1.0, (s + 1) / 100))
    S, B = shape.seq_len, per_gpu_batch
    n_micro = B // micro

    def step(tokens, mask):
        total = torch.zeros((), dtype=torch.float32, device=device)
        for i in range(n_micro):
            loss = next_token_loss(model, tokens[i * micro:(i + 1) * micro], mask[i * micro:(i + 1) * micro])
            (loss / n_micro).backward()
            total += loss.detach().float() / n_micro
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        sched.step()
        opt.zero_grad(set_to_none=True)
        if world > 1:
            dist.all_reduce(total, op=dist.ReduceOp.AVG)
        return total

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    gen = torch.Generator().manual_seed(1234 + rank)

    def host_batch():
        t = torch.randint(0, shape.vocab, (B, S), generator=gen, dtype=torch.int32).pin_memory()
        m = torch.ones(B, S, dtype=torch.float32)
        m[:, -1] = 0
        return t, m.pin_memory()

    t0, m0 = host_batch()
    dt, dm = t0.to(device), m0.to(device)
    for _ in range(warmup):
        step(dt, dm)
    sync()
    if clock_sampler is not None:
        clock_sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for _ in range(steps):
        step(dt, dm)
    e1.record()
    sync()
    dev_ms = e0.elapsed_time(e1)
    clocks = clock_sampler.stop() if clock_sampler is not None else None

    batches = [host_batch() for _ in range(steps + 1)]
    h2d = sum(t.numel() * t.element_size() for t in batches[0])
    loss = step(batches[0][0].to(device, non_blocking=True), batches[0][1].to(device, non_blocking=True)).item()
    sync()
    w0 = time.perf_counter()
    for k in range(steps):
        t, m = batches[k + 1]
        loss = step(t.to(device, non_blocking=True), m.to(device, non_blocking=True)).item()
    sync()
    e2e_ms = (time.perf_counter() - w0) * 1e3
    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=device)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    tokens_per_step = B * world * S
    out = {
        "value": tokens_per_step * steps / (dev_ms / 1e3), "ms_per_step": dev_ms / steps,
        "e2e_value": tokens_per_step * steps / (e2e_ms / 1e3), "e2e_ms_per_step": e2e_ms / steps,
        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "final_loss": loss, "params": n_params, "microbatch_per_gpu": micro,
        "peak_mem_gib": torch.cuda.max_memory_allocated() / 2**30, "clocks": clocks, "steps": steps, "warmup": warmup,
        "ln_vocab": math.log(shape.vocab),
    }
    del model, opt
    return out
