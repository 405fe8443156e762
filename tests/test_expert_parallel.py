"""Expert-parallel dispatch/combine over gloo ranks on CPU: two ranks, each holding half of the experts, must reproduce the
single-process MoE block (outputs and gradients)."""
import os
import sys

import torch
import torch.multiprocessing as mp


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from levanter_b200.models.mixtral import MixtralConfig, MixtralSparseMoeBlock
    from levanter_b200.parallel.expert import ExpertParallel

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = MixtralConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=1, num_heads=2, num_kv_heads=2,
                            n_routed_experts=4, num_experts_per_tok=2)
        torch.manual_seed(0)
        full = MixtralSparseMoeBlock(cfg)  # same weights on both ranks
        ep = ExpertParallel(None)
        torch.manual_seed(0)
        sharded = MixtralSparseMoeBlock(cfg, ep=ep)
        n_local = 4 // world
        with torch.no_grad():
            sharded.gate.weight.copy_(full.gate.weight)
            for name in ("w1", "w2", "w3"):
                getattr(sharded.experts, name).copy_(getattr(full.experts, name)[rank * n_local:(rank + 1) * n_local])
        g = torch.Generator().manual_seed(10 + rank)  # every rank routes its own tokens
        x = torch.randn(2, 16, 32, generator=g, requires_grad=True)
        y_ref, _ = full(x)
        gy = torch.randn(y_ref.shape, generator=g)
        y_ref.backward(gy)
        gx_ref = x.grad.clone()
        x.grad = None
        y, extras = sharded(x)
        y.backward(gy)
        ok = torch.allclose(y, y_ref, atol=1e-5) and torch.allclose(x.grad, gx_ref, atol=1e-5)
        # expert weight gradients: the shard's gradient sums the contributions of both ranks' tokens
        gw = sharded.experts.w1.grad.clone()
        ref_gw = full.experts.w1.grad.clone()
        dist.all_reduce(ref_gw)
        ok = ok and torch.allclose(gw, ref_gw[rank * n_local:(rank + 1) * n_local], atol=1e-5)
        torch.save({"ok": bool(ok), "err": float((y - y_ref).abs().max())}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_matches_local_moe(tmp_path):
    mp.spawn(_worker, args=(2, 29641, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"r{r}.pt")
        assert res["ok"], res
