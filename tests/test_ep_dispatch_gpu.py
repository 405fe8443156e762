"""Expert-parallel exchange kernels.  On one GPU several buffers stand in for the ranks (the kernels never wait on one
another, so the ranks' launches run one after the other); on two GPUs the sharded MoE block on the peer-memory exchange is
compared with the unsharded block and with the all-to-all path, outputs and gradients, with timings."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _expected_layout(assign, W, E):
    """assign[r]: expert of every (token, choice) pair of rank r.  Returns per owner rank the list of (source rank, pair)
    in buffer order with None for padding rows, and the padded offsets."""
    n_local = E // W
    layouts, offsets = [], []
    for d in range(W):
        rows, off = [], [0]
        for le in range(n_local):
            ge = d * n_local + le
            for r in range(W):
                order = torch.argsort(assign[r], stable=True).tolist()
                rows += [(r, p) for p in order if assign[r][p] == ge]
            while len(rows) % 128:
                rows.append(None)
            off.append(len(rows))
        layouts.append(rows)
        offsets.append(off)
    return layouts, offsets


@pytest.mark.parametrize("W,E,T,k,H", [(2, 4, 300, 2, 256), (4, 8, 517, 2, 128), (2, 8, 64, 1, 64), (8, 8, 200, 2, 128)])
def test_exchange_kernels_with_ranks_emulated_on_one_device(W, E, T, k, H):
    from levanter_b200.ops import ep_dispatch as K
    from levanter_b200.ops import lib

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(W * 100 + E)
    n_local = E // W
    R = T * k
    cap = K.capacity_rows(R, n_local, 3.0)
    x = [torch.randn(T, H, device=dev, generator=g).bfloat16() for _ in range(W)]
    assign = [torch.randint(0, E, (R,), device=dev, generator=g) for _ in range(W)]
    assign[0][assign[0] == E - 1] = 0  # one expert gets nothing from rank 0
    sort_idx = [torch.argsort(a, stable=True) for a in assign]
    counts = [torch.bincount(a, minlength=E).int() for a in assign]
    tables = [torch.zeros(W * E, dtype=torch.int32, device=dev) for _ in range(W)]
    bufs = [torch.full((cap, H), 7.0, device=dev).bfloat16() for _ in range(W)]  # stale contents the kernels must not leave
    tptr, bptr = K.ptr_array([t.data_ptr() for t in tables]), K.ptr_array([b.data_ptr() for b in bufs])
    for r in range(W):
        K.counts_push(counts[r], tptr, W, r)
    for t in tables:
        assert torch.equal(t.view(W, E), torch.stack(counts))
    offsets = [torch.empty(n_local + 1, dtype=torch.int32, device=dev) for _ in range(W)]
    tile_group = [torch.empty(cap // 128, dtype=torch.int32, device=dev) for _ in range(W)]
    for r in range(W):
        K.rows(True, tables[r], W, r, x[r], sort_idx[r], k, bptr, R, cap, offsets[r], tile_group[r], True)
    lib.check_status()
    layouts, offs = _expected_layout([a.cpu() for a in assign], W, E)
    for d in range(W):
        assert offsets[d].tolist() == offs[d]
        want = torch.zeros(len(layouts[d]), H, dtype=torch.bfloat16, device=dev)
        for i, item in enumerate(layouts[d]):
            if item is not None:
                want[i] = x[item[0]][item[1] // k]
        assert torch.equal(bufs[d][:len(layouts[d])], want)
        tg = tile_group[d].tolist()
        for b, grp in enumerate(tg):
            lo = b * 128
            exp = next((le for le in range(n_local) if offs[d][le] <= lo < offs[d][le + 1]), -1)
            assert grp == exp
    # the way back: what every pair's row became on its owner returns in (token, choice) order
    for d in range(W):
        bufs[d].mul_(2)
    for r in range(W):
        out = torch.empty(R, H, dtype=torch.bfloat16, device=dev)
        K.rows(False, tables[r], W, r, out, sort_idx[r], 1, bptr, R, cap)
        assert torch.equal(out, (x[r].repeat_interleave(k, dim=0).float() * 2).bfloat16())
    lib.check_status()


def test_rows_beyond_capacity_are_dropped_and_reported():
    from levanter_b200.ops import ep_dispatch as K
    from levanter_b200.ops import lib

    dev = torch.device("cuda")
    W, E, T, k, H = 2, 2, 256, 1, 64
    x = [torch.ones(T, H, device=dev).bfloat16() for _ in range(W)]
    assign = [torch.zeros(T, dtype=torch.long, device=dev) for _ in range(W)]  # every row goes to rank 0
    cap = 384  # 512 rows arrive
    tables = [torch.zeros(W * E, dtype=torch.int32, device=dev) for _ in range(W)]
    bufs = [torch.zeros(cap + 128, H, device=dev).bfloat16() for _ in range(W)]  # a guard block past the capacity
    tptr, bptr = K.ptr_array([t.data_ptr() for t in tables]), K.ptr_array([b.data_ptr() for b in bufs])
    for r in range(W):
        K.counts_push(torch.bincount(assign[r], minlength=E).int(), tptr, W, r)
    idx = torch.arange(T, device=dev)
    for r in range(W):
        K.rows(True, tables[r], W, r, x[r], idx, 1, bptr, T, cap, None, None, False)
    torch.cuda.synchronize()
    with pytest.raises(lib.KernelStatusError):
        lib.check_status()
    assert bufs[0][:cap].float().sum().item() == cap * H and bufs[0][cap:].float().abs().sum().item() == 0
    out = torch.full((T, H), 5.0, device=dev).bfloat16()
    K.rows(False, tables[1], W, 1, out, idx, 1, bptr, T, cap)
    torch.cuda.synchronize()
    lib.clear_status()
    assert out[:128].float().sum().item() == 128 * H and out[128:].float().abs().sum().item() == 0  # rank 1's rows 128.. were dropped


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from levanter_b200.models.mixtral import MixtralConfig, MixtralSparseMoeBlock
    from levanter_b200.ops import lib
    from levanter_b200.parallel.expert import ExpertParallel

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        res = {"errs": {}, "times": {}}

        def build(hidden, inter, E, with_full=True):
            cfg = MixtralConfig(seq_len=64, hidden_dim=hidden, intermediate_dim=inter, num_layers=1, num_heads=2, num_kv_heads=2,
                                n_routed_experts=E, num_experts_per_tok=2)
            torch.manual_seed(0)
            ep = ExpertParallel(None)
            n_local = E // world
            with torch.device(dev):  # initialise on the GPU: the large case has billions of weights
                sharded = MixtralSparseMoeBlock(cfg, ep=ep).bfloat16()
                if not with_full:
                    return None, sharded, ep, n_local
                full = MixtralSparseMoeBlock(cfg).bfloat16()  # same seed, hence the same weights, on every rank
            with torch.no_grad():
                sharded.gate.weight.copy_(full.gate.weight)
                for name in ("w1", "w2", "w3"):
                    getattr(sharded.experts, name).copy_(getattr(full.experts, name)[rank * n_local:(rank + 1) * n_local])
            return full, sharded, ep, n_local

        full, sharded, ep, n_local = build(256, 512, 4)
        g = torch.Generator(device=dev).manual_seed(10 + rank)  # every rank routes its own tokens
        x = torch.randn(3, 64, 256, device=dev, generator=g).bfloat16().requires_grad_()
        gy = torch.randn(3, 64, 256, device=dev, generator=g).bfloat16()

        def run(block):
            x.grad = None
            for p in block.parameters():
                p.grad = None
            y, _ = block(x)
            y.backward(gy)
            return y.detach().float(), x.grad.float().clone(), block.experts.w1.grad.float().clone()

        y_ref, gx_ref, gw_ref = run(full)
        dist.all_reduce(gw_ref)  # the shard's weight gradient sums the contributions of both ranks' tokens
        gw_ref = gw_ref[rank * n_local:(rank + 1) * n_local]
        for comm in ("peer", "nccl"):
            os.environ["LEVANTER_B200_EP_COMM"] = comm
            n0 = lib.launch_count
            y, gx, gw = run(sharded)
            used = getattr(ep, "_exchanges", None)
            assert (comm == "peer") == bool(used) or comm == "nccl"
            rel = lambda a, b: float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))  # noqa: E731
            res["errs"][comm] = (rel(y, y_ref), rel(gx, gx_ref), rel(gw, gw_ref))
            res["launches_" + comm] = lib.launch_count - n0
        lib.check_status()
        del full, sharded

        # timing at Mixtral's layer shape: 8192 tokens per rank, top-2 of 8 experts, hidden 4096, MLP 14336
        _, big, ep2, _ = build(4096, 14336, 8, with_full=False)
        xb = torch.randn(2, 4096, 4096, device=dev).bfloat16().requires_grad_()
        gb = torch.randn(2, 4096, 4096, device=dev).bfloat16()

        def step():
            y, _ = big(xb)
            y.backward(gb)

        for comm in ("peer", "nccl"):
            os.environ["LEVANTER_B200_EP_COMM"] = comm
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                step()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 5], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res["times"][comm] = float(t)
        lib.check_status()
        torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_moe_block_on_peer_exchange_matches_unsharded(tmp_path):
    import json

    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, 29677, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"r{r}.pt")
        for comm, errs in res["errs"].items():
            assert max(errs) < 3e-2, (comm, errs)
        assert res["launches_peer"] > 0
    print("EP_MOE_BLOCK_FWD_BWD_MS", json.dumps(res["times"]))
