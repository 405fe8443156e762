"""Fully sharded layers (zero stage 3) on two GPUs: the copy job that assembles a layer (on its own and riding on a GEMM),
the weight-gradient GEMM with the reduce-scatter in its epilogue (rows per rank a multiple of 128 and not), and whole
optimizer steps through the engine on the peer transport against the library transport and against stage 1."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    return dist


class _Stack(torch.nn.Module):
    def __init__(self, shapes, n_layers, device):
        super().__init__()
        from levanter_b200.nn import Linear

        self.layers = torch.nn.ModuleList()
        for _ in range(n_layers):
            blk = torch.nn.Module()
            for i, (n, k) in enumerate(shapes):
                setattr(blk, f"w{i}", Linear(k, n, device=device, dtype=torch.bfloat16))
            self.layers.append(blk)
        self.head = Linear(64, 64, device=device, dtype=torch.bfloat16)


def _kernel_worker(rank, world, port, out_dir):
    dist = _setup(rank, world, port)
    try:
        from levanter_b200.config import Policy
        from levanter_b200.ops import lib
        from levanter_b200.ops.gemm import gemm
        from levanter_b200.parallel.engine import ShardedEngine
        from levanter_b200.parallel.mesh import DeviceMesh

        dev = torch.device("cuda", rank)
        torch.manual_seed(0)  # the same initial weights on every rank
        shapes = [(1024, 512), (320, 256), (512, 1024)]  # 320 rows: 160 per rank, a 128-row block straddles the two owners
        model = _Stack(shapes, 3, dev)
        full0 = {n: p.detach().clone() for n, p in model.named_parameters()}
        eng = ShardedEngine(model, Policy.parse("p=f32,c=bfloat16"), DeviceMesh(replica=1, data=world, model=1), device=dev, comm="p2p",
                            zero_stage=3)
        st = eng.stream
        assert eng.zero_stage == 3 and st is not None and st.peer and len(st.params) == 9
        res = {}
        # ---- stand-alone copy job: layer 1 assembled in slot 1
        st.gather_now(1)
        torch.cuda.synchronize()
        res["gather_standalone"] = all(torch.equal(sp.param.data, full0[sp.name]) for sp in st.by_layer[1])
        # ---- copy job riding on GEMMs: layer 2 into slot 0 while unrelated products run
        st.prefetch(2)
        a = torch.randn(2048, 1024, device=dev).bfloat16()
        b = torch.randn(1024, 1024, device=dev).bfloat16()
        c = gemm(a, b)  # carries the first share of the job
        for _ in range(3):
            gemm(a, b)
        st.ensure(2)
        torch.cuda.synchronize()
        lib.check_status()
        res["gather_on_gemm"] = all(torch.equal(sp.param.data, full0[sp.name]) for sp in st.by_layer[2])
        res["units_on_gemms"] = st.stats["units_on_gemms"]
        from levanter_b200.ops import gemm as G

        G.SPLITK_MODE = "general"  # the product that carried the job ran whole-K tiles: compare with the same tiling, bit for bit
        res["gemm_with_job_ok"] = bool(torch.equal(c, gemm(a, b)))
        G.SPLITK_MODE = "splitk"
        # ---- weight gradients: dy^T x summed over the ranks, this rank's rows, accumulated over two calls
        g = torch.Generator(device=dev).manual_seed(10 + rank)
        errs = []
        for sp in st.by_layer[0]:
            N, K = sp.shape
            want = torch.zeros(N, K, dtype=torch.float32, device=dev)
            for _ in range(2):
                dy = torch.randn(768, N, device=dev, generator=g).bfloat16()
                x = torch.randn(768, K, device=dev, generator=g).bfloat16()
                sp.param.grad_sink(dy, x)
                part = dy.float().t() @ x.float()
                dist.all_reduce(part)
                want += part / world
            torch.cuda.synchronize()
            lib.check_status()
            got = st._grad_rows(sp)
            ref = want[rank * sp.rows:(rank + 1) * sp.rows]
            errs.append(((got - ref).abs().max() / ref.abs().max()).item())
        res["dw_errs"] = errs
        res["fused_weight_grads"] = st.stats["fused_weight_grads"]
        torch.save(res, os.path.join(out_dir, f"k{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_copy_job_and_fused_weight_gradient(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_kernel_worker, args=(2, 29641, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"k{r}.pt")
        assert res["gather_standalone"] and res["gather_on_gemm"] and res["gemm_with_job_ok"], res
        assert res["units_on_gemms"] > 0 and res["fused_weight_grads"] == 6, res
        assert max(res["dw_errs"]) < 1e-3, res  # fp32 partial products, fp32 sums: only the order of additions differs


def _engine_worker(rank, world, port, out_dir):
    dist = _setup(rank, world, port)
    try:
        from levanter_b200.config import Policy
        from levanter_b200.models.llama import LlamaConfig
        from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
        from levanter_b200.ops import lib
        from levanter_b200.optim import AdamConfig, ParamInfo
        from levanter_b200.parallel.engine import ShardedEngine
        from levanter_b200.parallel.mesh import DeviceMesh

        dev = torch.device("cuda", rank)
        mesh = DeviceMesh(replica=1, data=world, model=1)
        cfg = LlamaConfig(seq_len=256, hidden_dim=256, intermediate_dim=512, num_layers=4, num_heads=2, num_kv_heads=2, gradient_checkpointing=False)
        results = {}
        for tag, comm, stage in (("stage1", "nccl", 1), ("stage3_nccl", "nccl", 3), ("stage3_peer", "p2p", 3)):
            model = cfg.build(512, seed=0, device=dev)
            eng = ShardedEngine(model, Policy.parse("p=f32,c=bfloat16"), mesh, device=dev, comm=comm, zero_stage=stage)
            assert eng.zero_stage == stage
            ocfg = AdamConfig(learning_rate=1e-2, warmup=0.0, weight_decay=0.1, max_grad_norm=1.0)
            eng.set_optimizer(ocfg.build(10, ParamInfo(model)), optimizer_config=ocfg, num_train_steps=10)
            g = torch.Generator().manual_seed(100 + rank)
            losses, norms, first = [], [], None
            for step in range(3):
                for micro in range(2):  # two micro-batches per step: the streamed gradients accumulate across them
                    tokens = torch.randint(0, 512, (2, 256), generator=g, dtype=torch.int32).cuda()
                    loss = compute_next_token_loss(model, LmExample.causal(tokens)) / 2
                    loss.backward()
                    losses.append(float(loss.detach()))
                eng.step(loss=loss)
                norms.append(float(eng.last_grad_norm))
                if step == 0:
                    first = {k: v.float().cpu() for k, v in eng.full_master().items()}
            torch.cuda.synchronize()
            lib.check_status()
            full = eng.full_master()
            results[tag] = ({k: v.float().cpu() for k, v in full.items()}, norms, losses,
                            dict(eng.stream.stats) if eng.stream is not None else None, first)
            from levanter_b200.ops.gemm import set_copy_job_provider

            set_copy_job_provider(None)
            del eng, model
        torch.save(results, os.path.join(out_dir, f"e{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_zero3_steps_match_stage1_steps(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_engine_worker, args=(2, 29643, str(tmp_path)), nprocs=2, join=True)
    res = [torch.load(tmp_path / f"e{r}.pt") for r in range(2)]
    for r in range(2):
        w1, n1, l1, _, f1 = res[r]["stage1"]
        for tag in ("stage3_nccl", "stage3_peer"):
            w3, n3, l3, stats, f3 = res[r][tag]
            # the first step sees the same weights: gradients agree to fp32 rounding (only the order of the sums differs), and so
            # do the updated weights, up to elements whose gradient is rounding noise
            assert abs(n1[0] - n3[0]) <= 1e-5 * abs(n1[0]), (tag, n1, n3)
            assert l1[:2] == l3[:2], tag
            for k in f1:
                assert (f1[k] - f3[k]).abs().max() < 2e-4, (tag, k, (f1[k] - f3[k]).abs().max())
            # later steps: Adam at this learning rate amplifies those elements, so compare the bulk and the trajectory
            assert all(abs(a - b) <= 2e-3 * abs(a) for a, b in zip(n1, n3)), (tag, n1, n3)
            assert all(abs(a - b) < 1e-3 for a, b in zip(l1, l3)), (tag, l1, l3)
            for k in w1:
                assert ((w1[k] - w3[k]).abs() > 2e-3).float().mean().item() < 2e-2, (tag, k)
        # the two transports of stage 3 do the same arithmetic up to the order of fp32 additions
        wa, na, la, _, fa = res[r]["stage3_nccl"]
        wb, nb, lb, stats, fb = res[r]["stage3_peer"]
        assert la[:2] == lb[:2] and all(abs(a - b) < 1e-4 for a, b in zip(la, lb)), (la, lb)
        assert all(abs(a - b) <= 1e-4 * abs(a) for a, b in zip(na, nb)), (na, nb)
        for k in fa:
            assert ((fa[k] - fb[k]).abs() > 1e-4).float().mean().item() < 1e-3, k
        assert stats["fused_weight_grads"] == 3 * 2 * 4 * 7 and stats["library_weight_grads"] == 0, stats
        assert stats["units_on_gemms"] > 0, stats
    for k in res[0]["stage3_peer"][0]:
        assert torch.equal(res[0]["stage3_peer"][0][k], res[1]["stage3_peer"][0][k]), k
