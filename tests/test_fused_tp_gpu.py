"""Fused all-gather -> GEMM and GEMM -> reduce-scatter on two GPUs against NCCL collectives + plain matmuls, with timings."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from levanter_b200.ops import lib
    from levanter_b200.ops.fused_tp import all_gather_matmul, matmul_reduce_scatter, reduce_scatter_staging_elems
    from levanter_b200.ops.gemm import gemm
    from levanter_b200.parallel.symm import SymmetricBuffer

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        g = torch.Generator(device=dev).manual_seed(rank)
        rows, K, N = 4096, 4096, 4096
        # ---- all-gather -> GEMM
        xs = SymmetricBuffer(rows * K, torch.bfloat16, dev, None)
        xs.tensor.copy_(torch.randn(rows * K, device=dev, generator=g).bfloat16())
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
        y = all_gather_matmul(xs, rows, K, w)
        full = torch.empty(world * rows, K, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(full, xs.tensor.view(rows, K))
        y_ref = gemm(full, w)
        torch.cuda.synchronize()
        lib.check_status()
        err1 = (y.float() - y_ref.float()).abs().max().item() / y_ref.float().abs().max().item()
        # ---- GEMM -> reduce-scatter
        M = world * rows
        x2 = torch.randn(M, K // world, device=dev, generator=g).bfloat16()
        w2 = (torch.randn(N, K // world, device=dev, generator=g) * 0.02).bfloat16()
        staging = SymmetricBuffer(reduce_scatter_staging_elems(M, N), torch.float32, dev, None)
        z = matmul_reduce_scatter(x2, w2, staging)
        part = gemm(x2, w2, out_dtype=torch.float32)
        z_ref = torch.empty(rows, N, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(z_ref, part)
        torch.cuda.synchronize()
        lib.check_status()
        err2 = (z.float() - z_ref).abs().max().item() / z_ref.abs().max().item()
        staging_bf = SymmetricBuffer(reduce_scatter_staging_elems(M, N, torch.bfloat16), torch.bfloat16, dev, None)
        z2 = matmul_reduce_scatter(x2, w2, staging_bf)
        staging_bf2 = SymmetricBuffer(reduce_scatter_staging_elems(M, N, torch.bfloat16), torch.bfloat16, dev, None)
        torch.cuda.synchronize()
        lib.check_status()
        err3 = (z2.float() - z_ref).abs().max().item() / z_ref.abs().max().item()

        def timeit(fn, n=10):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)

        def nccl_ag():
            dist.all_gather_into_tensor(full, xs.tensor.view(rows, K))
            gemm(full, w)

        def nccl_rs():
            p = gemm(x2, w2, out_dtype=torch.float32)
            dist.reduce_scatter_tensor(z_ref, p)

        z_bf = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)

        def nccl_rs_bf16():
            p = gemm(x2, w2)
            dist.reduce_scatter_tensor(z_bf, p)

        times = {"fused_ag_gemm_ms": timeit(lambda: all_gather_matmul(xs, rows, K, w)), "nccl_ag_gemm_ms": timeit(nccl_ag),
                 "fused_gemm_rs_ms": timeit(lambda: matmul_reduce_scatter(x2, w2, staging)),
                 "fused_gemm_rs_bf16_ms": timeit(lambda: matmul_reduce_scatter(x2, w2, staging_bf)),
                 "fused_gemm_rs_bf16_local_only_ms": timeit(lambda: matmul_reduce_scatter(x2, w2, staging_bf2, _local_only=True)), "nccl_gemm_rs_ms": timeit(nccl_rs), "nccl_gemm_rs_bf16_ms": timeit(nccl_rs_bf16),
                 "gemm_only_ms": timeit(lambda: gemm(full, w)), "gemm_partial_only_ms": timeit(lambda: gemm(x2, w2))}
        lib.check_status()
        torch.save({"err1": err1, "err2": err2, "err3": err3, "times": times, "shape": (M, N, K)}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_tp_gemms_match_nccl(tmp_path):
    import json

    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 2)
    mp.spawn(_worker, args=(world, 29651, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        assert res["err1"] < 2e-2, res
        assert res["err2"] < 2e-2, res
        assert res["err3"] < 3e-2, res
    print("FUSED_TP_TIMES", json.dumps(res["times"]), res["shape"])
