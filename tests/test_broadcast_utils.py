"""Host-side plumbing: a tree that exists on one process reaches all (whole or sliced over the batch axis), the named barrier,
and the optional Ray bootstrap when Ray is absent."""
import datetime
import os
import sys

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), CUDA_VISIBLE_DEVICES="")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        from levanter_b200.distributed import sync_global_devices
        from levanter_b200.utils.torch_utils import broadcast_shard

        tree = None
        if rank == 0:
            tree = {"tokens": torch.arange(24).reshape(4, 6), "aux": (torch.ones(3) * 2.5, [torch.tensor([7], dtype=torch.int16)]), "n": 3}
        whole = broadcast_shard(tree, source=0)
        part = broadcast_shard(tree, source=0, shard_dim=0)
        sync_global_devices("test")
        torch.save({"whole": whole, "part": part}, os.path.join(out, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_broadcast_shard_whole_and_sliced(tmp_path):
    mp.spawn(_worker, args=(2, 29741, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        got = torch.load(tmp_path / f"r{r}.pt")
        w = got["whole"]
        assert torch.equal(w["tokens"], torch.arange(24).reshape(4, 6)) and w["n"] == 3
        assert torch.equal(w["aux"][0], torch.ones(3) * 2.5) and w["aux"][1][0].dtype == torch.int16
        assert torch.equal(got["part"]["tokens"], torch.arange(24).reshape(4, 6)[2 * r:2 * r + 2])
        assert got["part"]["aux"][0].shape == (3,)  # 3 rows do not divide over 2 ranks: kept whole


def test_single_process_paths():
    from levanter_b200.distributed import auto_ray_cluster, sync_global_devices
    from levanter_b200.utils.cloud_utils import sync_global_devices as same
    from levanter_b200.utils.torch_utils import broadcast_shard

    t = {"x": torch.ones(2)}
    assert broadcast_shard(t) is t
    sync_global_devices("nothing to wait for")
    assert same is sync_global_devices
    try:
        import ray  # noqa: F401
    except ImportError:
        assert auto_ray_cluster() is False  # nothing here needs Ray: absent means "not started", not an error
