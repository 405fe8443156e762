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


def _helpers_worker(rank, world, port, out):
    import json

    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), CUDA_VISIBLE_DEVICES="")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    res = {}
    try:
        from levanter_b200.data.loader import check_sharded_consistency
        from levanter_b200.distributed import broadcast_one_to_all, is_local_leader, process_count, process_index
        from levanter_b200.parallel.mesh import DeviceMesh
        from levanter_b200.utils.torch_utils import multihost_broadcast_sync

        res["index"], res["count"], res["leader"] = process_index(), process_count(), is_local_leader()
        res["object"] = broadcast_one_to_all({"run": "abc"} if rank == 0 else None)
        res["synced"] = multihost_broadcast_sync(f"from {rank}")
        mesh = DeviceMesh(1, 1, 2)  # both ranks on the model axis: they must load identical batches
        check_sharded_consistency(torch.arange(8).reshape(2, 4), mesh)
        try:
            check_sharded_consistency(torch.arange(8).reshape(2, 4) + rank, mesh)
            res["mismatch"] = "not noticed"
        except RuntimeError as e:
            res["mismatch"] = str(e)
        data_mesh = DeviceMesh(1, 2, 1)  # a data axis only: ranks hold different rows, nothing to compare
        check_sharded_consistency(torch.arange(8).reshape(2, 4) + rank, data_mesh)
        json.dump(res, open(os.path.join(out, f"h{rank}.json"), "w"))
    finally:
        dist.destroy_process_group()


def test_process_helpers_and_the_identical_batch_check_on_two_ranks(tmp_path):
    import json

    mp.spawn(_helpers_worker, args=(2, 29743, str(tmp_path)), nprocs=2, join=True)
    r = [json.load(open(tmp_path / f"h{i}.json")) for i in range(2)]
    assert [x["index"] for x in r] == [0, 1] and [x["count"] for x in r] == [2, 2] and [x["leader"] for x in r] == [True, False]
    assert r[0]["object"] == r[1]["object"] == {"run": "abc"} and r[0]["synced"] == r[1]["synced"] == "from 0"
    assert all("differs between tensor-parallel ranks" in x["mismatch"] for x in r)
