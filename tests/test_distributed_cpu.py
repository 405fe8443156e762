"""Multi-process behaviour on CPU (gloo, two ranks): sharded training equals single-process training, the loader gives each
rank its slice, and failures surface as errors on the survivors rather than hangs: a peer that dies is noticed through its
heartbeat before the next step, and a collective with a short time-out ends with an error."""
import datetime
import json
import os
import sys
import time

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
VOCAB = 64


def _init(rank, world, port, timeout_s=60):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      CUDA_VISIBLE_DEVICES="")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))
    return dist


def _train(tmp, steps=3, batch=8, opt_dict=None, trainer_extra=None, hidden=32, expect_stage=None, return_average=False, lora=False):
    from levanter_b200 import config as C
    from levanter_b200.data.dataset import ListAsyncDataset
    from levanter_b200.models.llama import LlamaConfig
    from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
    from levanter_b200.optim import AdamConfig
    from levanter_b200.trainer import Trainer, TrainerConfig

    cfg = C.decode(TrainerConfig, {"num_train_steps": steps, "train_batch_size": batch, "require_accelerator": False, "tracker": {"type": "noop"},
                                   "log_dir": f"{tmp}/logs", "id": "t", "seed": 1, "checkpointer": {"base_path": f"{tmp}/ckpt", "save_interval": "10h"},
                                   **(trainer_extra or {})})
    g = torch.Generator().manual_seed(0)
    starts = torch.randint(0, VOCAB, (64,), generator=g)
    data = ListAsyncDataset([LmExample.causal(((s + torch.arange(16)) % VOCAB).to(torch.int32)) for s in starts], is_complete=True)
    mcfg = LlamaConfig(seq_len=16, hidden_dim=hidden, intermediate_dim=2 * hidden, num_layers=3 if hidden > 32 else 2, num_heads=2, num_kv_heads=2,
                       gradient_checkpointing=False)
    opt = AdamConfig(learning_rate=3e-3, warmup=0.0, weight_decay=0.0, lr_schedule="constant", min_lr_ratio=1.0)
    if opt_dict is not None:
        from levanter_b200.optim import OptimizerConfig

        opt = C.decode(OptimizerConfig, opt_dict)
    losses = {}
    with Trainer(cfg, opt, compute_next_token_loss) as trainer:
        from levanter_b200.parallel.tp import build_sharded_from_seed, gather_full_state

        tp = trainer.tensor_parallel
        if lora:  # adapters on the attention projections; only they train
            from levanter_b200.lora import LoraConfig, lora_trainable_params_filter, loraize

            model = loraize(mcfg.build(VOCAB, seed=3), LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj"]), seed=11)
            state = trainer.initial_state(0, model=model, is_trainable=lora_trainable_params_filter(model))
        else:
            state = trainer.initial_state(0, model_init=lambda: build_sharded_from_seed(lambda tp: mcfg.build(VOCAB, seed=3, tp=tp), tp))
        trainer.add_hook(lambda info: losses.__setitem__(info.step, float(info.loss)), every=1)
        if expect_stage is not None:
            assert state.engine.zero_stage == expect_stage, state.engine.zero_stage
        info = trainer.train(state, trainer.data_loader(data).iter_from_step(int(state.step)))
        if return_average:  # the averaged weights, whole on every rank
            return {k: v.detach().clone() for k, v in info.state.eval_model.named_parameters()}, [losses[k] for k in sorted(losses)]
        if expect_stage == 3:
            st = state.engine.stream
            assert st is not None and st.stats["library_weight_grads"] > 0
            full = state.engine.full_master()  # whole matrices again, assembled from every rank's rows
            return {k: full[k].detach().clone() for k, _ in info.state.model.named_parameters()}, [losses[k] for k in sorted(losses)]
        if tp is not None and state.engine.zero_stage == 3:
            # the module's parameters are views of staging slots here: take the master rows of every data rank, then join the
            # model-axis slices
            import torch.distributed as dist

            full = state.engine.full_master()
            out = {}
            for name, p in info.state.model.named_parameters():
                t, dim = full[name].detach().clone(), getattr(p, "tp_dim", None)
                if dim is not None:
                    parts = [torch.empty_like(t) for _ in range(tp.size)]
                    dist.all_gather(parts, t.contiguous(), group=tp.group)
                    t = torch.cat(parts, dim=dim)
                out[name] = t
            return out, [losses[k] for k in sorted(losses)]
        if tp is not None:
            return gather_full_state(info.state.model, tp), [losses[k] for k in sorted(losses)]
    return {k: v.detach().clone() for k, v in info.state.model.named_parameters()}, [losses[k] for k in sorted(losses)]


def _sharded_worker(rank, world, port, tmp, opt_dict=None, trainer_extra=None, hidden=32, expect_stage=None, steps=3, lora=False):
    dist = _init(rank, world, port)
    try:
        params, losses = _train(tmp, steps=steps, opt_dict=opt_dict, trainer_extra=trainer_extra, hidden=hidden, expect_stage=expect_stage, lora=lora)
        if rank == 0:
            torch.save({"params": params, "losses": losses}, f"{tmp}/dist.pt")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_training_matches_single_process(tmp_path):
    single, losses = _train(str(tmp_path / "single"))
    mp.spawn(_sharded_worker, args=(2, 29711, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=2e-5)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=2e-5), k


def test_two_rank_zero3_layer_streaming_matches_single_process(tmp_path):
    """zero_stage 3 on two ranks (library transport on gloo): layer matrices live as row slices, are gathered per layer and
    their gradients reduce-scattered as autograd produces them; losses and final weights equal one process."""
    single, losses = _train(str(tmp_path / "single"), hidden=64)
    mp.spawn(_sharded_worker, args=(2, 29723, str(tmp_path), None, {"zero_stage": 3, "per_device_parallelism": 2}, 64, 3), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=2e-5)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=2e-5), k


def test_zero3_under_two_replicas_matches_single_process(tmp_path):
    """Four ranks: replica 2 x data 2.  Layer matrices are row-sliced over the data axis inside each replica, and the gradient
    rows a rank owns are averaged over the replicas before its optimizer step."""
    single, losses = _train(str(tmp_path / "single"), hidden=64)
    mp.spawn(_sharded_worker, args=(4, 29727, str(tmp_path), None, {"zero_stage": 3, "replica_ici_axis_size": 2}, 64, 3), nprocs=4, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=2e-5)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=2e-5), k


def test_two_way_tensor_parallel_training_matches_single_process(tmp_path):
    """model axis 2 (heads and MLP columns split, all-reduce after the row-parallel projections and of the input gradients of
    the column-parallel ones): three optimizer steps give the losses and the weights of the unsharded run."""
    # (a larger Adam epsilon than usual: with 1e-8 the elements whose gradient is rounding noise take full-size steps of random
    # sign, and the split reductions of tensor parallelism change that noise)
    opt = {"type": "adam", "learning_rate": 3e-3, "warmup": 0.0, "weight_decay": 0.0, "lr_schedule": "constant", "min_lr_ratio": 1.0,
           "epsilon": 1e-4, "max_grad_norm": 0.5}
    single, losses = _train(str(tmp_path / "single"), opt_dict=opt)
    mp.spawn(_sharded_worker, args=(2, 29724, str(tmp_path), opt, {"model_axis_size": 2, "tensor_parallel_axes": ["mlp", "heads"]}), nprocs=2,
             join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=2e-5)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=2e-5), k


def test_tensor_parallel_with_zero3_over_the_data_axis_matches_single_process(tmp_path):
    """Four ranks: data 2 x model 2.  Heads and MLP columns are split over the model axis; each model rank's slices are
    row-sliced again over the data axis (zero stage 3), gathered per layer and their gradients reduce-scattered."""
    opt = {"type": "adam", "learning_rate": 3e-3, "warmup": 0.0, "weight_decay": 0.0, "lr_schedule": "constant", "min_lr_ratio": 1.0,
           "epsilon": 1e-4, "max_grad_norm": 0.5}
    single, losses = _train(str(tmp_path / "single"), opt_dict=opt, hidden=128)
    extra = {"model_axis_size": 2, "tensor_parallel_axes": ["mlp", "heads"], "zero_stage": 3}
    mp.spawn(_sharded_worker, args=(4, 29728, str(tmp_path), opt, extra, 128), nprocs=4, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=3e-5)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=3e-5), k


MUON = {"type": "muon", "learning_rate": 2e-2, "adam_lr": 3e-3, "warmup": 0.0, "lr_schedule": "constant", "min_lr_ratio": 1.0}


def test_two_rank_muon_shares_newton_schulz_and_matches_single_process(tmp_path):
    """Muon on two data ranks: every matrix is orthogonalised by one rank and broadcast; the trajectory equals one process."""
    single, losses = _train(str(tmp_path / "single"), opt_dict=MUON)
    mp.spawn(_sharded_worker, args=(2, 29721, str(tmp_path), MUON), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=5e-5)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=5e-5), k


def test_two_replicas_take_the_same_step_as_one_process(tmp_path):
    """replica axis 2 x data axis 1 (pure data parallelism): gradients are averaged over the replicas."""
    single, losses = _train(str(tmp_path / "single"))
    mp.spawn(_sharded_worker, args=(2, 29722, str(tmp_path), None, {"replica_ici_axis_size": 2}), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=2e-5)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=2e-5), k


def _first_half_worker(rank, world, port, tmp, hidden=32, trainer_extra=None, opt_dict=None):
    dist = _init(rank, world, port)
    try:
        _train(tmp, steps=3, hidden=hidden, trainer_extra=trainer_extra, opt_dict=opt_dict)
    finally:
        dist.destroy_process_group()


def test_zero3_checkpoint_written_by_two_ranks_resumes_on_one(tmp_path):
    """The same with streamed layers: the row slices of weights and moments are gathered into whole tensors on save."""
    full, losses = _train(str(tmp_path / "full"), steps=6, hidden=64)
    mp.spawn(_first_half_worker, args=(2, 29716, str(tmp_path / "res"), 64, {"zero_stage": 3}), nprocs=2, join=True)
    resumed, tail = _train(str(tmp_path / "res"), steps=6, hidden=64)
    assert len(tail) == 3 and tail == pytest.approx(losses[3:], abs=3e-5)
    for k, v in full.items():
        assert torch.allclose(v, resumed[k], atol=3e-5), k


def test_checkpoint_written_by_two_ranks_resumes_on_one(tmp_path):
    """Resume on a different process count: the sharded optimizer state is gathered on save and re-sliced on load."""
    full, losses = _train(str(tmp_path / "full"), steps=6)
    mp.spawn(_first_half_worker, args=(2, 29715, str(tmp_path / "res")), nprocs=2, join=True)
    resumed, tail = _train(str(tmp_path / "res"), steps=6)
    assert len(tail) == 3 and tail == pytest.approx(losses[3:], abs=3e-5)
    for k, v in full.items():
        assert torch.allclose(v, resumed[k], atol=3e-5), k


def _second_half_average_worker(rank, world, port, tmp, extra):
    dist = _init(rank, world, port)
    try:
        avg, tail = _train(tmp, steps=6, trainer_extra=extra, return_average=True)
        if rank == 0:
            torch.save({"avg": avg, "tail": tail}, f"{tmp}/avg.pt")
    finally:
        dist.destroy_process_group()


def test_averaged_weights_written_by_two_ranks_resume_on_one_and_on_two(tmp_path):
    extra = {"model_averaging": {"type": "ema", "beta": 0.5}}
    full, losses = _train(str(tmp_path / "full"), steps=6, trainer_extra=extra, return_average=True)
    for name in ("one", "two"):
        mp.spawn(_first_half_worker, args=(2, 29717, str(tmp_path / name), 32, extra), nprocs=2, join=True)
    resumed, tail = _train(str(tmp_path / "one"), steps=6, trainer_extra=extra, return_average=True)
    assert len(tail) == 3 and tail == pytest.approx(losses[3:], abs=3e-5)
    for k, v in full.items():
        assert torch.allclose(v, resumed[k], atol=3e-5), k
    mp.spawn(_second_half_average_worker, args=(2, 29718, str(tmp_path / "two"), extra), nprocs=2, join=True)
    got = torch.load(tmp_path / "two" / "avg.pt")
    assert len(got["tail"]) == 3 and got["tail"] == pytest.approx(losses[3:], abs=3e-5)
    for k, v in full.items():
        assert torch.allclose(v, got["avg"][k], atol=3e-5), k


def _loader_worker(rank, world, port, tmp):
    dist = _init(rank, world, port)
    try:
        from levanter_b200.data.dataset import ListAsyncDataset
        from levanter_b200.data.loader import DataLoader
        from levanter_b200.parallel.mesh import DeviceMesh

        mesh = DeviceMesh.create(replica=1, data=world, model=1) if hasattr(DeviceMesh, "create") else DeviceMesh(1, world, 1)
        ds = ListAsyncDataset([torch.tensor([i]) for i in range(40)], is_complete=True)
        dl = DataLoader(ds, 8, mesh=mesh, max_buffered_batches=0, pin_memory=False)
        it = dl.iter_from_step(2)
        rows = [next(it).reshape(-1).tolist() for _ in range(2)]
        json.dump(rows, open(f"{tmp}/rows{rank}.json", "w"))
    finally:
        dist.destroy_process_group()


def test_loader_gives_each_rank_its_slice_and_resumes_by_step(tmp_path):
    mp.spawn(_loader_worker, args=(2, 29712, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (json.load(open(tmp_path / f"rows{r}.json")) for r in range(2))
    # global batch 2 is rows 16..23, batch 3 is 24..31; rank 0 takes the first half of each
    assert r0 == [[16, 17, 18, 19], [24, 25, 26, 27]] and r1 == [[20, 21, 22, 23], [28, 29, 30, 31]]


def _dying_peer_worker(rank, world, port, tmp):
    dist = _init(rank, world, port, timeout_s=5)
    from levanter_b200.utils.watchdog import PeerFailure, Watchdog

    out = {}
    try:
        wd = Watchdog(f"{tmp}/hb", rank, world, interval=0.1, peer_timeout=1.0).start()
        t = torch.ones(1)
        dist.all_reduce(t)  # step 0: both ranks are here
        wd.beat(0)
        if rank == 1:
            wd.stop()       # rank 1 leaves between steps, with nothing in flight
            os._exit(0)
        t0 = time.time()
        try:
            while True:     # rank 0 checks the heartbeats before each further "launch"
                wd.raise_if_failed()
                time.sleep(0.05)
                if time.time() - t0 > 20:
                    out["outcome"] = "never noticed"
                    break
        except PeerFailure as e:
            out["outcome"], out["after"], out["message"] = "peer failure", time.time() - t0, str(e)
        # and a collective that is issued anyway ends with an error after the group's short time-out instead of hanging
        t1 = time.time()
        try:
            dist.all_reduce(torch.ones(1))
            out["collective"] = "returned"
        except Exception as e:  # noqa: BLE001
            out["collective"], out["collective_after"] = type(e).__name__, time.time() - t1
        wd.stop()
    finally:
        if rank == 0:
            json.dump(out, open(f"{tmp}/out.json", "w"))
            os._exit(0)  # the group cannot be destroyed cleanly with a dead peer


def test_dead_peer_is_noticed_before_the_next_step_and_collectives_time_out(tmp_path):
    ctx = mp.spawn(_dying_peer_worker, args=(2, 29713, str(tmp_path)), nprocs=2, join=False)
    deadline = time.time() + 90
    while not os.path.exists(tmp_path / "out.json") and time.time() < deadline:
        time.sleep(0.2)
    time.sleep(0.3)
    for p in ctx.processes:
        p.join(timeout=5)
        if p.is_alive():
            p.terminate()
    out = json.load(open(tmp_path / "out.json"))
    assert out["outcome"] == "peer failure" and out["after"] < 10 and "rank 1" in out["message"]
    assert out["collective"] != "returned" and out["collective_after"] < 30


def _raising_rank_worker(rank, world, port, tmp):
    dist = _init(rank, world, port, timeout_s=5)
    from levanter_b200.utils.watchdog import PeerFailure, Watchdog

    try:
        with Watchdog(f"{tmp}/hb", rank, world, interval=0.1, peer_timeout=30.0) as wd:
            dist.barrier()
            if rank == 1:
                raise ValueError("loss is NaN")  # the context manager writes the failure marker on the way out
            t0 = time.time()
            while time.time() - t0 < 20:
                wd.raise_if_failed()
                time.sleep(0.05)
    except PeerFailure as e:
        json.dump({"message": str(e), "after": time.time() - t0}, open(f"{tmp}/out.json", "w"))
    except ValueError:
        pass
    finally:
        os._exit(0)


def test_failure_marker_carries_the_reason_to_the_peers(tmp_path):
    ctx = mp.spawn(_raising_rank_worker, args=(2, 29714, str(tmp_path)), nprocs=2, join=False)
    deadline = time.time() + 60
    while not os.path.exists(tmp_path / "out.json") and time.time() < deadline:
        time.sleep(0.2)
    time.sleep(0.3)
    for p in ctx.processes:
        p.join(timeout=5)
    out = json.load(open(tmp_path / "out.json"))
    assert "rank 1 failed" in out["message"] and "loss is NaN" in out["message"] and out["after"] < 5


@pytest.mark.parametrize("index,opt", list(enumerate(["lion", "soap", "kron", "mini", "adopt", "cautious", "mars", "rmsprop", "scion", "sophia-h"])))
def test_every_other_optimizer_on_two_data_ranks_matches_single_process(tmp_path, index, opt):
    """Whatever the optimizer keeps (moments on slices, whole-matrix preconditioners, per-group scalars, Hessian estimates), two
    data ranks take the steps one process takes."""
    extra = {"update_interval": 2} if opt == "sophia-h" else {"precondition_frequency": 2} if opt == "soap" else {}
    od = {"type": opt, "learning_rate": 3e-3, "warmup": 0.0, "weight_decay": 0.0, "lr_schedule": "constant", "min_lr_ratio": 1.0, **extra}
    single, losses = _train(str(tmp_path / "single"), opt_dict=od)
    mp.spawn(_sharded_worker, args=(2, 29750 + index, str(tmp_path), od), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=1e-4)
    for k, v in single.items():
        if opt == "adopt":
            # the second step divides by |first gradient| with no clipping: where that is almost zero, the last bit of the gradient
            # (summed in another order on two ranks) decides the size of the step, so a few elements move apart
            assert float(((v - got["params"][k]).abs() > 1e-4).float().mean()) < 0.01, k
        else:
            assert torch.allclose(v, got["params"][k], atol=1e-4), k


def test_skip_step_reaches_the_same_verdicts_on_two_ranks_as_on_one(tmp_path):
    """The skip-step wrapper judges a step by the loss of the whole batch: with a zero-sigma window (a step is dropped as soon
    as its loss or gradient norm is above the window's mean) two data ranks drop the same steps as one process."""
    od = {"type": "adam", "learning_rate": 3e-3, "warmup": 0.0, "weight_decay": 0.0, "lr_schedule": "constant", "min_lr_ratio": 1.0,
          "skip_bad_steps": {"rolling_interval_length": 4, "sigma_factor": 0.0}}
    single, losses = _train(str(tmp_path / "single"), steps=8, opt_dict=od)
    mp.spawn(_sharded_worker, args=(2, 29761, str(tmp_path), od, None, 32, None, 8), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=1e-4)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=1e-4), k


def _tagged_eval(tmp, trainer_extra=None, hidden=32):
    from levanter_b200 import config as C
    from levanter_b200.data.dataset import ListAsyncDataset
    from levanter_b200.eval import TaggedEvaluator
    from levanter_b200.models.llama import LlamaConfig
    from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
    from levanter_b200.optim import AdamConfig
    from levanter_b200.trainer import Trainer, TrainerConfig

    cfg = C.decode(TrainerConfig, {"num_train_steps": 1, "train_batch_size": 8, "require_accelerator": False, "tracker": {"type": "noop"},
                                   "log_dir": f"{tmp}/logs", "id": "e", "seed": 1, "checkpointer": {"base_path": f"{tmp}/ckpt", "save_interval": "10h"},
                                   **(trainer_extra or {})})
    g = torch.Generator().manual_seed(5)

    def examples(n):
        return ListAsyncDataset([LmExample.causal(torch.randint(0, VOCAB, (16,), generator=g, dtype=torch.int32)) for _ in range(n)], is_complete=True)

    sets = [(examples(7), ["web/a"]), (examples(6), ["web/b"]), (examples(1), ["code"])]  # 14 examples: the last batch of 4 is ragged
    mcfg = LlamaConfig(seq_len=16, hidden_dim=hidden, intermediate_dim=2 * hidden, num_layers=3 if hidden > 32 else 2, num_heads=2, num_kv_heads=2,
                       gradient_checkpointing=False)
    with Trainer(cfg, AdamConfig(), compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=lambda: mcfg.build(VOCAB, seed=3))
        ev = TaggedEvaluator(4, sets, device_mesh=trainer.device_mesh if cfg.num_devices > 1 else None)
        r = ev.evaluate(state.model)
    return {"micro": r.micro_avg_loss, "macro": r.macro_avg_loss, **{f"tag/{k}": v for k, v in r.tag_micro_losses.items()},
            **{f"macro/{k}": v for k, v in r.tag_macro_losses.items()}}


def _tagged_eval_worker(rank, world, port, tmp, trainer_extra, hidden):
    dist = _init(rank, world, port)
    try:
        torch.save(_tagged_eval(tmp, trainer_extra, hidden), f"{tmp}/eval{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("port,extra,hidden", [(29771, None, 32), (29772, {"zero_stage": 3}, 64)])
def test_tagged_evaluation_on_two_ranks_equals_one_process(tmp_path, port, extra, hidden):
    """Every rank scores its part of each evaluation batch (the last one is ragged) and the sums are reduced: overall, per-tag and
    parent-tag losses equal one process, on every rank, also when the layers are gathered from row slices during the forward pass."""
    single = _tagged_eval(str(tmp_path / "single"), None, hidden)
    assert {"tag/web/a", "tag/web/b", "tag/code", "tag/web", "macro/web"} <= set(single)
    mp.spawn(_tagged_eval_worker, args=(2, port, str(tmp_path), extra, hidden), nprocs=2, join=True)
    for rank in range(2):
        got = torch.load(tmp_path / f"eval{rank}.pt")
        assert set(got) == set(single)
        for k, v in single.items():
            assert got[k] == pytest.approx(v, rel=1e-5), (rank, k)


def test_lora_training_on_two_ranks_matches_single_process(tmp_path):
    """Only the adapters train: the frozen base weights stay bit-identical, the adapters take the same steps on two data ranks as
    on one process."""
    single, losses = _train(str(tmp_path / "single"), steps=4, lora=True)
    mp.spawn(_sharded_worker, args=(2, 29781, str(tmp_path), None, None, 32, None, 4, True), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=2e-5) and losses[-1] < losses[0]
    assert any("lora" in k.lower() for k in single)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=2e-5), k


def test_batch_size_schedule_with_accumulation_on_two_ranks_matches_single_process(tmp_path):
    """The batch grows from 4 to 8 sequences at step 2 and every rank takes two sequences per micro-batch: one process accumulates
    2 then 4 micro-batches, two ranks 1 then 2 each, and both take the same steps."""
    extra = {"train_batch_size": [{"start": 0, "value": 4}, {"start": 2, "value": 8}], "per_device_parallelism": 2}
    single, losses = _train(str(tmp_path / "single"), steps=5, trainer_extra=extra)
    mp.spawn(_sharded_worker, args=(2, 29783, str(tmp_path), None, extra, 32, None, 5), nprocs=2, join=True)
    got = torch.load(tmp_path / "dist.pt")
    assert got["losses"] == pytest.approx(losses, abs=2e-5)
    for k, v in single.items():
        assert torch.allclose(v, got["params"][k], atol=2e-5), k


@pytest.mark.parametrize("index,opt", list(enumerate(["muon", "soap", "sophia-h", "lion"])))
def test_other_optimizers_written_by_two_ranks_resume_on_one(tmp_path, index, opt):
    """Optimizers whose state is kept whole on every rank (matrix preconditioners, the Hessian estimate) and a sliced one: the
    checkpoint two ranks wrote continues on one process as the uninterrupted run does."""
    extra = {"update_interval": 2} if opt == "sophia-h" else {"precondition_frequency": 2} if opt == "soap" else {}
    od = {"type": opt, "learning_rate": 3e-3, "warmup": 0.0, "weight_decay": 0.0, "lr_schedule": "constant", "min_lr_ratio": 1.0, **extra}
    full, losses = _train(str(tmp_path / "full"), steps=6, opt_dict=od)
    mp.spawn(_first_half_worker, args=(2, 29785 + index, str(tmp_path / "res"), 32, None, od), nprocs=2, join=True)
    resumed, tail = _train(str(tmp_path / "res"), steps=6, opt_dict=od)
    assert len(tail) == 3 and tail == pytest.approx(losses[3:], abs=1e-4)
    for k, v in full.items():
        assert torch.allclose(v, resumed[k], atol=1e-4), k
