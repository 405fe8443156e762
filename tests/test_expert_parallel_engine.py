"""Expert-parallel Mixtral through the trainer and the sharded engine on two gloo ranks: the experts are sliced over the ranks
(rank-local buckets: scaled, not reduced; not gathered), everything else is sharded as usual.  Training must match the
single-process model with all experts, and a checkpoint written by the two ranks must resume on one process that holds
every expert."""
import dataclasses
import datetime
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
VOCAB = 64


def _init(rank, world, port):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      CUDA_VISIBLE_DEVICES="")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    return dist


def _train(tmp, steps, rank=0, world=1, batch=8):
    from levanter_b200 import config as C
    from levanter_b200.data.dataset import ListAsyncDataset
    from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
    from levanter_b200.models.mixtral import MixtralConfig
    from levanter_b200.optim import AdamConfig
    from levanter_b200.trainer import Trainer, TrainerConfig

    cfg = C.decode(TrainerConfig, {"num_train_steps": steps, "train_batch_size": batch, "require_accelerator": False, "tracker": {"type": "noop"},
                                   "log_dir": f"{tmp}/logs", "id": "t", "seed": 1, "checkpointer": {"base_path": f"{tmp}/ckpt", "save_interval": "10h"}})
    g = torch.Generator().manual_seed(0)
    starts = torch.randint(0, VOCAB, (64,), generator=g)
    data = ListAsyncDataset([LmExample.causal(((s + torch.arange(16)) % VOCAB).to(torch.int32)) for s in starts], is_complete=True)
    # the load-balancing loss is not linear in the batch (per-rank token fractions), so it is left out of the comparison
    full_cfg = MixtralConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, n_routed_experts=4,
                             num_experts_per_tok=2, lbl_coef=None, rzl_coef=0.001, gradient_checkpointing=False)
    opt = AdamConfig(learning_rate=3e-3, warmup=0.0, weight_decay=0.0, lr_schedule="constant", min_lr_ratio=1.0)

    def model_init():
        full = full_cfg.build(VOCAB, seed=3)
        if world == 1:
            return full
        sliced = dataclasses.replace(full_cfg, expert_parallel=True).build(VOCAB, seed=3)
        src = dict(full.named_parameters())
        with torch.no_grad():
            for name, p in sliced.named_parameters():
                v = src[name]
                d = getattr(p, "ep_dim", None)
                if d is not None:
                    assert p.shape[d] * world == v.shape[d]
                    v = v.narrow(d, rank * p.shape[d], p.shape[d])
                p.copy_(v)
        return sliced

    losses = {}
    with Trainer(cfg, opt, compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=model_init)
        trainer.add_hook(lambda info: losses.__setitem__(info.step, float(info.loss)), every=1)
        info = trainer.train(state, trainer.data_loader(data).iter_from_step(int(state.step)))
    return {k: v.detach().clone() for k, v in info.state.model.named_parameters()}, [losses[k] for k in sorted(losses)]


def _worker(rank, world, port, tmp, steps):
    dist = _init(rank, world, port)
    try:
        params, losses = _train(tmp, steps, rank, world)
        torch.save({"params": params, "losses": losses}, f"{tmp}/rank{rank}.pt")
    finally:
        dist.destroy_process_group()


def test_expert_parallel_training_matches_single_process_and_resumes_on_one(tmp_path):
    single, losses = _train(str(tmp_path / "single"), steps=6)
    (tmp_path / "ep").mkdir()
    mp.spawn(_worker, args=(2, 29731, str(tmp_path / "ep"), 3), nprocs=2, join=True)
    for rank in range(2):
        got = torch.load(tmp_path / "ep" / f"rank{rank}.pt")
        assert got["losses"] == pytest.approx(losses[:3], abs=3e-5)
    # the two ranks' checkpoint holds every expert: one process with the whole model continues from it
    resumed, tail = _train(str(tmp_path / "ep"), steps=6)
    assert len(tail) == 3 and tail == pytest.approx(losses[3:], abs=5e-5)
    for k, v in single.items():
        assert torch.allclose(v, resumed[k], atol=5e-5), k


def test_expert_parallel_checkpoint_resumes_on_two_ranks(tmp_path):
    """The checkpoint holds every expert; on resume with sliced experts every rank reads back its own slice (parameters and
    optimizer moments)."""
    _, losses = _train(str(tmp_path / "single"), steps=6)
    (tmp_path / "ep").mkdir()
    mp.spawn(_worker, args=(2, 29735, str(tmp_path / "ep"), 3), nprocs=2, join=True)
    mp.spawn(_worker, args=(2, 29737, str(tmp_path / "ep"), 6), nprocs=2, join=True)
    for rank in range(2):
        got = torch.load(tmp_path / "ep" / f"rank{rank}.pt")
        assert len(got["losses"]) == 3 and got["losses"] == pytest.approx(losses[3:], abs=5e-5)


def _train_ep_tp(tmp, steps, rank=0, world=1):
    """Mixtral with the experts sliced over the data axis (2) and attention heads split over the model axis (2)."""
    from levanter_b200 import config as C
    from levanter_b200.data.dataset import ListAsyncDataset
    from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
    from levanter_b200.models.mixtral import MixtralConfig
    from levanter_b200.optim import OptimizerConfig
    from levanter_b200.parallel.tp import build_sharded_from_seed, gather_full_state
    from levanter_b200.trainer import Trainer, TrainerConfig

    extra = {"model_axis_size": 2, "tensor_parallel_axes": ["mlp", "heads"]} if world > 1 else {}
    cfg = C.decode(TrainerConfig, {"num_train_steps": steps, "train_batch_size": 8, "require_accelerator": False, "tracker": {"type": "noop"},
                                   "log_dir": f"{tmp}/logs", "id": "t", "seed": 1, "checkpointer": {"base_path": f"{tmp}/ckpt", "save_interval": "10h"},
                                   **extra})
    g = torch.Generator().manual_seed(0)
    starts = torch.randint(0, VOCAB, (64,), generator=g)
    data = ListAsyncDataset([LmExample.causal(((s + torch.arange(16)) % VOCAB).to(torch.int32)) for s in starts], is_complete=True)
    full_cfg = MixtralConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, n_routed_experts=4,
                             num_experts_per_tok=2, lbl_coef=None, rzl_coef=0.001, gradient_checkpointing=False)
    opt = C.decode(OptimizerConfig, {"type": "adam", "learning_rate": 3e-3, "warmup": 0.0, "weight_decay": 0.0, "lr_schedule": "constant",
                                     "min_lr_ratio": 1.0, "epsilon": 1e-4, "max_grad_norm": 0.5})
    losses = {}
    with Trainer(cfg, opt, compute_next_token_loss) as trainer:
        tp = trainer.tensor_parallel

        def model_init():
            if world == 1:
                return full_cfg.build(VOCAB, seed=3)
            from levanter_b200.parallel.expert import ExpertParallel

            ep = ExpertParallel.from_mesh(tp.mesh)
            assert ep is not None and ep.size == 2 and tp.size == 2
            sliced_cfg = dataclasses.replace(full_cfg, expert_parallel=True)
            # (the group is also found on the model's expert blocks when it is not passed)
            return build_sharded_from_seed(lambda tp: (sliced_cfg if tp is not None else full_cfg).build(VOCAB, seed=3, tp=tp), tp,
                                           ep if rank % 2 == 0 else None)

        state = trainer.initial_state(0, model_init=model_init)
        trainer.add_hook(lambda info: losses.__setitem__(info.step, float(info.loss)), every=1)
        info = trainer.train(state, trainer.data_loader(data).iter_from_step(int(state.step)))
        params = gather_full_state(info.state.model, tp) if tp is not None else {k: v.detach().clone() for k, v in info.state.model.named_parameters()}
        ep_dims = {n: getattr(p, "ep_dim", None) for n, p in info.state.model.named_parameters()}
    return params, [losses[k] for k in sorted(losses)], ep_dims


def _worker_ep_tp(rank, world, port, tmp, steps):
    dist = _init(rank, world, port)
    try:
        params, losses, ep_dims = _train_ep_tp(tmp, steps, rank, world)
        torch.save({"params": params, "losses": losses, "ep_dims": ep_dims}, f"{tmp}/rank{rank}.pt")
    finally:
        dist.destroy_process_group()


def test_expert_parallel_with_tensor_parallel_matches_single_process(tmp_path):
    """Four ranks: mesh data 2 x model 2.  Experts sliced over the data axis, attention over the model axis; the losses and the
    weights (expert slices re-assembled from the two data ranks) equal the single-process run."""
    single, losses, _ = _train_ep_tp(str(tmp_path / "single"), steps=3)
    (tmp_path / "d").mkdir()
    mp.spawn(_worker_ep_tp, args=(4, 29741, str(tmp_path / "d"), 3), nprocs=4, join=True)
    got = [torch.load(tmp_path / "d" / f"rank{r}.pt") for r in range(4)]
    for r in range(4):
        assert got[r]["losses"] == pytest.approx(losses, abs=3e-5)
    # which ranks share a model-axis group depends on the mesh layout: find the two data ranks by their differing expert slices
    ep_names = [n for n, d in got[0]["ep_dims"].items() if d is not None]
    assert ep_names
    for name, want in single.items():
        d = got[0]["ep_dims"][name]
        if d is None:
            assert torch.allclose(got[0]["params"][name], want, atol=5e-5), name
            continue
        n = want.shape[d] // 2
        slices = {0: want.narrow(d, 0, n), 1: want.narrow(d, n, n)}
        seen = set()
        for r in range(4):
            have = got[r]["params"][name]
            match = [i for i, s in slices.items() if torch.allclose(have, s, atol=5e-5)]
            assert match, (name, r)
            seen.add(match[0])
        assert seen == {0, 1}, name
