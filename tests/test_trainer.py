"""Trainer on CPU: the loss goes down, micro-batching gives the same update as one big batch, hooks run on their cadence,
checkpoints restore the exact trajectory (model, optimizer state, step and data position), model averaging is evaluated
(modelled on the reference's tests/test_train_step.py, test_grad_accum.py, test_checkpoint.py, test_trainer_resume.py)."""
import copy
import datetime
import os

import pytest
import torch

from levanter_b200 import config as C
from levanter_b200.checkpoint import Checkpointer, CheckpointInterval, discover_latest_checkpoint, load_checkpoint, save_checkpoint
from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
from levanter_b200.optim import AdamConfig
from levanter_b200.trainer import Trainer, TrainerConfig

VOCAB = 64


def _cfg(tmp, steps=6, batch=8, pdp=-1, **kw):
    d = {"num_train_steps": steps, "train_batch_size": batch, "per_device_parallelism": pdp, "require_accelerator": False,
         "tracker": {"type": "noop"}, "log_dir": f"{tmp}/logs", "id": "t", "seed": 1,
         "checkpointer": {"base_path": f"{tmp}/ckpt", "save_interval": "10h"}}
    d.update(kw)
    return C.decode(TrainerConfig, d)


def _model_cfg():
    return LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, gradient_checkpointing=False)


def _data(n=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    # a learnable pattern: token t+1 = (token t + 1) mod VOCAB
    starts = torch.randint(0, VOCAB, (n,), generator=g)
    return ListAsyncDataset([LmExample.causal(((s + torch.arange(16)) % VOCAB).to(torch.int32)) for s in starts], is_complete=True)


def _opt(lr=3e-3):
    return AdamConfig(learning_rate=lr, warmup=0.0, weight_decay=0.0, lr_schedule="constant", min_lr_ratio=1.0)


def _run(tmp, steps, pdp=-1, data=None, **kw):
    cfg = _cfg(tmp, steps=steps, pdp=pdp, **kw)
    by_step = {}  # (the trainer forces every hook once more after the last step, so a step can be seen twice)
    with Trainer(cfg, _opt(), compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=lambda: _model_cfg().build(VOCAB, seed=3))
        trainer.add_hook(lambda info: by_step.__setitem__(info.step, float(info.loss)), every=1)
        loader = trainer.data_loader(data or _data()).iter_from_step(int(state.step))
        info = trainer.train(state, loader)
    return info, [by_step[k] for k in sorted(by_step)]


def test_loss_decreases(tmp_path):
    info, losses = _run(str(tmp_path), steps=30)
    assert info.step == 29 and len(losses) == 30
    assert sum(losses[-5:]) / 5 < sum(losses[:5]) / 5 - 0.3


def test_microbatching_matches_full_batch(tmp_path):
    a, la = _run(str(tmp_path / "a"), steps=3, pdp=-1)
    b, lb = _run(str(tmp_path / "b"), steps=3, pdp=2)
    assert la == pytest.approx(lb, abs=2e-5)
    for (n, p), (_, q) in zip(a.state.model.named_parameters(), b.state.model.named_parameters()):
        assert torch.allclose(p, q, atol=2e-5), n


def test_hooks_cadence_and_step_numbering(tmp_path):
    cfg = _cfg(str(tmp_path), steps=7)
    seen, seen3 = [], []
    with Trainer(cfg, _opt(), compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=lambda: _model_cfg().build(VOCAB, seed=3))
        trainer.add_hook(lambda info: seen.append(info.step), every=1)
        trainer.add_hook(lambda info: seen3.append(info.step), every=3)
        trainer.train(state, trainer.data_loader(_data()).iter_from_step(0))
    # every hook is forced once more after the last step
    assert seen == list(range(7)) + [6] and seen3 == [0, 3, 6, 6]


def test_resume_reproduces_uninterrupted_run(tmp_path):
    full, lf = _run(str(tmp_path / "full"), steps=6)
    # first half: 3 steps, the final forced save lands at step 2 (the step just completed)
    _run(str(tmp_path / "res"), steps=3)
    ck = discover_latest_checkpoint(str(tmp_path / "res/ckpt/t"))
    assert ck is not None and ck.endswith("step-2")
    resumed, lr = _run(str(tmp_path / "res"), steps=6)
    assert len(lr) == 3  # only steps 3..5 ran
    assert lr == pytest.approx(lf[3:], abs=1e-5)
    for (n, p), (_, q) in zip(full.state.model.named_parameters(), resumed.state.model.named_parameters()):
        assert torch.allclose(p, q, atol=1e-5), n


def test_model_averaging_is_tracked_and_evaluated(tmp_path):
    cfg = _cfg(str(tmp_path), steps=4, model_averaging={"type": "ema", "beta": 0.5})
    with Trainer(cfg, _opt(1e-2), compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=lambda: _model_cfg().build(VOCAB, seed=3))
        info = trainer.train(state, trainer.data_loader(_data()).iter_from_step(0))
    live = dict(info.state.model.named_parameters())
    avg = dict(info.state.eval_model.named_parameters())
    k = next(iter(live))
    assert not torch.allclose(live[k], avg[k])  # the averaged weights trail the live ones


# ------------------------------------------------------------------------------------------------ checkpointer policies
class _Info:
    def __init__(self, step, state=None):
        self.step, self.state = step, state


def test_checkpointer_step_policies_and_time_policy(tmp_path):
    now = [datetime.datetime(2024, 1, 1)]
    saved = []
    ck = Checkpointer(str(tmp_path), datetime.timedelta(minutes=10), [CheckpointInterval(every=5, until=10), CheckpointInterval(every=20)],
                      dt_now_injection=lambda: now[0])
    ck.save_checkpoint = lambda info, dest, commit_callback=None, **kw: (saved.append((info.step, kw.get("is_temporary", False))),
                                                                           commit_callback and commit_callback())
    for step in range(1, 45):
        now[0] += datetime.timedelta(minutes=1)
        ck.on_step(_Info(step))
    perm = [s for s, tmp in saved if not tmp]
    temp = [s for s, tmp in saved if tmp]
    assert perm == [5, 10, 20, 40]
    assert temp and all(s not in perm for s in temp)  # time-based saves between the permanent ones are temporary
    with pytest.raises(ValueError):
        Checkpointer(str(tmp_path), None, [CheckpointInterval(every=5, until=None), CheckpointInterval(every=20, until=100)])


def test_save_and_load_tree_round_trip(tmp_path):
    m = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    tree = {"model": {k: v.detach() for k, v in m.state_dict().items()}, "step": 12, "extra": {"count": torch.tensor(5)}}
    path = save_checkpoint(tree, 12, str(tmp_path / "step-12"))
    assert os.path.exists(os.path.join(path, "metadata.json"))
    m2 = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    load_checkpoint(m2, str(tmp_path), subpath="model")
    for (k, a), (_, b) in zip(m.state_dict().items(), m2.state_dict().items()):
        assert torch.equal(a, b), k
    (tmp_path / "step-20").mkdir()  # no metadata: not a checkpoint
    assert discover_latest_checkpoint(str(tmp_path)).endswith("step-12")
    with pytest.raises(FileNotFoundError):
        load_checkpoint(m2, str(tmp_path / "nothing_here"))


def test_sophia_h_through_trainer(tmp_path):
    """Sophia-H gets the batch objective from the trainer: the run passes the Hessian refresh and the estimate changes."""
    from levanter_b200.optim import OptimizerConfig

    ocfg = C.decode(OptimizerConfig, {"type": "sophia-h", "learning_rate": 1e-3, "warmup": 0.0, "update_interval": 2,
                                      "lr_schedule": "constant", "min_lr_ratio": 1.0})
    cfg = _cfg(str(tmp_path), steps=5, pdp=4)
    with Trainer(cfg, ocfg, compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=lambda: _model_cfg().build(VOCAB, seed=3))
        info = trainer.train(state, trainer.data_loader(_data()).iter_from_step(0))
    assert info.step == 4

    def find(st):
        if hasattr(st, "hessian_count"):
            return st
        if isinstance(st, (tuple, list)):
            for x in st:
                r = find(x)
                if r is not None:
                    return r
        for name in ("inner_state",):
            if hasattr(st, name):
                return find(getattr(st, name))
        return None

    soph = find(state.engine.opt_state)
    assert soph is not None and soph.hessian_count == 2  # steps 2 and 4 of 5
    assert any(float(h.abs().sum()) > 0 for h in soph.h.values())


def test_mid_run_checkpoint_commits_without_waiting(tmp_path):
    """A save made by ``on_step`` becomes discoverable on its own (no ``wait_until_finished``), and the temporary checkpoint
    it replaces is deleted while the run is still going."""
    import time
    from types import SimpleNamespace

    cfg = _cfg(str(tmp_path), steps=1)
    with Trainer(cfg, _opt(), compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=lambda: _model_cfg().build(VOCAB, seed=3))
        base = str(tmp_path / "ck")
        now = [datetime.datetime(2024, 1, 1)]
        ck = Checkpointer(base, datetime.timedelta(minutes=10), [], dt_now_injection=lambda: now[0])
        ck.on_step(SimpleNamespace(step=0, state=state))
        found = []
        for step in (1, 2):
            now[0] += datetime.timedelta(minutes=11)
            ck.on_step(SimpleNamespace(step=step, state=state))
            deadline = time.monotonic() + 30
            while time.monotonic() < deadline:
                latest = discover_latest_checkpoint(base)
                if latest is not None and latest.endswith(f"step-{step}"):
                    break
                time.sleep(0.05)
            found.append(discover_latest_checkpoint(base))
        assert found[0].endswith("step-1") and found[1].endswith("step-2")
        deadline = time.monotonic() + 30
        while os.path.exists(os.path.join(base, "step-1")) and time.monotonic() < deadline:
            time.sleep(0.05)
        assert not os.path.exists(os.path.join(base, "step-1")), "the replaced temporary checkpoint is still there"
        ck.wait_until_finished()
