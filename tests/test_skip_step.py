"""Skip-step: dropping outlier updates against a rolling window, and the checkpoint layout that lets runs with and without the
wrapper start from each other's checkpoints (levanter_b200/optim/skipstep.py; scenarios after the reference's tests/test_skip_step.py)."""
import pytest
import torch

from levanter_b200 import config as C
from levanter_b200.checkpoint import discover_latest_checkpoint
from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
from levanter_b200.optim import AdamConfig
from levanter_b200.optim import transforms as T
from levanter_b200.optim.skipstep import SkipStepConfig, SkipStepState
from levanter_b200.tensorstore_serialization import leaf_key_paths, tree_deserialize_leaves_tensorstore, tree_serialize_leaves_tensorstore
from levanter_b200.trainer import Trainer, TrainerConfig


class _CountState(dict):
    pass


def _counting_inner():
    """An inner transformation that counts its calls and passes the gradient through negated."""
    def init(params):
        return {"calls": torch.zeros((), dtype=torch.int64)}

    def update(updates, state, params=None, **extra):
        return {k: -v for k, v in updates.items()}, {"calls": state["calls"] + 1}

    return T.GradientTransformation(init, update)


P = {"w": torch.tensor([1.0, 2.0]), "b": torch.tensor([0.5])}
G = {"w": torch.tensor([0.1, 0.1]), "b": torch.tensor([0.1])}


def _warm(opt, state, n, loss=1.0):
    for i in range(n):
        _, state = opt.update(G, state, P, loss=torch.tensor(loss + 0.01 * (i % 2)))
    return state


def test_config_from_bool_int_or_config():
    assert SkipStepConfig.from_bool_int_or_config(False) is None
    assert SkipStepConfig.from_bool_int_or_config(True) == SkipStepConfig()
    assert SkipStepConfig.from_bool_int_or_config(32).rolling_interval_length == 32
    c = SkipStepConfig(rolling_interval_length=7, sigma_factor=2.0)
    assert SkipStepConfig.from_bool_int_or_config(c) is c
    with pytest.raises(ValueError):
        SkipStepConfig.from_bool_int_or_config("yes")


def test_initial_state():
    opt = SkipStepConfig(rolling_interval_length=5).wrap(_counting_inner())
    s = opt.init(P)
    assert isinstance(s, SkipStepState) and s.losses.shape == (5,) and s.grad_norms.shape == (5,)
    assert not s.valid_mask.any() and s.current_idx == 0 and s.count == 0 and int(s.inner_opt_state["calls"]) == 0


def test_the_loss_is_a_required_keyword():
    opt = SkipStepConfig(rolling_interval_length=5).wrap(_counting_inner())
    with pytest.raises(ValueError, match="[Ll]oss"):
        opt.update(G, opt.init(P), P)


def test_nothing_is_skipped_before_half_a_window_is_seen():
    opt = SkipStepConfig(rolling_interval_length=8, sigma_factor=1.0).wrap(_counting_inner())
    s = opt.init(P)
    # wild values from the first step on: fewer than four points, so every update is applied
    for i, loss in enumerate([1.0, 1000.0, 1.0]):
        u, s = opt.update(G, s, P, loss=torch.tensor(loss))
        assert float(u["w"][0]) == pytest.approx(-0.1) and int(s.inner_opt_state["calls"]) == i + 1
    assert s.count == 3 and s.current_idx == 3 and s.valid_mask.tolist() == [True] * 3 + [False] * 5


@pytest.mark.parametrize("trigger", ["loss", "grad_norm"])
def test_an_outlier_is_skipped_and_the_inner_state_is_kept(trigger):
    opt = SkipStepConfig(rolling_interval_length=6, sigma_factor=2.0).wrap(_counting_inner())
    s = _warm(opt, opt.init(P), 6)
    calls = int(s.inner_opt_state["calls"])
    big_g = {k: v * 1e4 for k, v in G.items()}
    u, s2 = opt.update(big_g if trigger == "grad_norm" else G, s, P, loss=torch.tensor(1e4 if trigger == "loss" else 1.0))
    assert all(float(v.abs().sum()) == 0 for v in u.values())  # a zero update
    assert int(s2.inner_opt_state["calls"]) == calls  # the inner transformation did not run
    # the outlier still enters the window
    assert float(s2.losses[s.current_idx]) == pytest.approx(1e4 if trigger == "loss" else 1.0)
    assert s2.current_idx == (s.current_idx + 1) % 6 and s2.count == 6
    # an ordinary step right after is applied again
    u, s3 = opt.update(G, s2, P, loss=torch.tensor(1.0))
    assert float(u["w"][0]) == pytest.approx(-0.1) and int(s3.inner_opt_state["calls"]) == calls + 1


def test_the_window_is_circular_and_the_count_is_capped():
    opt = SkipStepConfig(rolling_interval_length=4, sigma_factor=100.0).wrap(_counting_inner())
    s = opt.init(P)
    for i in range(6):
        _, s = opt.update(G, s, P, loss=torch.tensor(float(i)))
    assert s.count == 4 and s.current_idx == 2
    assert s.losses.tolist() == [4.0, 5.0, 2.0, 3.0] and s.valid_mask.all()


def test_adam_config_builds_the_wrapper_and_trains_through_outliers():
    cfg = AdamConfig(learning_rate=0.1, warmup=0.0, weight_decay=0.0, lr_schedule="constant", min_lr_ratio=1.0, max_grad_norm=None,
                     skip_bad_steps=SkipStepConfig(rolling_interval_length=4, sigma_factor=2.0))
    assert not cfg.fused_kernel_eligible()
    opt = cfg.build(100)
    p = {"w.weight": torch.tensor([1.0, -1.0])}
    s = opt.init(p)
    for i in range(4):
        u, s = opt.update({"w.weight": torch.tensor([0.5, 0.5])}, s, p, loss=torch.tensor(1.0 + 0.01 * i))
        p = {"w.weight": p["w.weight"] + u["w.weight"]}
    before = p["w.weight"].clone()
    u, s = opt.update({"w.weight": torch.tensor([0.5, 0.5])}, s, p, loss=torch.tensor(50.0))
    assert float(u["w.weight"].abs().sum()) == 0 and torch.equal(p["w.weight"] + u["w.weight"], before)
    assert AdamConfig(skip_bad_steps=16).build(10) is not None and AdamConfig(skip_bad_steps=True).build(10) is not None


def test_checkpoint_keys_splice_the_inner_state_in_place():
    inner = T.chain(T.clip_by_global_norm(1.0), T.scale_by_adam(0.9, 0.95, 1e-8), T.scale(-1.0))
    plain = dict(leaf_key_paths(inner.init(P), "opt"))
    wrapped = dict(leaf_key_paths(SkipStepConfig(rolling_interval_length=5).wrap(inner).init(P), "opt"))
    assert set(plain) <= set(wrapped)
    assert set(wrapped) - set(plain) == {f"opt._skipstep_{f}" for f in ("losses", "grad_norms", "valid_mask", "current_idx", "count")}
    assert any(k.endswith(".mu.w") for k in plain)


def test_a_wrapped_state_loads_from_a_checkpoint_written_without_the_wrapper_and_back(tmp_path):
    inner = T.chain(T.scale_by_adam(0.9, 0.95, 1e-8), T.scale(-1.0))
    _, plain = inner.update(G, inner.init(P), P)  # one step, so that the moments are not zero
    tree_serialize_leaves_tensorstore(str(tmp_path / "plain"), plain)
    wrapped_opt = SkipStepConfig(rolling_interval_length=5).wrap(inner)
    with pytest.raises(FileNotFoundError):
        tree_deserialize_leaves_tensorstore(str(tmp_path / "plain"), wrapped_opt.init(P))
    restored = tree_deserialize_leaves_tensorstore(str(tmp_path / "plain"), wrapped_opt.init(P), allow_missing=True)
    assert isinstance(restored, SkipStepState) and restored.count == 0 and not restored.valid_mask.any()
    for (ka, a), (kb, b) in zip(leaf_key_paths(restored.inner_opt_state), leaf_key_paths(plain)):
        assert ka == kb and torch.equal(torch.as_tensor(a), torch.as_tensor(b))

    # the other direction: a run without the wrapper reads the moments out of a wrapped checkpoint
    s = _warm(wrapped_opt, restored, 3)
    tree_serialize_leaves_tensorstore(str(tmp_path / "wrapped"), s)
    back = tree_deserialize_leaves_tensorstore(str(tmp_path / "wrapped"), inner.init(P))
    for (ka, a), (kb, b) in zip(leaf_key_paths(back), leaf_key_paths(s.inner_opt_state)):
        assert ka == kb and torch.equal(torch.as_tensor(a), torch.as_tensor(b))
    again = tree_deserialize_leaves_tensorstore(str(tmp_path / "wrapped"), wrapped_opt.init(P))
    assert again.count == 3 and again.current_idx == 3 and torch.equal(again.losses, s.losses)


VOCAB = 64


def _train(tmp, steps, skip):
    cfg = C.decode(TrainerConfig, {"num_train_steps": steps, "train_batch_size": 8, "require_accelerator": False, "tracker": {"type": "noop"},
                                   "log_dir": f"{tmp}/logs", "id": "t", "seed": 1, "checkpointer": {"base_path": f"{tmp}/ckpt", "save_interval": "10h"}})
    g = torch.Generator().manual_seed(0)
    starts = torch.randint(0, VOCAB, (256,), generator=g)
    data = ListAsyncDataset([LmExample.causal(((s + torch.arange(16)) % VOCAB).to(torch.int32)) for s in starts], is_complete=True)
    opt = AdamConfig(learning_rate=3e-3, warmup=0.0, weight_decay=0.0, lr_schedule="constant", min_lr_ratio=1.0, skip_bad_steps=skip)
    mc = LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, gradient_checkpointing=False)
    losses = {}
    with Trainer(cfg, opt, compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=lambda: mc.build(VOCAB, seed=3))
        first = int(state.step)
        trainer.add_hook(lambda info: losses.__setitem__(info.step, float(info.loss)), every=1)
        info = trainer.train(state, trainer.data_loader(data).iter_from_step(first))
    return first, losses, info


def test_a_run_with_skip_step_resumes_from_a_checkpoint_written_without_it(tmp_path):
    d = str(tmp_path)
    _, ref, _ = _train(d + "/ref", 6, skip=False)
    _train(d + "/run", 3, skip=False)
    assert discover_latest_checkpoint(d + "/run/ckpt/t").endswith("step-2")
    first, losses, info = _train(d + "/run", 6, skip=8)  # same run directory, now with the wrapper
    assert first == 3 and sorted(losses) == [3, 4, 5]
    # the moments came from the checkpoint (a fresh optimizer would give other losses) and no step is skipped this early
    assert [losses[i] for i in (3, 4, 5)] == pytest.approx([ref[i] for i in (3, 4, 5)], abs=1e-5)
    # and back again: the plain optimizer continues from the wrapped run's checkpoint
    first, _, _ = _train(d + "/run", 8, skip=False)
    assert first == 6
