"""Gradient transformations against PyTorch's own optimizers and closed forms, the composition helpers (chain, masked,
multi_transform, inject_hyperparams) and the learning-rate schedule registry (levanter_b200/optim/transforms.py, optim/config.py)."""
import math

import pytest
import torch

from levanter_b200 import config as C
from levanter_b200.optim import AdamConfig
from levanter_b200.optim import transforms as T
from levanter_b200.optim.config import LrSchedule


def _params():
    g = torch.Generator().manual_seed(0)
    return {"a.weight": torch.randn(4, 3, generator=g), "a.bias": torch.randn(3, generator=g)}


def _grads(step):
    g = torch.Generator().manual_seed(100 + step)
    return {"a.weight": torch.randn(4, 3, generator=g), "a.bias": torch.randn(3, generator=g)}


def _run(opt, steps=4):
    params = {k: v.clone() for k, v in _params().items()}
    state = opt.init(params)
    for s in range(steps):
        updates, state = opt.update({k: v.clone() for k, v in _grads(s).items()}, state, params)
        T.apply_updates(params, updates)
    return params, state


def _run_torch(make, steps=4):
    params = {k: torch.nn.Parameter(v.clone()) for k, v in _params().items()}
    opt = make(list(params.values()))
    for s in range(steps):
        for k, g in _grads(s).items():
            params[k].grad = g.clone()
        opt.step()
    return {k: v.detach() for k, v in params.items()}


@pytest.mark.parametrize("nesterov", [False, True])
def test_momentum_matches_torch_sgd(nesterov):
    ours, _ = _run(T.chain(T.trace(0.9, nesterov=nesterov), T.scale(-0.1)))
    ref = _run_torch(lambda p: torch.optim.SGD(p, lr=0.1, momentum=0.9, nesterov=nesterov))
    for k in ours:
        assert torch.allclose(ours[k], ref[k], atol=1e-6), k


def test_rms_scaling_matches_torch_rmsprop():
    ours, _ = _run(T.chain(T.scale_by_rms(decay=0.95, eps=1e-8), T.scale(-0.01)))
    ref = _run_torch(lambda p: torch.optim.RMSprop(p, lr=0.01, alpha=0.95, eps=1e-8))
    for k in ours:
        assert torch.allclose(ours[k], ref[k], atol=1e-6), k
    _, state = _run(T.scale_by_rms(initial_scale=1.0), steps=0)
    assert all(float(v.min()) == 1.0 for v in state.nu.values())


def test_adam_with_decoupled_decay_and_clipping_matches_torch_adamw():
    ours, _ = _run(T.chain(T.scale_by_adam(0.9, 0.95, 1e-8), T.add_decayed_weights(0.1), T.scale(-0.01)))
    ref = _run_torch(lambda p: torch.optim.AdamW(p, lr=0.01, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1))
    for k in ours:
        assert torch.allclose(ours[k], ref[k], atol=1e-5), k
    clipped, _ = T.clip_by_global_norm(0.5).update({k: v.clone() for k, v in _grads(0).items()}, T.EmptyState())
    assert float(T.global_norm(clipped)) == pytest.approx(0.5, rel=1e-5)
    small = {k: v * 1e-3 for k, v in _grads(0).items()}
    same, _ = T.clip_by_global_norm(0.5).update({k: v.clone() for k, v in small.items()}, T.EmptyState())
    assert all(torch.equal(same[k], small[k]) for k in small)


def test_lion_sign_and_ema_by_hand():
    g0, g1 = _grads(0), _grads(1)
    opt = T.scale_by_lion(0.9, 0.99)
    s = opt.init(_params())
    u0, s = opt.update(dict(g0), s)
    u1, s = opt.update(dict(g1), s)
    assert torch.equal(u0["a.bias"], torch.sign(0.1 * g0["a.bias"]))
    mu1 = 0.01 * g0["a.bias"]
    assert torch.equal(u1["a.bias"], torch.sign(0.9 * mu1 + 0.1 * g1["a.bias"])) and s.count == 2
    assert torch.allclose(s.mu["a.bias"], 0.99 * mu1 + 0.01 * g1["a.bias"])

    signs, _ = T.scale_by_sign().update({"x": torch.tensor([-2.0, 0.0, 3.0])}, T.EmptyState())
    assert signs["x"].tolist() == [-1.0, 0.0, 1.0]

    e = T.ema(0.5, debias=True)
    st = e.init({"x": torch.zeros(1)})
    out, st = e.update({"x": torch.tensor([4.0])}, st)
    assert out["x"].item() == pytest.approx(4.0)  # debiased: the first value itself
    out, st = e.update({"x": torch.tensor([0.0])}, st)
    assert out["x"].item() == pytest.approx((0.5 * 2.0) / 0.75) and st.count == 2
    plain = T.ema(0.5)
    out, _ = plain.update({"x": torch.tensor([4.0])}, plain.init({"x": torch.zeros(1)}))
    assert out["x"].item() == pytest.approx(2.0)


def test_identity_schedules_and_learning_rate_scaling():
    u = {"x": torch.ones(2)}
    same, state = T.identity().update(dict(u), T.identity().init(u))
    assert torch.equal(same["x"], u["x"]) and state == T.EmptyState()
    sched = T.scale_by_schedule(lambda c: 0.5 ** c)
    st = sched.init(u)
    seen = []
    for _ in range(3):
        out, st = sched.update({"x": torch.ones(2)}, st)
        seen.append(out["x"][0].item())
    assert seen == [1.0, 0.5, 0.25] and st.count == 3
    out, _ = T.scale_by_learning_rate(0.1).update({"x": torch.ones(2)}, T.EmptyState())
    assert out["x"][0].item() == pytest.approx(-0.1)
    lr = T.scale_by_learning_rate(lambda c: 0.1 * (c + 1), flip_sign=False)
    st = lr.init(u)
    _, st = lr.update({"x": torch.ones(2)}, st)
    out, st = lr.update({"x": torch.ones(2)}, st)
    assert out["x"][0].item() == pytest.approx(0.2)

    f = T.join_schedules([T.linear_schedule(0.0, 1.0, 10), T.cosine_decay_schedule(1.0, 90, alpha=0.1)], [10])
    assert f(0) == 0.0 and f(5) == pytest.approx(0.5) and f(10) == pytest.approx(1.0) and f(100) == pytest.approx(0.1)
    assert T.constant_schedule(3.0)(10 ** 6) == 3.0 and T.linear_schedule(1.0, 0.0, 10, transition_begin=5)(10) == pytest.approx(0.5)


def test_masked_and_multi_transform_route_leaves():
    grads = {"a.weight": torch.ones(2), "a.bias": torch.ones(2), "frozen": None}
    only_w = T.masked(T.scale(10.0), lambda tree: {k: k.endswith("weight") for k in tree})
    out, _ = only_w.update({k: (None if v is None else v.clone()) for k, v in grads.items()}, only_w.init(grads))  # (updates are consumed in place)
    assert out["a.weight"].tolist() == [10.0, 10.0] and out["a.bias"].tolist() == [1.0, 1.0] and out["frozen"] is None

    routed = T.multi_transform({"big": T.scale(2.0), "small": T.chain(T.trace(0.5), T.scale(-1.0))},
                               lambda tree: {k: ("big" if k.endswith("weight") else "small") for k in tree})
    st = routed.init({k: v for k, v in grads.items()})
    assert set(st.inner_states) == {"big", "small"}
    out, st = routed.update({k: (None if v is None else v.clone()) for k, v in grads.items()}, st)
    out, st = routed.update({k: (None if v is None else v.clone()) for k, v in grads.items()}, st)
    assert out["a.weight"].tolist() == [2.0, 2.0] and out["a.bias"].tolist() == [-1.5, -1.5]  # momentum kept its own state


def test_injected_hyperparameters_follow_the_schedule_and_are_logged_in_the_state():
    opt = T.inject_hyperparams(lambda learning_rate: T.scale(-learning_rate))(learning_rate=lambda c: 0.1 / (c + 1))
    p = {"x": torch.zeros(1)}
    st = opt.init(p)
    u0, st = opt.update({"x": torch.ones(1)}, st, p)
    u1, st = opt.update({"x": torch.ones(1)}, st, p)
    assert u0["x"].item() == pytest.approx(-0.1) and u1["x"].item() == pytest.approx(-0.05)
    assert st.count == 2 and float(st.hyperparams["learning_rate"]) == pytest.approx(0.05)


def test_learning_rate_schedules_from_the_registry():
    assert set(LrSchedule._registry_root._choice_registry) >= {"constant", "cosine", "linear", "inv_sqrt", "inv", "power"}
    cos2 = C.decode(AdamConfig, {"learning_rate": 1.0, "warmup": 0.0, "min_lr_ratio": 0.0, "lr_schedule": {"type": "cosine", "exponent": 2.0}})
    plain = AdamConfig(learning_rate=1.0, warmup=0.0, min_lr_ratio=0.0, lr_schedule="cosine")
    assert cos2.lr_scheduler(100)(50) == pytest.approx(plain.lr_scheduler(100)(50) ** 2)

    inv = AdamConfig(learning_rate=1.0, warmup=0.0, min_lr_ratio=0.1, lr_schedule="inv").lr_scheduler(100)
    # lr / ((lr / min_lr - 1) * max(step, 1) / decay_steps + 1): the step count is clamped to 1, as in the reference
    assert inv(0) == inv(1) == pytest.approx(1.0 / (9 * 1 / 100 + 1)) and inv(100) == pytest.approx(0.1) and inv(10) > inv(50) > inv(99)
    by_name = C.decode(AdamConfig, {"learning_rate": 1.0, "warmup": 0.0, "min_lr_ratio": 0.1, "lr_schedule": {"type": "inv"}}).lr_scheduler(100)
    assert [by_name(s) for s in (0, 10, 99)] == [inv(s) for s in (0, 10, 99)]

    inv_sqrt = C.decode(AdamConfig, {"learning_rate": 1.0, "warmup": 100, "min_lr_ratio": 0.0, "lr_schedule": {"type": "inv_sqrt", "timescale": 100}})
    f = inv_sqrt.lr_scheduler(10000)
    assert f(100) == pytest.approx(1.0) and f(400) == pytest.approx(1 / math.sqrt(4.0))

    power = C.decode(AdamConfig, {"learning_rate": 1e-2, "warmup": 0.0, "lr_schedule": {"type": "power", "batch_size": 8, "seq_length": 128, "a": 4.6, "b": -0.51}})
    g = power.lr_scheduler(10 ** 6)
    assert g(0) == 1e-2 and g(10 ** 5) == pytest.approx(min(1e-2, 8 * 4.6 * (10 ** 5 * 8 * 128) ** -0.51))
    with pytest.raises(ValueError):
        C.decode(AdamConfig, {"lr_schedule": {"type": "power", "a": -1.0}})
    with pytest.raises(ValueError):
        AdamConfig(lr_schedule="sawtooth").lr_scheduler(10)
    with pytest.raises(ValueError):
        AdamConfig(warmup=1.5).lr_scheduler(10)


def test_hessian_vector_products_noise_trees_block_clipping_and_norm_logging():
    import levanter_b200.tracker as Tr
    from levanter_b200.optim.util import hvp, log_norm_passthrough, scan_aware_clip_by_block_rms, tree_gaussian_like

    # f(x, y) = x^T A x + sum(x) * sum(y): Hessian blocks 2A (x, x), ones (x, y), zero (y, y)
    A = torch.tensor([[2.0, 1.0], [1.0, 3.0]])
    params = {"x": torch.tensor([1.0, -1.0]), "y": torch.tensor([0.5, 0.25, 2.0]), "ids": None}

    def f(p):
        return p["x"] @ A @ p["x"] + p["x"].sum() * p["y"].sum()

    v = {"x": torch.tensor([1.0, 2.0]), "y": torch.tensor([1.0, 0.0, -1.0]), "ids": None}
    hv = hvp(f, params, v)
    assert torch.allclose(hv["x"], 2 * A @ v["x"] + v["y"].sum()) and torch.allclose(hv["y"], torch.full((3,), v["x"].sum()))
    assert set(hv) == {"x", "y"} and not params["x"].requires_grad  # the caller's tensors are left as they were

    g = torch.Generator().manual_seed(0)
    noise = tree_gaussian_like({"w": torch.zeros(200, 200, dtype=torch.bfloat16), "i": torch.zeros(3, dtype=torch.int32), "n": None}, generator=g)
    assert noise["i"] is None and noise["n"] is None and noise["w"].dtype == torch.bfloat16
    assert abs(float(noise["w"].float().mean())) < 0.02 and abs(float(noise["w"].float().std()) - 1.0) < 0.02

    clip = scan_aware_clip_by_block_rms(1.0)
    out, _ = clip.update({"big": torch.full((4,), 3.0), "small": torch.full((4,), 0.5)}, clip.init({}))
    assert torch.allclose(out["big"], torch.ones(4)) and torch.allclose(out["small"], torch.full((4,), 0.5))  # each tensor by its own RMS

    with Tr.defer_tracker_for_jit() as logged:
        same, _ = log_norm_passthrough("optim/pre_clip_norm").update({"a": torch.tensor([3.0, 4.0])}, T.EmptyState())
    assert same["a"].tolist() == [3.0, 4.0] and logged["optim/pre_clip_norm"] == pytest.approx(5.0)
