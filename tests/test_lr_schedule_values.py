"""Learning-rate schedule values at named steps: warm-up, decay shapes, cycles given as a count / a length / a list of
boundaries, re-warm-up and the stable phase of warm-up-stable-decay (levanter_b200/optim/config.py; the numbers are the ones the
reference's tests/test_optimizer_config.py expects of its schedules)."""
import numpy as np

from levanter_b200.optim import AdamConfig


def _sched(steps, **kw):
    kw.setdefault("weight_decay", 0.0)
    return AdamConfig(**kw).lr_scheduler(steps)


def test_linear_decay_to_zero_has_no_plateau():
    f = _sched(861, learning_rate=2e-6, warmup=0.03, min_lr_ratio=0.0, lr_schedule="linear", max_grad_norm=None, cycles=None,
               weight_decay_modules=None, default_weight_decay_mask=None)
    assert f(0) == 0.0
    assert np.isclose(f(int(861 * 0.03)), 2e-6)
    assert np.isclose(f(860), 0.0)
    assert np.isclose(f(int(861 * (0.03 + 0.97 / 2))), 1e-6)


def test_constant():
    f = _sched(1000, learning_rate=1e-3, warmup=0.0, min_lr_ratio=1.0, lr_schedule="constant", cycles=None)
    assert f(0) == 1e-3 and f(500) == 1e-3 and f(999) == 1e-3


def test_warmup_then_cosine():
    f = _sched(1000, learning_rate=1e-2, warmup=0.1, min_lr_ratio=0.1, lr_schedule="cosine", cycles=None)
    assert np.isclose(f(0), 0.0) and np.isclose(f(50), 0.5e-2) and np.isclose(f(100), 1e-2)
    assert np.isclose(f(999), 1e-3, atol=1e-5)
    assert all(f(s) > f(s + 1) for s in range(100, 998, 50))


def _check_two_linear_cycles(f):
    assert np.isclose(f(0), 0.0) and np.isclose(f(50), 5e-4)
    assert np.isclose(f(499), 0.2 * 5e-4, atol=1e-5)  # first nadir
    assert np.isclose(f(500), 5e-4)  # the second cycle starts at the top (no re-warm-up asked for)
    assert np.isclose(f(499 + 250), (5e-4 + 0.2 * 5e-4) / 2, atol=1e-5)
    assert np.isclose(f(999), 0.2 * 5e-4, atol=1e-5)


def test_linear_with_a_cycle_count():
    _check_two_linear_cycles(_sched(1000, learning_rate=5e-4, warmup=50, min_lr_ratio=0.2, lr_schedule="linear", cycles=2))


def test_linear_with_a_cycle_length():
    _check_two_linear_cycles(_sched(1000, learning_rate=5e-4, warmup=50, min_lr_ratio=0.2, lr_schedule="linear", cycle_length=500))


def _check_stable_then_decay_cycles(f):
    for start, stable_end, end in ((0, 269, 300), (300, 659, 700), (701, 969, 1000)):
        assert np.isclose(f(start), 1e-3) and np.isclose(f(stable_end), 1e-3)
        assert f(stable_end + 2) < 1e-3
    assert np.isclose(f(299), 1e-4, rtol=0.05) and np.isclose(f(999), 1e-4, rtol=0.05)


def test_stable_then_decay_with_cycle_boundaries():
    _check_stable_then_decay_cycles(_sched(1000, learning_rate=1e-3, warmup=0.0, decay=0.1, min_lr_ratio=0.1, lr_schedule="cosine",
                                           cycles=[300, 700]))


def test_stable_then_decay_with_cycle_lengths():
    _check_stable_then_decay_cycles(_sched(1000, learning_rate=1e-3, warmup=0.0, decay=0.1, min_lr_ratio=0.1, lr_schedule="cosine",
                                           cycle_length=[300, 400]))


def test_inverse_square_root():
    f = _sched(100_000, learning_rate=1e-3, warmup=0.1, min_lr_ratio=0.1, lr_schedule="inv_sqrt", cycles=None)
    assert np.isclose(f(0), 0.0) and np.isclose(f(5000), 0.5e-3)
    assert f(50000) < f(30000) < f(10000)


def test_rewarmup_at_the_start_of_later_cycles():
    f = _sched(1000, learning_rate=1e-2, warmup=0.2, min_lr_ratio=0.2, lr_schedule="linear", cycles=2, rewarmup=0.05)
    assert np.isclose(f(0), 0.0) and np.isclose(f(100), 1e-2)
    assert np.isclose(f(300), 0.6e-2) and np.isclose(f(500), 0.2e-2)
    top = 500 + int(0.05 * 500)
    assert np.isclose(f(top), 1e-2) and f(top - 1) < f(top) and f(top + 1) < f(top)
    assert f(998) > f(999) and np.isclose(f(999), 0.2e-2, atol=1e-4)
