"""Smaller components: background iteration, time-delta codec, LoRA, Sophia, model averaging, token re-initialisation,
stop-signal helpers, page cloning (modelled on the reference's test_background_iterable.py, test_datetime_utils.py,
test_lora.py, test_sophia.py, test_model_averaging.py, test_sft.py, inference/test_inference_utils.py, test_clone_pages.py)."""
import datetime
import json
import os
import time

import numpy as np
import pytest
import torch
import torch.nn as nn

from levanter_b200.utils.background_iterable import BackgroundIterable
from levanter_b200.utils.datetime_utils import encode_timedelta, parse_timedelta


# ------------------------------------------------------------------------------------------------ background iteration
def test_background_iterable_order_reentrancy_and_empty():
    it = BackgroundIterable(lambda: iter(range(50)), max_capacity=4)
    assert list(it) == list(range(50))
    assert list(it) == list(range(50))  # a fresh producer per iteration
    assert list(BackgroundIterable(lambda: iter(()), max_capacity=2)) == []


def test_background_iterable_reraises_producer_errors():
    def gen():
        yield 1
        raise ValueError("boom in producer")

    got = []
    with pytest.raises(ValueError, match="boom in producer"):
        for x in BackgroundIterable(gen, max_capacity=2):
            got.append(x)
    assert got == [1]


def test_background_iterable_stop_unblocks_a_full_queue():
    def endless():
        i = 0
        while True:
            yield i
            i += 1

    it = iter(BackgroundIterable(endless, max_capacity=2))
    assert next(it) == 0
    t0 = time.time()
    it.stop()
    assert time.time() - t0 < 5


def test_background_iterable_over_async_producers():
    import asyncio

    async def numbers():
        for i in range(20):
            await asyncio.sleep(0)
            yield i

    it = BackgroundIterable(numbers, max_capacity=3)
    assert list(it) == list(range(20)) and list(it) == list(range(20))

    async def nothing():
        return
        yield  # pragma: no cover

    assert list(BackgroundIterable(nothing, max_capacity=2)) == []

    async def failing():
        yield 1
        raise ValueError("boom in async producer")

    got = []
    with pytest.raises(ValueError, match="boom in async producer"):
        for x in BackgroundIterable(failing, max_capacity=2):
            got.append(x)
    assert got == [1]

    async def endless():
        i = 0
        while True:
            yield i
            i += 1
            await asyncio.sleep(0)

    run = iter(BackgroundIterable(endless, max_capacity=2))
    assert next(run) == 0 and next(run) == 1
    t0 = time.time()
    run.stop()
    assert time.time() - t0 < 5
    with pytest.raises(StopIteration):
        while True:
            next(run)


def test_background_iterable_without_a_capacity_limit_runs_ahead():
    produced = []

    def gen():
        for i in range(100):
            produced.append(i)
            yield i

    it = iter(BackgroundIterable(gen, max_capacity=None))
    assert next(it) == 0
    deadline = time.time() + 5
    while len(produced) < 100 and time.time() < deadline:
        time.sleep(0.01)
    assert len(produced) == 100  # the producer did not wait for the consumer
    assert list(it) == list(range(1, 100))


# ------------------------------------------------------------------------------------------------ time deltas
@pytest.mark.parametrize("text,seconds", [("30m", 1800), ("1h30m", 5400), ("1d2h3m4.5s", 93784.5), ("15", 15), ("2 hours", 7200), ("90s", 90)])
def test_parse_timedelta(text, seconds):
    assert parse_timedelta(text).total_seconds() == pytest.approx(seconds)


def test_encode_timedelta_round_trip():
    for td in (datetime.timedelta(minutes=15), datetime.timedelta(days=1, hours=2, seconds=3), datetime.timedelta(seconds=0.5)):
        assert parse_timedelta(encode_timedelta(td)) == td


# ------------------------------------------------------------------------------------------------ LoRA
def _tiny_llama():
    from levanter_b200.models.llama import LlamaConfig

    return LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, gradient_checkpointing=False).build(50, seed=0)


def test_loraize_targets_zero_init_and_merge(tmp_path):
    from levanter_b200.layers.attention import AttentionMask
    from levanter_b200.lora import (LoraConfig, LoraLinear, lora_state_dict, lora_trainable_params_filter, loraize, merge_lora_modules,
                                    save_peft_pretrained)

    base = _tiny_llama().eval()
    ids = torch.randint(0, 50, (2, 16), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        ref = base.activations(ids, AttentionMask.causal()).clone()
    cfg = LoraConfig(r=4, alpha=8.0, target_modules=["q_proj", "v_proj"])
    m = loraize(base, cfg, seed=1)
    wrapped = [n for n, mod in m.named_modules() if isinstance(mod, LoraLinear)]
    assert len(wrapped) == 4 and all(n.endswith(("q_proj", "v_proj")) for n in wrapped)
    with torch.no_grad():
        assert torch.allclose(m.activations(ids, AttentionMask.causal()), ref, atol=1e-6)  # B starts at zero: no change yet
    train = lora_trainable_params_filter(m)
    names = [n for n, _ in m.named_parameters()]
    assert all(("lora" in n) == train(n) for n in names) and any(train(n) for n in names)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.05)
        moved = m.activations(ids, AttentionMask.causal()).clone()
    assert not torch.allclose(moved, ref, atol=1e-4)
    sd = lora_state_dict(m)
    assert len(sd) == 8 and all(k.startswith("base_model.model.") for k in sd)
    save_peft_pretrained(m, cfg, "some/base", str(tmp_path / "peft"))
    acfg = json.load(open(tmp_path / "peft" / "adapter_config.json"))
    assert acfg["r"] == 4 and acfg["lora_alpha"] == 8.0 and sorted(acfg["target_modules"]) == ["q_proj", "v_proj"]
    assert any(f.startswith("adapter_model") for f in os.listdir(tmp_path / "peft"))
    merged = merge_lora_modules(m)
    assert not any(isinstance(mod, LoraLinear) for mod in merged.modules())
    with torch.no_grad():
        assert torch.allclose(merged.activations(ids, AttentionMask.causal()), moved, atol=1e-5)


# ------------------------------------------------------------------------------------------------ Sophia
def test_sophia_h_minimises_a_quadratic():
    from levanter_b200 import config as C
    from levanter_b200.optim import OptimizerConfig
    from levanter_b200.optim import transforms as T

    cfg = C.decode(OptimizerConfig, {"type": "sophia-h", "learning_rate": 5e-2, "warmup": 0.0, "weight_decay": 0.0, "min_lr_ratio": 1.0,
                                     "lr_schedule": "constant", "update_interval": 2})
    torch.manual_seed(0)
    target = {"w.weight": torch.randn(6, 6)}
    scales = {"w.weight": torch.linspace(0.5, 4.0, 36).reshape(6, 6)}
    params = {"w.weight": torch.zeros(6, 6)}
    opt = cfg.build(120)
    state = opt.init(params)

    def objective(p):
        return sum((scales[k] * (p[k] - target[k]) ** 2).sum() for k in p)

    first = float(objective(params))
    for _ in range(120):
        leaves = {k: v.clone().requires_grad_() for k, v in params.items()}
        loss = objective(leaves)
        grads = dict(zip(leaves, torch.autograd.grad(loss, list(leaves.values()))))
        updates, state = opt.update(grads, state, params, obj_fn=objective)
        T.apply_updates(params, updates)
    assert float(objective(params)) < 0.05 * first  # clipped steps of at most lr per element: 120 steps cover the distance


# ------------------------------------------------------------------------------------------------ model averaging
def test_ema_decay_sqrt_phases():
    from levanter_b200.optim.model_averaging import EmaDecaySqrtConfig

    avg = EmaDecaySqrtConfig(beta=0.5, switch_step=3).create({"w": torch.zeros(1)})
    vals = []
    for step in range(1, 8):
        avg = avg.update({"w": torch.ones(1)}, step)
        p = avg.model_params if not callable(avg.model_params) else avg.model_params()
        vals.append(float(p["w"]))
    assert all(b >= a - 1e-7 for a, b in zip(vals, vals[1:])) and 0.5 <= vals[0] < 1.0 and vals[-1] <= 1.0 + 1e-6


# ------------------------------------------------------------------------------------------------ SFT token re-initialisation
def test_reinitialize_some_tokens_draws_rows_near_the_matrix_statistics():
    from levanter_b200.main.sft import reinitialize_some_tokens

    class Tok:
        vocab = {"<a>": 3, "<b>": 7}

        def convert_tokens_to_ids(self, t):
            return self.vocab.get(t)

        def convert_ids_to_tokens(self, i):
            return {v: k for k, v in self.vocab.items()}.get(i)

    class Engine:
        def __init__(self, model):
            self.model = model

        def full_master(self):
            return {n: p.detach().clone() for n, p in self.model.named_parameters()}

        def load_full_params(self, full):
            with torch.no_grad():
                for n, p in self.model.named_parameters():
                    if n in full:
                        p.copy_(full[n])

    class State:
        pass

    m = _tiny_llama()
    st = State()
    st.model, st.engine = m, Engine(m)
    emb_name = next(n for n, _ in m.named_parameters() if "token_embeddings" in n)
    before = dict(m.named_parameters())[emb_name].detach().clone()
    reinitialize_some_tokens(st, Tok(), ["<a>", "<b>"], key=0)
    after = dict(m.named_parameters())[emb_name].detach()
    changed = (after != before).any(dim=1).nonzero().flatten().tolist()
    assert changed == [3, 7]
    assert float(after[[3, 7]].abs().max()) < 6 * float(before.std()) + float(before.mean().abs()) + 1e-3
    with pytest.raises(ValueError):
        reinitialize_some_tokens(st, Tok(), [], key=0)
    with pytest.raises(ValueError):
        reinitialize_some_tokens(st, Tok(), ["<not in the vocabulary>"], key=0)


# ------------------------------------------------------------------------------------------------ inference helpers
def test_is_stop_signal_and_purge():
    from levanter_b200.inference.utils import INVALID, get_unique_in_order, is_stop_signal, purge

    stops = np.array([[INVALID, 5, 6], [INVALID, INVALID, 9]], dtype=np.int32)
    assert is_stop_signal(np.array([1, 5, 6]), stops) and is_stop_signal(np.array([7, 8, 9]), stops)
    assert not is_stop_signal(np.array([5, 6, 1]), stops)
    assert not is_stop_signal(np.array([1, 2, 3]), np.full((2, 3), INVALID, dtype=np.int32))  # padding-only rows never match
    assert not is_stop_signal(np.array([1, 2, 3]), np.zeros((0, 3), dtype=np.int32))
    out = purge(np.array([4, 5, 6, 7]), np.array([False, True, False, True]))
    assert out.tolist() == [4, 6, INVALID, INVALID]
    uniq, index = get_unique_in_order(np.array([3, 1, 3, 2, 1]), size=4)
    assert uniq.tolist() == [3, 1, 2, INVALID] and index.tolist() == [0, 1, 0, 2, 1]


def test_clone_pages_shares_full_pages_and_copies_a_partial_last_page():
    from levanter_b200.inference.page_table import PageTable

    pt = PageTable.init(max_pages=8, max_seqs=3, page_size=4, max_pages_per_seq=4)
    pt, parent = pt.assign_seq_id_to_seq()
    pt, _ = pt.allocate_for_seq(np.array([parent] * 6, dtype=np.int32), np.arange(6, dtype=np.int32))  # 6 tokens: one full page + half
    pt, child = pt.assign_seq_id_to_seq()
    pt = pt.clone_pages_from(parent, child)
    pp, cp = pt.page_indices[parent], pt.page_indices[child]
    assert cp[0] == pp[0] and pt.page_ref_counts[pp[0]] == 2       # the full page is shared
    assert cp[1] != pp[1] and pt.page_ref_counts[cp[1]] == 1      # the partial last page gets a fresh copy target
    assert pt.seq_lens[child] == 6
    pt = pt.free_pages(child)
    assert pt.page_ref_counts[pp[0]] == 1 and not pt.used_mask[child]
