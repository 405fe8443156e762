"""Functional helpers kept for parity with the reference's public surface: a train step on a plain parameter tree, the
saveable-state mask, matrix views of linear layers, and the paged-attention oracle under its reference name."""
import torch


def test_take_train_step_matches_manual_adam_and_respects_the_trainable_filter():
    from levanter_b200.optim import AdamConfig
    from levanter_b200.trainer_state import take_train_step

    torch.manual_seed(0)
    params = {"a.weight": torch.randn(4, 3), "b.weight": torch.randn(2, 2)}
    before = {k: v.clone() for k, v in params.items()}
    grads = {k: torch.randn_like(v) for k, v in params.items()}
    opt = AdamConfig(learning_rate=1e-2, weight_decay=0.0, warmup=0.0, lr_schedule="constant", min_lr_ratio=1.0, max_grad_norm=None).build(10)
    state = opt.init({"a.weight": params["a.weight"]})
    out, state, updates = take_train_step(opt, params, state, grads, is_trainable=lambda n: n.startswith("a."))
    assert out is params and set(updates) == {"a.weight"}
    assert torch.equal(params["b.weight"], before["b.weight"])  # frozen
    # first Adam step with bias correction: -lr * sign-like g / (|g| + eps)
    g = grads["a.weight"]
    expect = before["a.weight"] - 1e-2 * g / (g.abs() + 1e-8)
    torch.testing.assert_close(params["a.weight"], expect, atol=1e-5, rtol=1e-4)


def test_saveable_training_mask_keeps_trainable_float_parameters_only():
    from levanter_b200.config import Policy
    from levanter_b200.models.llama import LlamaConfig
    from levanter_b200.parallel.engine import ShardedEngine
    from levanter_b200.trainer_state import TrainerState, make_training_key, saveable_training_mask

    model = LlamaConfig(seq_len=8, hidden_dim=16, intermediate_dim=32, num_layers=1, num_heads=2, num_kv_heads=2).build(32, seed=0)
    trainable = lambda n: "mlp" in n  # noqa: E731
    eng = ShardedEngine(model, Policy.parse("f32"), None, device="cpu", is_trainable=trainable)
    st = TrainerState(0, model, eng, make_training_key(0), Policy.parse("f32"), None, trainable)
    mask = saveable_training_mask(st)
    assert mask["step"] and mask["training_key"] and mask["opt_state"] and not mask["model_averaging"]
    assert any(mask["model"].values()) and all(("mlp" in k) == v for k, v in mask["model"].items())


def test_linear_layers_as_matrices():
    from levanter_b200.optim.util import flatten_linear_layers, map_flattened_linear_layers, unflatten_linear_layers

    tree = {"w": torch.randn(4, 3), "experts": torch.randn(2, 5, 4, 3), "bias": torch.randn(4), "none": None}
    flat = flatten_linear_layers(tree)
    assert flat["w"].shape == (1, 4, 3) and flat["experts"].shape == (10, 4, 3) and flat["bias"].shape == (4,)
    back = unflatten_linear_layers(tree, flat)
    assert all(back[k] is None if tree[k] is None else torch.equal(back[k], tree[k]) for k in tree)
    # per-matrix map: Frobenius normalisation of each matrix, biases doubled
    out = map_flattened_linear_layers(lambda m: m / m.norm(), tree, or_else=lambda v: 2 * v)
    assert out["experts"].shape == tree["experts"].shape
    torch.testing.assert_close(out["experts"].reshape(10, -1).norm(dim=1), torch.ones(10))
    torch.testing.assert_close(out["w"].norm(), torch.tensor(1.0))
    assert torch.equal(out["bias"], 2 * tree["bias"]) and out["none"] is None


def test_default_ragged_paged_attention_is_the_oracle():
    from levanter_b200.layers.attention import default_ragged_paged_attention
    from levanter_b200.ops.paged_attention import ragged_paged_attention_reference

    torch.manual_seed(0)
    q = torch.randn(3, 4, 8)
    pages = torch.randn(6, 4, 4, 8)  # [page, slot, 2 * kv_head, head]
    kv_lens = torch.tensor([5, 6], dtype=torch.int32)
    page_idx = torch.tensor([[0, 1, -1], [2, 3, -1]], dtype=torch.int32)
    cu = torch.tensor([0, 1, 3], dtype=torch.int32)
    a = default_ragged_paged_attention(q, pages, kv_lens, page_idx, cu, 2, 0.35)
    b = ragged_paged_attention_reference(q, pages, kv_lens, page_idx, cu, 2, 0.35)
    assert torch.equal(a, b)


def test_trainer_checkpoint_path_and_artifacts(tmp_path):
    import gzip

    from levanter_b200 import config as C
    from levanter_b200.models.lm_model import compute_next_token_loss
    from levanter_b200.optim import AdamConfig
    from levanter_b200.trainer import Trainer, TrainerConfig

    def cfg(**kw):
        d = {"num_train_steps": 1, "train_batch_size": 2, "require_accelerator": False, "tracker": {"type": "noop"}, "log_dir": f"{tmp_path}/logs",
             "id": "run7", "checkpointer": {"base_path": f"{tmp_path}/ckpt"}}
        d.update(kw)
        return C.decode(TrainerConfig, d)

    with Trainer(cfg(), AdamConfig(), compute_next_token_loss) as trainer:
        assert trainer.checkpoint_path == f"{tmp_path}/ckpt/run7"
        text = trainer.write_artifact("notes.txt", "hello", type="text")
        blob = trainer.write_artifact("blob.bin.gz", b"\\x00\\x01\\x02")
        assert text == f"{tmp_path}/logs/run7/artifacts/notes.txt" and open(text).read() == "hello"
        assert gzip.open(blob, "rb").read() == b"\\x00\\x01\\x02"
    with Trainer(cfg(load_checkpoint_path="/some/other/run"), AdamConfig(), compute_next_token_loss) as trainer:
        assert trainer.checkpoint_path == "/some/other/run"


def test_total_dataset_tokens_future_feeds_the_epoch_progress_hook():
    import levanter_b200.tracker as T
    from levanter_b200.callbacks import get_total_dataset_tokens, log_epoch_progress
    from levanter_b200.data.dataset import EpochDataset, ListAsyncDataset

    class Recorder(T.NoopTracker):
        def __init__(self):
            self.logged, self.summary = [], {}

        def log(self, metrics, *, step, commit=None):
            self.logged.append((step, dict(metrics)))

        def log_summary(self, metrics):
            self.summary.update(metrics)

    rec = Recorder()
    with T.current_tracker(rec):
        ds = EpochDataset(ListAsyncDataset(list(range(50)), is_complete=True))
        fut = get_total_dataset_tokens(ds, 16)
        assert fut.result(timeout=10) == 800 and rec.summary == {"dataset/total_tokens": 800}
        hook = log_epoch_progress(fut, tokens_per_example=16, batch_size=5, max_epochs=2)

        class Info:
            def __init__(self, step):
                self.step, self.next_step = step, step + 1

        hook(Info(4))
        hook(Info(99))
    assert rec.logged[0] == (4, {"train/current_epoch": 16 * 5 * 5 / 800})
    assert rec.logged[1] == (99, {"train/current_epoch": 2})  # capped at max_epochs


def test_upload_to_hub_passes_the_repository_and_revision(monkeypatch, tmp_path):
    import sys
    import types

    from levanter_b200.compat.hf_checkpoints import RepoRef, upload_to_hub

    calls = []
    fake = types.ModuleType("huggingface_hub")
    fake.upload_folder = lambda **kw: calls.append(kw)
    monkeypatch.setitem(sys.modules, "huggingface_hub", fake)
    upload_to_hub(str(tmp_path), "org/model@dev", commit_message="step 10")
    upload_to_hub(str(tmp_path), RepoRef("org/other"))
    assert calls[0] == {"folder_path": str(tmp_path), "repo_id": "org/model", "revision": "dev", "commit_message": "step 10"}
    assert calls[1]["repo_id"] == "org/other" and calls[1]["revision"] is None


def test_trainable_subsets_and_casting_by_trainability():
    from levanter_b200.lora import LoraConfig, lora_trainable_params_filter, loraize
    from levanter_b200.models.llama import LlamaConfig
    from levanter_b200.optim import transforms as T
    from levanter_b200.trainer_state import (cast_params_by_trainability, init_optimizer_for_trainables, make_floating_point_trainable_filter,
                                             trainables_only)
    from levanter_b200.config import Policy

    model = loraize(LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=1, num_heads=2, num_kv_heads=2).build(40, seed=0),
                    LoraConfig(r=2, target_modules=["q_proj"]), seed=0)
    model.register_parameter("table", torch.nn.Parameter(torch.arange(4), requires_grad=False))
    is_lora = lora_trainable_params_filter(model)
    train = trainables_only(model, is_lora)
    assert train and all("lora" in n for n in train) and len(train) == 2
    everything = trainables_only(model)
    assert "table" not in everything and len(everything) == sum(1 for _ in model.parameters()) - 1
    f = make_floating_point_trainable_filter(model, is_lora)
    assert f(next(iter(train))) and not f("table") and not f("embeddings.token_embeddings.weight")
    state = init_optimizer_for_trainables(T.scale_by_adam(0.9, 0.95, 1e-8), train)
    assert set(state.mu) == set(train)
    cast_params_by_trainability(model, Policy.parse("p=f32,c=bf16"), is_lora)
    for n, p in model.named_parameters():
        if n == "table":
            assert p.dtype == torch.int64
        else:
            assert p.dtype == (torch.float32 if n in train else torch.bfloat16), n
