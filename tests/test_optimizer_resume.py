"""Every registered optimizer resumes exactly: a run interrupted after three steps and continued from its checkpoint follows the
same losses and ends at the same weights as an uninterrupted run (the optimizer states differ a lot in shape: moments, factored
preconditioners, eigenbases, per-group scalars, Hessian estimates, counters)."""
import pytest
import torch

from levanter_b200 import config as C
from levanter_b200.checkpoint import discover_latest_checkpoint
from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
from levanter_b200.optim import OptimizerConfig
from levanter_b200.trainer import Trainer, TrainerConfig

VOCAB = 64
OPTIMIZERS = ["adam", "adam+windows", "adopt", "cautious", "kron", "lion", "mars", "mini", "muon", "rmsprop", "scion", "soap", "sophia-h"]


def _run(tmp, steps, opt_name, dropout=False, averaging=None, return_average=False):
    cfg = C.decode(TrainerConfig, {"num_train_steps": steps, "train_batch_size": 8, "require_accelerator": False, "tracker": {"type": "noop"},
                                   "log_dir": f"{tmp}/logs", "id": "t", "seed": 1, "checkpointer": {"base_path": f"{tmp}/ckpt", "save_interval": "10h"},
                                   **({"model_averaging": averaging} if averaging else {})})
    g = torch.Generator().manual_seed(0)
    starts = torch.randint(0, VOCAB, (128,), generator=g)
    data = ListAsyncDataset([LmExample.causal(((s + torch.arange(16)) % VOCAB).to(torch.int32)) for s in starts], is_complete=True)
    extra = {"update_interval": 2} if opt_name == "sophia-h" else {"precondition_frequency": 2} if opt_name == "soap" else {}
    if opt_name == "adam+windows":  # Adam with every stateful wrapper: skip-step window, update-norm window, RMS clipping
        opt_name, extra = "adam", {"skip_bad_steps": 4, "clip_update_norm": {"rolling_interval_length": 4, "sigma_factor": 2.0}, "update_rms_clipping": 1.0}
    opt = C.decode(OptimizerConfig, {"type": opt_name, "learning_rate": 3e-3, "warmup": 0.0, "weight_decay": 0.01, "lr_schedule": "constant", "min_lr_ratio": 1.0, **extra})  # (a schedule that does not depend on the run length)
    mc = LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, gradient_checkpointing=False)
    if dropout:
        from levanter_b200.models.gpt2 import Gpt2Config

        mc = Gpt2Config(seq_len=16, hidden_dim=32, num_layers=2, num_heads=2, gradient_checkpointing=False, resid_pdrop=0.2, embed_pdrop=0.1, attn_pdrop=0.1)
    losses = {}
    with Trainer(cfg, opt, compute_next_token_loss) as trainer:
        state = trainer.initial_state(0, model_init=lambda: mc.build(VOCAB, seed=3))
        first = int(state.step)
        trainer.add_hook(lambda info: losses.__setitem__(info.step, float(info.loss)), every=1)
        info = trainer.train(state, trainer.data_loader(data).iter_from_step(first))
        if return_average:
            return first, losses, {n: p.detach().clone() for n, p in info.state.eval_model.named_parameters()}
    return first, losses, {n: p.detach().clone() for n, p in info.state.model.named_parameters()}


@pytest.mark.parametrize("opt_name", OPTIMIZERS)
def test_an_interrupted_run_continues_as_if_it_had_not_stopped(tmp_path, opt_name):
    d = str(tmp_path)
    _, full_losses, full_params = _run(d + "/full", 6, opt_name)
    _run(d + "/run", 3, opt_name)
    assert discover_latest_checkpoint(d + "/run/ckpt/t").endswith("step-2")
    first, losses, params = _run(d + "/run", 6, opt_name)
    assert first == 3 and sorted(losses) == [3, 4, 5]
    assert [losses[i] for i in (3, 4, 5)] == pytest.approx([full_losses[i] for i in (3, 4, 5)], rel=2e-5, abs=2e-5)
    for n in full_params:
        assert torch.allclose(params[n], full_params[n], atol=2e-5), n


def test_dropout_masks_are_a_function_of_the_step_so_resuming_does_not_change_them(tmp_path):
    d = str(tmp_path)
    _, full_losses, full_params = _run(d + "/full", 6, "adam", dropout=True)
    _, no_dropout, _ = _run(d + "/plain", 6, "adam", dropout=False)
    _run(d + "/run", 3, "adam", dropout=True)
    first, losses, params = _run(d + "/run", 6, "adam", dropout=True)
    assert first == 3 and [losses[i] for i in (3, 4, 5)] == pytest.approx([full_losses[i] for i in (3, 4, 5)], rel=2e-5, abs=2e-5)
    for n in full_params:
        assert torch.allclose(params[n], full_params[n], atol=2e-5), n
    again = _run(d + "/again", 6, "adam", dropout=True)[1]
    assert [again[i] for i in range(6)] == pytest.approx([full_losses[i] for i in range(6)], abs=1e-6)  # and the same from run to run


@pytest.mark.parametrize("averaging", [{"type": "ema", "beta": 0.5}, {"type": "ema_decay_sqrt", "beta": 0.5, "switch_step": 2, "decay_steps": 6}])
def test_the_averaged_weights_resume_too(tmp_path, averaging):
    d = str(tmp_path)
    _, _, full_avg = _run(d + "/full", 6, "adam", averaging=averaging, return_average=True)
    _, _, full_raw = _run(d + "/raw", 6, "adam", averaging=averaging)
    assert any(not torch.allclose(full_avg[n], full_raw[n], atol=1e-4) for n in full_avg)  # the average lags behind the weights
    _run(d + "/run", 3, "adam", averaging=averaging)
    first, _, avg = _run(d + "/run", 6, "adam", averaging=averaging, return_average=True)
    assert first == 3
    for n in full_avg:
        assert torch.allclose(avg[n], full_avg[n], atol=2e-5), n
