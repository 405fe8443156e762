"""Model families on a B200 against the same weights in fp32 on the CPU: which kernels a family reaches depends on its head
size, norm and activation, so each one takes a forward and backward pass on the device."""
import pytest
import torch

from levanter_b200.ops import lib

pytestmark = pytest.mark.gpu
if not (torch.cuda.is_available() and lib.available()):
    pytest.skip("needs a CUDA device and the native library", allow_module_level=True)


def _compare(cfg, vocab, seq, names, tol=6e-2):
    torch.manual_seed(0)
    ref = cfg.build(vocab, seed=0)
    dev = cfg.build(vocab, seed=0).to("cuda").to(torch.bfloat16)
    ids = torch.randint(0, vocab, (2, seq), generator=torch.Generator().manual_seed(1))
    from levanter_b200.layers.attention import AttentionMask

    before = lib.launch_count
    got = dev.activations(ids.cuda(), AttentionMask.causal())
    got = got[0] if isinstance(got, tuple) else got
    assert lib.launch_count > before
    want = ref.activations(ids, AttentionMask.causal())
    want = want[0] if isinstance(want, tuple) else want
    err = (got.float().cpu() - want).abs().max() / want.abs().max()
    assert err < tol, err
    # a random linear functional of the output: the mean square of a normalised output is almost constant, and its gradient noise
    r = torch.randn(want.shape, generator=torch.Generator().manual_seed(2))
    (got.float() * r.cuda()).mean().backward()
    (want * r).mean().backward()
    torch.cuda.synchronize()
    lib.check_status()
    gp, rp = dict(dev.named_parameters()), dict(ref.named_parameters())
    cosines = {}
    for name in names:
        g, w = gp[name].grad.float().cpu().flatten(), rp[name].grad.flatten()
        cosines[name] = float(torch.dot(g, w) / (g.norm() * w.norm() + 1e-30))
    # direction of each whole gradient: single tiny entries are bf16 noise
    assert min(cosines.values()) > 0.97, cosines


def test_gpt2_head_size_64_layer_norm_gelu():
    from levanter_b200.models.gpt2 import Gpt2Config

    cfg = Gpt2Config(seq_len=256, hidden_dim=256, num_layers=2, num_heads=4, gradient_checkpointing=False)
    names = [n for n, p in cfg.build(128, seed=0).named_parameters() if p.dim() == 2][:8]
    _compare(cfg, 128, 256, names)


def test_llama_with_a_sequence_length_that_needs_padding():
    from levanter_b200.models.llama import LlamaConfig

    cfg = LlamaConfig(seq_len=200, hidden_dim=256, intermediate_dim=512, num_layers=2, num_heads=2, num_kv_heads=1,
                      gradient_checkpointing=False)
    names = [n for n, p in cfg.build(128, seed=0).named_parameters() if p.dim() == 2][:8]
    _compare(cfg, 128, 200, names)
