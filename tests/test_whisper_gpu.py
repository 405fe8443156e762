"""Whisper on a B200: the bf16 model on the kernel paths (stem convolutions as GEMMs, encoder / decoder / cross attention on the
flash kernels with head size 64) against the same weights in fp32 on the CPU."""
import pytest
import torch

from levanter_b200.ops import lib

pytestmark = pytest.mark.gpu
if not (torch.cuda.is_available() and lib.available()):
    pytest.skip("needs a CUDA device and the native library", allow_module_level=True)

from levanter_b200.models.whisper import WhisperConfig, WhisperModel


def test_whisper_forward_and_backward_match_the_cpu_model():
    cfg = WhisperConfig(d_model=256, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=512, decoder_layers=2,
                        decoder_attention_heads=4, decoder_ffn_dim=512, num_mel_bins=80, max_source_positions=300, max_length=64,
                        vocab_size=512, gradient_checkpointing=False)
    torch.manual_seed(0)
    ref = WhisperModel.init(512, cfg)
    dev = WhisperModel.init(512, cfg)
    dev.load_state_dict(ref.state_dict())
    dev = dev.to("cuda").to(torch.bfloat16)
    mel = torch.randn(2, 80, 600)
    ids = torch.randint(3, 512, (2, 64))
    before = lib.launch_count
    out = dev(mel.cuda().bfloat16(), ids.cuda())
    assert lib.launch_count - before >= 2 * 2 + 2 * 3 + 2  # attention launches of both stacks plus the two stem GEMMs at least
    want = ref(mel, ids)
    err = (out.float().cpu() - want).abs().max() / want.abs().max()
    assert err < 5e-2, err
    out.float().square().mean().backward()
    want.square().mean().backward()
    torch.cuda.synchronize()
    lib.check_status()
    for name in ("encoder.conv1.weight", "encoder.conv2.weight", "decoder.layers.0.encoder_attn.q_proj.weight",
                 "encoder.layers.1.self_attn.v_proj.weight", "decoder.embed_tokens.weight"):
        g = dict(dev.named_parameters())[name].grad.float().cpu()
        w = dict(ref.named_parameters())[name].grad
        assert (g - w).abs().max() <= 0.08 * w.abs().max() + 1e-6, name
