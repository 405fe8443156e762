"""Whisper: numerical parity with the Hugging Face implementation on a tiny random model, loss masking, config round trip."""
import pytest
import torch

from levanter_b200.compat.hf_checkpoints import load_hf_state_dict, to_hf_state_dict
from levanter_b200.models.asr_model import ASRConfig, AudioTextExample
from levanter_b200.models.whisper import WhisperConfig, WhisperModel, whisper_sinusoids


def _tiny():
    return WhisperConfig(d_model=32, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=64, decoder_layers=2,
                         decoder_attention_heads=4, decoder_ffn_dim=64, num_mel_bins=8, max_source_positions=20, max_length=12,
                         vocab_size=50, gradient_checkpointing=False)


def test_matches_hf_whisper():
    transformers = pytest.importorskip("transformers")
    cfg = _tiny()
    hf_cfg = transformers.WhisperConfig(**{k: v for k, v in cfg.to_hf_config(50).items() if k not in ("model_type", "architectures")},
                                        pad_token_id=0, bos_token_id=1, eos_token_id=2, decoder_start_token_id=1,
                                        suppress_tokens=None, begin_suppress_tokens=None)
    torch.manual_seed(0)
    hf = transformers.WhisperForConditionalGeneration(hf_cfg).eval()
    model = WhisperModel.init(50, cfg).eval()
    missing = load_hf_state_dict(model, hf.state_dict(), ignore_prefix="model")
    assert missing == []
    mel = torch.randn(2, 8, 40)
    ids = torch.randint(3, 50, (2, 12))
    with torch.no_grad():
        ours = model(mel, ids)
        theirs = hf(input_features=mel, decoder_input_ids=ids).logits
    assert torch.allclose(ours, theirs, atol=2e-4, rtol=1e-4), (ours - theirs).abs().max()
    # exporting gives back the same tensors under the checkpoint's names
    sd = to_hf_state_dict(model)
    ref = hf.state_dict()
    for k, v in sd.items():
        key = k if k in ref else "model." + k
        assert key in ref, k
        assert torch.equal(v, ref[key]), k


def test_sinusoids_and_positions():
    s = whisper_sinusoids(6, 8)
    assert s.shape == (6, 8)
    assert torch.allclose(s[0], torch.tensor([0.0] * 4 + [1.0] * 4))
    m = WhisperModel.init(50, _tiny())
    assert float(m.decoder.embed_positions.weight.abs().sum()) == 0.0
    assert m.decoder.embed_tokens.weight.shape == (50, 32)


def test_loss_mask_and_loss():
    cfg = _tiny()
    model = WhisperModel.init(50, cfg)
    tokens = torch.tensor([[5, 6, 7, 0, 0, 0, 0, 0, 0, 0, 0, 0]])
    ex = AudioTextExample.init(torch.randn(1, 8, 40), tokens, ignore_id=0)
    # the last position never counts; a position counts only if the next token is not padding
    assert ex.loss_mask.tolist() == [[1, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0]]
    loss = model.compute_loss(ex)
    assert loss.dim() == 0 and torch.isfinite(loss)
    per_tok = model.compute_loss(ex, reduction=None)
    assert torch.allclose(per_tok.sum() / 2, loss)
    loss.backward()
    assert model.encoder.conv1.weight.grad is not None and model.decoder.embed_tokens.weight.grad is not None


def test_config_registry_and_hf_round_trip():
    assert ASRConfig.get_choice_class("whisper") is WhisperConfig
    cfg = _tiny()
    back = WhisperConfig.from_hf_config(cfg.to_hf_config(50))
    assert back.d_model == 32 and back.max_length == 12 and back.encoder_ffn_dim == 64 and back.num_mel_bins == 8
