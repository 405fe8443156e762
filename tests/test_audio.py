"""Audio pipeline: log-mel features against the Hugging Face Whisper extractor, the batch processor, a serial cache and a
tiny end-to-end ASR training run (modelled on the reference's tests/test_audio.py and tests/test_train_asr.py)."""
import json
import math
import wave

import numpy as np
import pytest
import torch

from levanter_b200 import config as C
from levanter_b200.data.audio import (AudioIODatasetConfig, AudioTextDataset, AudioTextUrlDataSource, BatchAudioProcessor,
                                      LogMelFeatureExtractor, ProcessedAudioCache, mel_filter_bank)
from levanter_b200.data.passthrough_tokenizer import PassthroughTokenizer


def _tone(seconds=1.0, f=440.0, sr=16000, seed=0):
    t = np.arange(int(seconds * sr)) / sr
    rng = np.random.default_rng(seed)
    return (0.5 * np.sin(2 * math.pi * f * t) + 0.01 * rng.standard_normal(t.shape)).astype(np.float32)


def test_log_mel_matches_hf_whisper_extractor():
    transformers = pytest.importorskip("transformers")
    hf = transformers.WhisperFeatureExtractor(feature_size=80)
    ours = LogMelFeatureExtractor()
    assert np.allclose(mel_filter_bank(201, 80, 16000, 0.0, 8000.0), np.asarray(hf.mel_filters), atol=1e-6)
    waves = [_tone(1.3, 300.0), _tone(0.7, 1200.0, seed=1)]
    a = ours(waves, sampling_rate=16000)["input_features"]
    b = hf(waves, sampling_rate=16000, return_tensors="np")["input_features"]
    assert a.shape == b.shape == (2, 80, 3000)
    assert np.abs(a - b).max() < 2e-3


def test_batch_processor_shapes_and_metadata():
    tok = PassthroughTokenizer(100, pad_token_id=0)
    bp = BatchAudioProcessor(LogMelFeatureExtractor(), tok, max_length=16)
    out = bp([(_tone(0.5), 16000, "5 6 7"), (_tone(0.2), 16000, "8 9")])
    assert out[0]["input_features"].shape == (80, 3000) and out[0]["input_features"].dtype == np.float32
    assert out[0]["input_ids"].shape == (16,) and out[0]["input_ids"][:4].tolist() == [5, 6, 7, 99]  # EOS appended, then padding
    assert out[1]["attention_mask"].sum() == 3
    assert set(bp.output_exemplar) == {"input_features", "input_ids", "attention_mask"}
    md = bp.metadata
    assert md["processor"]["feature_size"] == 80 and md["tokenizer"]["max_length"] == 16
    with pytest.raises(AssertionError):
        bp([(_tone(0.1), 16000, "1"), (_tone(0.1), 8000, "2")])


def _write_wav(path, x, sr=16000):
    with wave.open(str(path), "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(sr)
        w.writeframes((np.clip(x, -1, 1) * 32767).astype("<i2").tobytes())


def _write_corpus(d, n=8):
    rows = []
    for i in range(n):
        p = d / f"a{i}.wav"
        _write_wav(p, _tone(0.3 + 0.05 * i, 200.0 + 50 * i, seed=i))
        rows.append({"audio": {"path": str(p)}, "sentence": " ".join(str(3 + (i + j) % 20) for j in range(4))})
    with open(d / "train.jsonl", "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    return str(d / "train.jsonl")


def test_url_source_cache_and_dataset(tmp_path):
    url = _write_corpus(tmp_path)
    src = AudioTextUrlDataSource([url])
    first = next(iter(src.open_shard(src.shard_names[0])))
    assert first[1] == 16000 and first[2] == "3 4 5 6" and abs(len(first[0]) - 4800) <= 1
    tok = PassthroughTokenizer(100, pad_token_id=0)
    cache = ProcessedAudioCache.build_or_load(str(tmp_path / "cache"), src, LogMelFeatureExtractor(chunk_length=1), tok, max_length=8)
    assert len(cache.cache) == 8
    ds = AudioTextDataset(cache, ignore_index=0)
    ex = ds.as_sync_dataset()[2] if hasattr(ds, "as_sync_dataset") else None
    if ex is None:
        import asyncio

        ex = asyncio.run(ds.get_batch([2]))[0]
    assert ex.audio.shape == (80, 100) and ex.tokens.shape == (8,)
    # 4 transcript ids + EOS then padding: positions whose next token is padding carry no loss
    assert ex.loss_mask.tolist() == [1, 1, 1, 1, 0, 0, 0, 0]


@pytest.mark.entry
def test_train_asr_tiny(tmp_path, monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    from levanter_b200.main import train_asr

    url = _write_corpus(tmp_path, n=16)
    d = str(tmp_path)
    cfg = {
        "data": {"train_urls": [url], "validation_urls": [url], "cache_dir": f"{d}/cache", "tokenizer": "passthrough", "vocab_size": 100, "processor": "builtin",
                 "max_length": 8},
        "model": {"type": "whisper", "d_model": 32, "encoder_layers": 1, "decoder_layers": 1, "encoder_attention_heads": 2,
                  "decoder_attention_heads": 2, "encoder_ffn_dim": 64, "decoder_ffn_dim": 64, "max_length": 8, "vocab_size": 100,
                  "gradient_checkpointing": False},
        "trainer": {"num_train_steps": 3, "train_batch_size": 4, "require_accelerator": False, "tracker": {"type": "noop"},
                    "log_dir": f"{d}/logs", "id": "asrrun", "steps_per_eval": 2, "max_eval_batches": 1, "per_device_eval_parallelism": 4,
                    "checkpointer": {"base_path": f"{d}/ckpt", "save_interval": "1h"}},
        "optimizer": {"learning_rate": 1e-3, "warmup": 0.0},
    }
    train_asr.main(C.decode(train_asr.TrainASRConfig, cfg))


def test_audio_mixture_of_two_sources(tmp_path):
    import asyncio

    from levanter_b200.data.audio import AudioDatasetSourceConfig, AudioMixtureDatasetConfig
    from levanter_b200.data.mixture import MixtureDataset

    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    url_a, url_b = _write_corpus(tmp_path / "a", n=6), _write_corpus(tmp_path / "b", n=4)
    common = dict(cache_dir=f"{tmp_path}/cache", tokenizer="passthrough", vocab_size=100, processor="builtin", max_length=8)
    cfg = AudioMixtureDatasetConfig(configs={"a": AudioDatasetSourceConfig(train_urls=[url_a], validation_urls=[url_a]),
                                             "b": AudioDatasetSourceConfig(train_urls=[url_b]),
                                             "unused": AudioDatasetSourceConfig(train_urls=[url_b])},
                                    train_weights={"a": 0.75, "b": 0.25, "unused": 0.0}, mixture_block_size=4, shuffle=True, **common)
    caches = cfg.build_caches("train")
    assert set(caches) == {"a", "b"}  # a source with weight zero is not even built
    train = cfg.train_set(key=3)
    assert isinstance(train, MixtureDataset)
    rows = asyncio.run(train.get_batch(list(range(8))))
    assert all(r["input_features"].shape[0] == 80 and r["input_ids"].shape == (8,) for r in rows)
    val = cfg.validation_sets()
    assert set(val) == {"a"} and asyncio.run(val["a"].async_len()) == 6  # only the source that names validation data
    assert asyncio.run(caches["a"].async_len()) == 6 and asyncio.run(caches["b"].async_len()) == 4

    with pytest.raises(ValueError, match="At least one dataset"):
        AudioMixtureDatasetConfig(configs={}, train_weights={})
    with pytest.raises(ValueError, match="must be the same"):
        AudioMixtureDatasetConfig(configs={"a": AudioDatasetSourceConfig(train_urls=[url_a])}, train_weights={"b": 1.0})
    by_yaml = C.decode(AudioMixtureDatasetConfig, {"configs": {"a": {"train_urls": [url_a]}}, "train_weights": {"a": 1.0}, "shuffle": 16, **common})
    assert by_yaml.shuffle == 16 and asyncio.run(by_yaml.train_set(key=0).get_batch([0]))[0]["input_ids"].shape == (8,)
