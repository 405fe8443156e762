"""Audio-text data for speech recognition (src/levanter/data/audio.py:71-620): Whisper log-mel feature extraction, a
batch processor that turns ``(waveform, sampling_rate, text)`` into cached rows, single-source and mixture dataset configs
and the dataset that yields :class:`~levanter_b200.models.asr_model.AudioTextExample`.

The log-mel front end is implemented here in PyTorch (STFT with a Hann window, Slaney-normalised mel filters, log10,
8-decade dynamic range, ``(x + 4) / 4``) and reproduces the Hugging Face ``WhisperFeatureExtractor``; a Hugging Face
extractor object may be passed instead and is then used as is."""
from __future__ import annotations

import json
import logging
import os
import wave
from dataclasses import dataclass, field
from functools import cached_property
from typing import Any, Dict, Iterator, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..models.asr_model import AudioTextExample
from ..store.cache import CacheOptions, TreeCache, build_or_load_cache
from ..utils.fsspec_utils import expand_glob
from ._preprocessor import BatchProcessor
from .dataset import AsyncDataset, MappedAsyncDataset
from .mixture import MixtureDataset, StopStrategy
from .sharded_datasource import ShardedDataSource, UrlBackedShardedDataSource, WrappedHFDataSource, _open_text
from ..compat.hf_checkpoints import load_tokenizer
from .text import BatchTokenizer

logger = logging.getLogger(__name__)


# ------------------------------------------------------------------------------------------------ feature extraction
def _hz_to_mel(f):
    f = np.asarray(f, dtype=np.float64)
    lin = f / (200.0 / 3)
    log_region = f >= 1000.0
    return np.where(log_region, 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0), lin)


def _mel_to_hz(m):
    m = np.asarray(m, dtype=np.float64)
    lin = m * (200.0 / 3)
    return np.where(m >= 15.0, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), lin)


def mel_filter_bank(n_freqs: int, n_mels: int, sampling_rate: int, f_min: float = 0.0, f_max: Optional[float] = None) -> np.ndarray:
    """Slaney-style triangular mel filters with area normalisation, ``[n_freqs, n_mels]``."""
    f_max = f_max if f_max is not None else sampling_rate / 2.0
    fft_freqs = np.linspace(0, sampling_rate / 2.0, n_freqs)
    mel_pts = _mel_to_hz(np.linspace(_hz_to_mel(f_min), _hz_to_mel(f_max), n_mels + 2))
    fdiff = np.diff(mel_pts)
    ramps = mel_pts[None, :] - fft_freqs[:, None]
    lower = -ramps[:, :-2] / fdiff[:-1]
    upper = ramps[:, 2:] / fdiff[1:]
    fb = np.maximum(0.0, np.minimum(lower, upper))
    fb *= (2.0 / (mel_pts[2:n_mels + 2] - mel_pts[:n_mels]))[None, :]
    return fb.astype(np.float32)


@dataclass
class LogMelFeatureExtractor:
    """Whisper's front end.  ``__call__(waveforms, sampling_rate)`` -> ``{"input_features": float32[n, n_mels, frames]}``."""

    feature_size: int = 80
    sampling_rate: int = 16000
    hop_length: int = 160
    chunk_length: int = 30
    n_fft: int = 400
    padding_value: float = 0.0

    def __post_init__(self):
        self.n_samples = self.chunk_length * self.sampling_rate
        self.nb_max_frames = self.n_samples // self.hop_length
        self._filters = torch.from_numpy(mel_filter_bank(1 + self.n_fft // 2, self.feature_size, self.sampling_rate, 0.0, 8000.0))

    def to_dict(self) -> Dict[str, Any]:
        return dict(feature_extractor_type="LogMelFeatureExtractor", feature_size=self.feature_size, sampling_rate=self.sampling_rate,
                    hop_length=self.hop_length, chunk_length=self.chunk_length, n_fft=self.n_fft, padding_value=self.padding_value)

    def log_mel(self, wave_batch: torch.Tensor) -> torch.Tensor:
        """``[n, n_samples]`` float waveform -> ``[n, n_mels, frames]`` (runs on the tensor's device)."""
        window = torch.hann_window(self.n_fft, periodic=True, device=wave_batch.device)
        stft = torch.stft(wave_batch.float(), self.n_fft, self.hop_length, window=window, return_complex=True, center=True, pad_mode="reflect")
        power = stft[..., :-1].abs() ** 2
        mel = torch.matmul(self._filters.to(power.device).T, power)
        log_spec = torch.clamp(mel, min=1e-10).log10()
        log_spec = torch.maximum(log_spec, log_spec.amax(dim=(-2, -1), keepdim=True) - 8.0)
        return (log_spec + 4.0) / 4.0

    def __call__(self, raw_speech, sampling_rate: Optional[int] = None, return_tensors: Optional[str] = "np", **_) -> Dict[str, Any]:
        if sampling_rate is not None and sampling_rate != self.sampling_rate:
            raise ValueError(f"this extractor expects audio sampled at {self.sampling_rate} Hz, got {sampling_rate}")
        if isinstance(raw_speech, (np.ndarray, torch.Tensor)) and np.ndim(raw_speech) == 1:
            raw_speech = [raw_speech]
        batch = torch.full((len(raw_speech), self.n_samples), self.padding_value, dtype=torch.float32)
        for i, w in enumerate(raw_speech):
            w = torch.as_tensor(np.asarray(w), dtype=torch.float32)[: self.n_samples]
            batch[i, : w.numel()] = w
        feats = self.log_mel(batch)
        return {"input_features": feats.numpy() if return_tensors == "np" else feats}


def load_feature_extractor(name_or_obj=None):
    """A Hugging Face processor/feature extractor by name when it can be loaded, else the built-in log-mel front end."""
    if name_or_obj is None:
        return LogMelFeatureExtractor()
    if not isinstance(name_or_obj, str):
        return name_or_obj
    try:
        from transformers import AutoFeatureExtractor

        return AutoFeatureExtractor.from_pretrained(name_or_obj)
    except Exception as e:  # noqa: BLE001  (offline, unknown name, ...)
        logger.warning("could not load feature extractor %r (%s); using the built-in Whisper log-mel front end", name_or_obj, e)
        return LogMelFeatureExtractor()


# ------------------------------------------------------------------------------------------------ batch processor
class BatchAudioProcessor(BatchProcessor[Tuple[np.ndarray, int, str], dict]):
    """``(waveform, sampling_rate, text)`` -> ``{input_features f32[n_mels, frames], input_ids i32[max_length],
    attention_mask i32[max_length]}``; one sampling rate per batch (src/levanter/data/audio.py:71-148)."""

    def __init__(self, processor, tokenizer, enforce_bos=True, enforce_eos=True, *, batch_size=128, override_resources=None,
                 max_length=448, padding="max_length"):
        self.feature_extractor = getattr(processor, "feature_extractor", processor)
        if tokenizer.pad_token_id is None and getattr(tokenizer, "eos_token", None) is not None:
            tokenizer.pad_token = tokenizer.eos_token
        self.bt = BatchTokenizer(tokenizer, enforce_bos=enforce_bos, enforce_eos=enforce_eos, override_resources=override_resources,
                                 return_attention_mask=True, padding=padding, max_length=max_length)
        self.override_resources = override_resources
        self._batch_size = batch_size
        self.max_length = max_length

    def __call__(self, batch: Sequence[Tuple[np.ndarray, int, str]]) -> List[dict]:
        audio, rates, texts = zip(*batch)
        rates = set(rates)
        assert len(rates) == 1, "Sampling rates should be standardized"
        feats = self.feature_extractor(list(audio), sampling_rate=rates.pop(), return_tensors="np")["input_features"]
        toks = self.bt([{"text": t} for t in texts])
        out = []
        for f, t in zip(feats, toks):
            ids = np.asarray(t["input_ids"], dtype=np.int32)[: self.max_length]
            am = np.asarray(t.get("attention_mask", np.ones_like(ids)), dtype=np.int32)[: self.max_length]
            out.append({"input_features": np.asarray(f, dtype=np.float32), "input_ids": ids, "attention_mask": am})
        return out

    @property
    def output_exemplar(self):
        fe = self.feature_extractor
        frames = getattr(fe, "nb_max_frames", 3000)
        return {"input_features": np.zeros((getattr(fe, "feature_size", 80), frames), dtype=np.float32),
                "input_ids": np.zeros((self.max_length,), dtype=np.int32), "attention_mask": np.zeros((self.max_length,), dtype=np.int32)}

    @property
    def num_cpus(self) -> float:
        return self.override_resources.get("num_cpus", self.bt.num_cpus) if self.override_resources else self.bt.num_cpus

    @property
    def num_gpus(self) -> int:
        return self.override_resources.get("num_gpus", 0) if self.override_resources else 0

    @property
    def batch_size(self) -> int:
        return self._batch_size

    @property
    def metadata(self) -> Dict[str, Any]:
        fe = self.feature_extractor.to_dict() if hasattr(self.feature_extractor, "to_dict") else {"extractor": type(self.feature_extractor).__name__}
        return {"tokenizer": self.bt.metadata, "processor": json.loads(json.dumps(fe, default=str))}


# ------------------------------------------------------------------------------------------------ sources
def _read_audio_file(path: str) -> Tuple[np.ndarray, int]:
    """``.npy`` (float waveform, 16 kHz assumed unless a ``.rate`` file sits beside it) or PCM ``.wav``."""
    if path.endswith(".npy"):
        rate_file = path[:-4] + ".rate"
        rate = int(open(rate_file).read()) if os.path.exists(rate_file) else 16000
        return np.load(path).astype(np.float32), rate
    with wave.open(path, "rb") as w:
        n, width, rate, ch = w.getnframes(), w.getsampwidth(), w.getframerate(), w.getnchannels()
        raw = w.readframes(n)
    if width == 2:
        x = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
    elif width == 4:
        x = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
    elif width == 1:
        x = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    else:
        raise ValueError(f"unsupported sample width {width} in {path}")
    if ch > 1:
        x = x.reshape(-1, ch).mean(axis=1)
    return x, rate


def _resample_linear(x: np.ndarray, src: int, dst: int) -> np.ndarray:
    if src == dst:
        return x
    n = int(round(len(x) * dst / src))
    return np.interp(np.linspace(0, len(x) - 1, n), np.arange(len(x)), x).astype(np.float32)


def _resolve_audio(pointer, sampling_rate: int) -> Tuple[np.ndarray, int]:
    """An audio column value: ``{"array", "sampling_rate"}``, ``{"path"}``, a path string or a bare array."""
    if isinstance(pointer, Mapping):
        if pointer.get("array") is not None:
            x, sr = np.asarray(pointer["array"], dtype=np.float32), int(pointer.get("sampling_rate", sampling_rate))
        else:
            x, sr = _read_audio_file(pointer["path"])
    elif isinstance(pointer, str):
        x, sr = _read_audio_file(pointer)
    else:
        x, sr = np.asarray(pointer, dtype=np.float32), sampling_rate
    return _resample_linear(x, sr, sampling_rate), sampling_rate


class AudioTextUrlDataSource(UrlBackedShardedDataSource[Tuple[np.ndarray, int, str]]):
    """jsonl shards whose rows hold an audio pointer (see :func:`_resolve_audio`) and a transcript."""

    def __init__(self, urls, text_key="sentence", audio_key="audio", sampling_rate=16000):
        super().__init__(urls)
        self.text_key, self.audio_key, self.sampling_rate = text_key, audio_key, sampling_rate

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[Tuple[np.ndarray, int, str]]:
        url = self._shard_name_to_url_mapping[shard_name]
        with _open_text(url) as f:
            for i, line in enumerate(f):
                if i < row or not line.strip():
                    continue
                d = json.loads(line)
                x, sr = _resolve_audio(d[self.audio_key], self.sampling_rate)
                yield x, sr, d[self.text_key]


@dataclass(frozen=True)
class AudioDatasetSourceConfig:
    """Where the audio comes from: a hub dataset (``id``) or lists of jsonl urls (src/levanter/data/audio.py:151-224)."""

    id: Optional[str] = None
    name: Optional[str] = None
    stream: bool = True
    text_key: str = "sentence"
    audio_key: str = "audio"
    sampling_rate: int = 16000
    train_split: str = "train"
    validation_split: str = "validation"
    train_urls: List[str] = field(default_factory=list)
    validation_urls: List[str] = field(default_factory=list)
    cache_dir: str = "cache/"

    def get_shard_source(self, split: str) -> Optional[ShardedDataSource]:
        if self.id is not None:
            hf_split = self.train_split if split == "train" else self.validation_split if split == "validation" else split
            try:
                ds = WrappedHFDataSource(self.id, split=hf_split, name=self.name, streaming=self.stream)
            except Exception as e:  # noqa: BLE001
                logger.warning("could not open %s split %s: %s", self.id, hf_split, e)
                return None
            sr, ak, tk = self.sampling_rate, self.audio_key, self.text_key
            return ds.map(lambda d: (*_resolve_audio(d[ak], sr), d[tk]))
        urls = self.urls_for_split(split)
        if not urls:
            return None
        return AudioTextUrlDataSource(urls, self.text_key, self.audio_key, self.sampling_rate)

    def urls_for_split(self, split: str) -> List[str]:
        urls = self.train_urls if split == "train" else self.validation_urls if split == "validation" else None
        if urls is None:
            raise ValueError(f"Unknown split {split}")
        return [g for u in urls for g in expand_glob(u)]

    def doc_iterator(self, split: str):
        src = self.get_shard_source(split)
        if src is None:
            return iter(())
        return iter(src)


@dataclass(frozen=True)
class AudioTaskConfig:
    processor: str = "openai/whisper-tiny"
    """a Hugging Face processor name/path, or "builtin" for this module's own log-mel front end"""
    tokenizer: Optional[str] = None
    """defaults to the processor's tokenizer; "passthrough" reads transcripts as whitespace-separated ids"""
    vocab_size: Optional[int] = None  # only for the passthrough tokenizer
    enforce_bos: bool = True
    enforce_eos: bool = True
    max_length: int = 448
    cache_options: CacheOptions = field(default_factory=CacheOptions)

    @cached_property
    def the_processor(self):
        return load_feature_extractor(None if self.processor == "builtin" else self.processor)

    @property
    def the_feature_extractor(self):
        p = self.the_processor
        return getattr(p, "feature_extractor", p)

    @cached_property
    def the_tokenizer(self):
        name = self.tokenizer if self.tokenizer is not None else self.processor
        if name == "passthrough":
            from .passthrough_tokenizer import PassthroughTokenizer

            return PassthroughTokenizer(self.vocab_size or 51865, pad_token_id=0)
        return load_tokenizer(name)

    @property
    def pad_token_id(self) -> int:
        tok = self.the_tokenizer
        return tok.pad_token_id if tok.pad_token_id is not None else tok.eos_token_id


class ProcessedAudioCache(AsyncDataset[dict]):
    """A :class:`TreeCache` of processed rows (src/levanter/data/audio.py:271-356)."""

    def __init__(self, cache: TreeCache):
        super().__init__()
        self.cache = cache

    async def async_len(self) -> int:
        return await self.cache.async_len()

    async def final_length_is_known(self) -> bool:
        return await self.cache.final_length_is_known()

    def is_finite(self) -> bool:
        return True

    async def current_len(self) -> Optional[int]:
        return await self.cache.current_len()

    async def get_batch(self, indices: Sequence[int]) -> Sequence[dict]:
        return await self.cache.get_batch(indices)

    @staticmethod
    def build_or_load(cache_dir: str, source: ShardedDataSource, processor, tokenizer, enforce_bos=True, enforce_eos=True,
                      monitors=None, await_finished=True, override_resources=None, max_length=448,
                      cache_options: Optional[CacheOptions] = None) -> "ProcessedAudioCache":
        bp = BatchAudioProcessor(processor, tokenizer, enforce_bos, enforce_eos, override_resources=override_resources, max_length=max_length)
        cache = build_or_load_cache(cache_dir, source, bp, await_finished=await_finished, monitors=monitors, options=cache_options)
        return ProcessedAudioCache(cache)

    @staticmethod
    def load(cache_dir: str, exemplar=None) -> "ProcessedAudioCache":
        if exemplar is None:
            exemplar = {"input_features": np.zeros((0, 0), dtype=np.float32), "input_ids": np.zeros((0,), dtype=np.int32),
                        "attention_mask": np.zeros((0,), dtype=np.int32)}
        return ProcessedAudioCache(TreeCache.load(cache_dir, exemplar))


class AudioTextDataset(MappedAsyncDataset):
    """Cache rows -> :class:`AudioTextExample` (src/levanter/data/audio.py:446-473)."""

    def __init__(self, dataset: AsyncDataset, ignore_index: Optional[int] = None):
        def to_example(row) -> AudioTextExample:
            tokens = torch.from_numpy(np.asarray(row["input_ids"]).astype(np.int64))
            audio = torch.from_numpy(np.asarray(row["input_features"], dtype=np.float32))
            return AudioTextExample.init(audio, tokens, ignore_id=ignore_index)

        super().__init__(dataset, to_example)
        self.ignore_index = ignore_index


@dataclass(frozen=True)
class AudioIODatasetConfig(AudioDatasetSourceConfig, AudioTaskConfig):
    """One audio dataset with its processing (src/levanter/data/audio.py:359-443)."""

    def train_set(self, monitors=True, *, key=None, **_) -> Optional[AsyncDataset]:
        return self.build_or_load_cache("train", monitors=monitors)

    def validation_set(self, monitors=True) -> Optional[AsyncDataset]:
        return self.build_or_load_cache("validation", monitors=monitors)

    def validation_sets(self, monitors=True) -> Mapping[str, AsyncDataset]:
        v = self.validation_set(monitors)
        return {"": v} if v is not None else {}

    def build_or_load_cache(self, split: str, monitors=True) -> Optional[ProcessedAudioCache]:
        kind = split
        split_cache_dir = os.path.join(self.cache_dir, kind)
        try:
            return ProcessedAudioCache.load(split_cache_dir, BatchAudioProcessor(self.the_processor, self.the_tokenizer,
                                                                                 max_length=self.max_length).output_exemplar)
        except FileNotFoundError:
            pass
        source = self.get_shard_source(kind)
        if source is None:
            logger.info("No data for %s", kind)
            return None
        logger.info("Building cache for %s...", kind)
        # validation caches are awaited, training caches are read while they are being built
        return ProcessedAudioCache.build_or_load(split_cache_dir, source, self.the_processor, self.the_tokenizer, self.enforce_bos,
                                                 self.enforce_eos, monitors=monitors if isinstance(monitors, list) else None,
                                                 await_finished=(kind == "validation"), max_length=self.max_length,
                                                 cache_options=self.cache_options)


@dataclass(frozen=True)
class AudioMixtureDatasetConfig(AudioTaskConfig):
    """A weighted mixture of audio datasets (src/levanter/data/audio.py:486-620)."""

    cache_dir: Optional[str] = "cache/"
    configs: Dict[str, AudioDatasetSourceConfig] = field(default_factory=dict)
    train_weights: Dict[str, float] = field(default_factory=dict)
    stop_strategy: str = field(default=StopStrategy.RESTART_STRATEGY)
    mixture_block_size: int = 2048
    shuffle: Union[bool, int] = False

    def __post_init__(self):
        if len(self.configs) == 0:
            raise ValueError("At least one dataset must be provided")
        if set(self.configs.keys()) != set(self.train_weights.keys()):
            raise ValueError(f"The keys in configs and weights must be the same; got {self.configs.keys()} and {self.train_weights.keys()}")

    def build_caches(self, split: str, monitors=True) -> Dict[str, ProcessedAudioCache]:
        caches = {}
        for name, src_cfg in self.configs.items():
            if split == "train" and self.train_weights.get(name, 0) == 0:
                continue
            cache_dir = src_cfg.cache_dir if self.cache_dir is None else os.path.join(self.cache_dir, name)
            source = src_cfg.get_shard_source(split)
            split_dir = os.path.join(cache_dir, split)
            if source is None:
                try:
                    caches[name] = ProcessedAudioCache.load(split_dir)
                except FileNotFoundError:
                    logger.warning("Skipping %s for split %s because no source was provided", name, split)
                continue
            caches[name] = ProcessedAudioCache.build_or_load(split_dir, source, self.the_processor, self.the_tokenizer, self.enforce_bos,
                                                             self.enforce_eos, await_finished=(split == "validation"),
                                                             max_length=self.max_length, cache_options=self.cache_options)
        return caches

    def train_set(self, monitors=True, *, key=0, **_) -> AsyncDataset:
        caches = self.build_caches("train", monitors)
        datasets: Dict[str, AsyncDataset] = dict(caches)
        if self.shuffle is True:
            datasets = {n: d.shuffle(key + i) for i, (n, d) in enumerate(datasets.items())}
        elif isinstance(self.shuffle, int) and not isinstance(self.shuffle, bool) and self.shuffle > 0:
            datasets = {n: d.era_shuffle(self.shuffle, key=key + i) for i, (n, d) in enumerate(datasets.items())}
        return MixtureDataset(datasets=datasets, weights={k: v for k, v in self.train_weights.items() if k in datasets},
                              stop_strategy=self.stop_strategy, key=key, block_size=self.mixture_block_size)

    def validation_sets(self, monitors=True) -> Mapping[str, AsyncDataset]:
        return self.build_caches("validation", monitors)
