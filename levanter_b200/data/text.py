"""Text data for language modelling (src/levanter/data/text.py): tokenisation processors, the token cache views
(``TokenSeqDataset`` / ``CausalLmDataset``), chat and supervised formats with packing, and the dataset configs
(``LMTaskConfig``, single-source and mixture) that ``train_lm`` consumes.

Examples are produced on the host as CPU ``torch`` tensors; the loader stacks them into pinned buffers and the trainer
copies a step's batch to the GPU on a side stream."""
from __future__ import annotations

import abc
import dataclasses
import logging
import os
import re
from dataclasses import dataclass, field
from functools import cached_property
from itertools import chain
from typing import Any, Dict, Iterator, List, Literal, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..config import ChoiceRegistry
from ..models.lm_model import LmExample
from ..schedule import BatchSchedule
from ..store.cache import CacheMetadata, CacheOptions, TreeCache, build_or_load_cache
from ..store.jagged_array import JaggedArrayStore
from ..utils import fsspec_utils
from ..utils.hf_utils import num_cpus_used_by_tokenizer
from ._preprocessor import BatchProcessor
from .dataset import AsyncDataset, EpochDataset, MappedAsyncDataset, _fold_in
from .metrics_monitor import LoggerMetricsMonitor, LoggingMetricsMonitor, MetricsMonitor
from .mixture import MixtureDataset, StopStrategy, rescale_mixture_schedule_for_batch_schedule
from .packing import GreedyPrepackedDataset
from .passthrough_tokenizer import PassthroughTokenizer
from .sharded_datasource import JsonlDataSource, ShardedDataSource, UrlDataSource, WrappedHFDataSource

logger = logging.getLogger("levanter_b200.data.text")

LONG_STRING_WORKAROUND = 10_000
ws = re.compile(r"\s")
CANONICAL_INPUT_FIELD = "prompt"
CANONICAL_OUTPUT_FIELD = "response"
DEFAULT_IGNORE_INDEX = -100  # PyTorch's default ignore index


def _seq_len(Pos) -> int:
    return int(getattr(Pos, "size", Pos))


class TokenSeqDataset(AsyncDataset[np.ndarray]):
    """Fixed-length windows over the concatenation of all cached documents: item ``i`` is tokens
    ``[i * seq_len, (i + 1) * seq_len)`` of the flat ``input_ids`` array, whatever document boundaries fall inside."""

    def __init__(self, doc_cache: TreeCache, seq_len: int):
        super().__init__()
        self.doc_cache = doc_cache
        self.seq_len = seq_len
        self._cached_len: Optional[int] = None

    def _tokens(self) -> JaggedArrayStore:
        store = self.doc_cache._store_for_read() if not self.doc_cache.is_finished else self.doc_cache.store
        return store.tree[("input_ids",)]

    async def async_len(self) -> int:
        await self.doc_cache.finished()
        return self._tokens().data_size // self.seq_len

    async def final_length_is_known(self) -> bool:
        return await self.doc_cache.final_length_is_known()

    def is_finite(self) -> bool:
        return True

    async def current_len(self) -> Optional[int]:
        if not self.doc_cache.is_finished and await self.doc_cache.current_len() == 0:
            return 0
        return self._tokens().data_size // self.seq_len

    async def get_batch(self, indices: Sequence[int]) -> Sequence[np.ndarray]:
        if not len(indices):
            return []
        need = max(indices) + 1
        n = await self.wait_until_len_at_least(need)
        if n < need:
            raise ValueError("Requested indices beyond the end of the dataset")
        data = self._tokens().data
        return [data.read([int(i) * self.seq_len], [(int(i) + 1) * self.seq_len]) for i in indices]

    async def wait_until_len_at_least(self, length: int) -> int:
        if self._cached_len is not None and self._cached_len >= length:
            return self._cached_len
        n = await super().wait_until_len_at_least(length)
        self._cached_len = n
        return n


class CausalLmDataset(MappedAsyncDataset):
    """Token windows -> :class:`LmExample` (next-token loss mask; attention segments split at EOS when ``eos_id`` is set)."""

    def __init__(self, dataset: AsyncDataset, Pos, *, ignore_index: Optional[int] = None, eos_id: Optional[int] = None):
        self.Pos = Pos
        self.ignore_id = ignore_index
        self.eos_id = eos_id

        def _create_lm_example(tokens):
            t = torch.from_numpy(np.ascontiguousarray(tokens).astype(np.int32, copy=False))
            return LmExample.causal(tokens=t, ignore_id=self.ignore_id, eos_id=self.eos_id)

        super().__init__(dataset, _create_lm_example)

    async def async_len(self) -> int:
        return await self.dataset.async_len()


def _maybe_force_tokenizer_parallelism(tokenizer) -> None:
    if getattr(tokenizer, "is_fast", False) and os.getenv("TOKENIZERS_PARALLELISM") is None:
        os.environ["TOKENIZERS_PARALLELISM"] = "true"


class BatchTokenizer(BatchProcessor[dict, dict]):
    """Tokenises ``text_field`` of each row.  BOS/EOS are added when the tokenizer does not add them itself (probed on a
    short string).  Very long strings are cut at whitespace into pieces of at most ``_workaround_len`` characters and the
    encodings concatenated, because some fast tokenizers with ``Replace`` normalisers are quadratic in the string length."""

    def __init__(self, tokenizer, text_field="text", enforce_bos=True, enforce_eos=True, *, override_resources=None,
                 _workaround_len=LONG_STRING_WORKAROUND, return_attention_mask=False, padding=False, max_length=None):
        _maybe_force_tokenizer_parallelism(tokenizer)
        self.tokenizer = tokenizer
        self.text_field = text_field
        self.override_resources = override_resources
        self.return_attention_mask = return_attention_mask
        self.padding = padding
        self.max_length = max_length if max_length is not None else getattr(tokenizer, "model_max_length", None)
        if tokenizer.bos_token_id is None:
            enforce_bos = False
        if tokenizer.eos_token_id is None:
            enforce_eos = False
        if enforce_eos or enforce_bos:
            probe = tokenizer("1 2" if isinstance(tokenizer, PassthroughTokenizer) else "hi there")["input_ids"]
            self._need_to_add_eos = bool(enforce_eos and probe[-1] != tokenizer.eos_token_id)
            self._need_to_add_bos = bool(enforce_bos and probe[0] != tokenizer.bos_token_id)
        else:
            self._need_to_add_eos = self._need_to_add_bos = False
        self._workaround_len = _workaround_len

    def __call__(self, batch: Sequence[dict]) -> List[dict]:
        texts = [ex[self.text_field] for ex in batch]
        if self._need_to_add_bos:
            texts = [self.tokenizer.bos_token + " " + d for d in texts]
        if self._need_to_add_eos:
            texts = [d + " " + self.tokenizer.eos_token for d in texts]
        needs_merge: List[bool] = []
        if self._needs_long_sequence_workaround:
            texts, needs_merge = self._break_for_long_sequences(texts)
        if self.padding is not False:
            enc = self.tokenizer(texts, return_attention_mask=self.return_attention_mask, verbose=False, padding=self.padding,
                                 max_length=self.max_length, truncation=True)
        else:
            enc = self.tokenizer(texts, return_attention_mask=self.return_attention_mask, verbose=False)
        enc = {k: enc[k] for k in enc.keys()}
        if any(needs_merge):
            enc = self._merge_split_encodings(texts, enc, needs_merge)
        keys = list(enc.keys())
        return [{k: np.asarray(v, dtype=np.int32) for k, v in zip(keys, vals)} for vals in zip(*[enc[k] for k in keys])]

    def _break_for_long_sequences(self, batch: List[str]) -> Tuple[List[str], List[bool]]:
        out, needs_merge = [], []
        for d in batch:
            while len(d) > self._workaround_len:
                m = ws.search(d, self._workaround_len)
                split = len(d) if m is None else m.start()
                out.append(d[:split])
                needs_merge.append(True)  # this piece continues into the next
                d = d[split:]
            out.append(d)
            needs_merge.append(False)
        return out, needs_merge

    @staticmethod
    def _merge_split_encodings(batch, encoding, needs_merge) -> Dict[str, list]:
        merged: Dict[str, list] = {}
        for k, v in encoding.items():
            if len(v) == 0:
                continue
            out, pending = [], []
            for i in range(len(batch)):
                pending.append(list(v[i]))
                if not needs_merge[i]:
                    out.append(list(chain(*pending)))
                    pending = []
            if pending:
                out.append(list(chain(*pending)))
            merged[k] = out
        return merged

    @property
    def metadata(self) -> Dict[str, Any]:
        return {"tokenizer": self.tokenizer.name_or_path, "vocab_size": len(self.tokenizer),
                "return_attention_mask": self.return_attention_mask, "padding": self.padding, "max_length": self.max_length,
                "append_bos": self._need_to_add_bos, "append_eos": self._need_to_add_eos}

    @property
    def output_exemplar(self) -> dict:
        keys = ["input_ids"] + (["attention_mask"] if self.return_attention_mask else [])
        if not isinstance(self.tokenizer, PassthroughTokenizer):
            keys = list(self.tokenizer("hi there", return_attention_mask=self.return_attention_mask, verbose=False).keys())
        return {k: np.zeros((0,), dtype=np.int32) for k in keys}

    @property
    def name_or_path(self):
        return self.tokenizer.name_or_path

    @property
    def vocab_size(self):
        return self.tokenizer.vocab_size

    @cached_property
    def _needs_long_sequence_workaround(self) -> bool:
        backend = getattr(self.tokenizer, "backend_tokenizer", None)
        if backend is None:
            return False
        normalizer = getattr(backend, "normalizer", None)
        if normalizer is None:
            return False
        return type(normalizer).__name__ in ("Replace", "Sequence")

    @property
    def num_cpus(self) -> int:
        if self.override_resources is not None and self.override_resources.get("num_cpus") is not None:
            return self.override_resources["num_cpus"]
        return num_cpus_used_by_tokenizer(self.tokenizer)

    @property
    def num_gpus(self) -> int:
        return 0 if self.override_resources is None else self.override_resources.get("num_gpus", 0)


# ------------------------------------------------------------------------------------------------------ formats
class LmDatasetFormatBase(abc.ABC, ChoiceRegistry):
    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return "text"


@LmDatasetFormatBase.register_subclass("text")
@dataclass(frozen=True)
class TextLmDatasetFormat(LmDatasetFormatBase):
    text_key: str = "text"


@LmDatasetFormatBase.register_subclass("chat")
@dataclass(frozen=True)
class ChatLmDatasetFormat(LmDatasetFormatBase):
    messages_field: str = "messages"
    single_turn: bool = False
    chat_template: Optional[str] = None
    pack: bool = True
    mask_user_turns: bool = True


@LmDatasetFormatBase.register_subclass("supervised")
@dataclass(frozen=True)
class SupervisedLmDatasetFormat(LmDatasetFormatBase):
    input_field: str = CANONICAL_INPUT_FIELD
    output_field: str = CANONICAL_OUTPUT_FIELD
    separate_with: Union[str, int, None] = None
    pack: bool = True
    mask_inputs: bool = True


# ------------------------------------------------------------------------------------------------------ sources
@dataclass(frozen=True)
class LmDatasetSourceConfigBase(abc.ABC):
    """One dataset: where the raw rows come from, their format, optional tags and a cache-dir override."""
    tags: Optional[List[str]] = None
    cache_dir: Optional[str] = None
    format: LmDatasetFormatBase = field(default_factory=TextLmDatasetFormat)

    @abc.abstractmethod
    def get_shard_source(self, split) -> Optional[ShardedDataSource[dict]]:
        raise NotImplementedError

    def load_cache(self, split, tokenizer, override_cache_dir: Optional[str] = None, enforce_eos=True) -> TreeCache:
        base = override_cache_dir if override_cache_dir is not None else self.cache_dir
        if base is None:
            raise ValueError("cache_dir must be set or override_cache_dir must be provided")
        return load_lm_dataset_cache(os.path.join(base, split), self.format, tokenizer, enforce_eos=enforce_eos)


@dataclass(frozen=True)
class HfDatasetSourceConfig(LmDatasetSourceConfigBase):
    id: str = dataclasses.field(kw_only=True, default=None)  # type: ignore
    name: Optional[str] = None
    stream: bool = True

    def get_shard_source(self, split) -> Optional[ShardedDataSource[dict]]:
        if self.id is None:
            return None
        try:
            ds = WrappedHFDataSource(self.id, split=split, name=self.name, streaming=self.stream)
            if len(ds.shard_names) == 0:
                return None
        except ValueError as e:
            if str(e).startswith("Bad split"):
                logger.warning(f"Splits {split} not found for {self.id} {self.name}")
                return None
            raise
        return ds


@dataclass(frozen=True)
class UrlDatasetSourceConfig(LmDatasetSourceConfigBase):
    train_urls: List[str] = ()  # type: ignore
    validation_urls: List[str] = ()  # type: ignore

    def get_shard_source(self, split) -> Optional[ShardedDataSource[dict]]:
        urls = self.urls_for_split(split)
        if len(urls) == 0:
            return None
        return UrlDataSource(urls)

    def urls_for_split(self, split):
        if split == "train":
            return list(self.train_urls)
        if split == "validation":
            return list(self.validation_urls)
        raise ValueError(f"Unknown split {split}")


# --------------------------------------------------------------------------------------------------- processors
class ChatProcessor(BatchProcessor[dict, dict]):
    """Applies a chat template; emits ``input_ids`` and ``assistant_masks`` (1 on assistant tokens, from the template's
    ``{% generation %}`` blocks)."""

    def __init__(self, tokenizer, chat_template: Optional[str] = None, messages_field: str = "messages", mask_user_turns: bool = True):
        self.tokenizer = tokenizer
        self.chat_template = chat_template or getattr(tokenizer, "chat_template", None)
        self.messages_field = messages_field
        if self.chat_template is None:
            raise ValueError("No chat template provided and tokenizer has no default chat template")
        if mask_user_turns and not re.search(r"\{%-?\s*generation\s*-?%}", self.chat_template):
            raise ValueError("Chat template must contain {%generation%} to indicate the position of the assistant message "
                             f"if mask_user_turns is True. However, the provided template does not contain this tag: ```{self.chat_template}```.")

    def __call__(self, batch: Sequence[dict]) -> Sequence[dict]:
        messages = [ex[self.messages_field] for ex in batch]
        tok = self.tokenizer.apply_chat_template(messages, tokenize=True, chat_template=self.chat_template,
                                                 return_assistant_tokens_mask=True, return_dict=True)
        masks = tok["assistant_masks"]
        out = []
        for ex, ids, mask in zip(batch, tok["input_ids"], masks):
            if not np.any(mask):
                raise ValueError(f"Chat did not contain an assistant message for sequence {ex}")
            out.append({"input_ids": np.array(ids, dtype=np.int32), "assistant_masks": np.array(mask, dtype=np.int32)})
        return out

    @property
    def output_exemplar(self):
        return {"input_ids": np.zeros((0,), dtype=np.int32), "assistant_masks": np.zeros((0,), dtype=np.int32)}

    @property
    def num_cpus(self) -> int:
        return num_cpus_used_by_tokenizer(self.tokenizer)

    @property
    def metadata(self) -> Dict[str, Any]:
        return {"tokenizer": self.tokenizer.name_or_path, "vocab_size": len(self.tokenizer), "chat_template": self.chat_template,
                "messages_field": self.messages_field}


class SupervisedProcessor(BatchProcessor[dict, dict]):
    """``input + output`` tokenised together; ``sources_len`` = token count of the input alone (for masking the prompt)."""

    def __init__(self, tokenizer, input_field: str, output_field: str, separate_with: Union[str, int, None] = None):
        self.tokenizer = tokenizer
        self.input_field, self.output_field = input_field, output_field
        if isinstance(separate_with, int):
            separate_with = tokenizer.convert_ids_to_tokens(separate_with)
        self.separate_with = separate_with

    def __call__(self, batch: Sequence[dict]) -> Dict[str, Any]:
        sources = [ex[self.input_field] for ex in batch]
        targets = [ex[self.output_field] for ex in batch]
        if self.separate_with is not None:
            sources = [s + self.separate_with for s in sources]
        examples = [s + t for s, t in zip(sources, targets)]
        src_tok = self.tokenizer(sources, padding=False, truncation=True)
        ex_tok = self.tokenizer(examples, padding=False, truncation=True)
        return {"input_ids": [np.array(e, dtype=np.int32) for e in ex_tok["input_ids"]],
                "sources_len": np.array([len(s) for s in src_tok["input_ids"]], dtype=np.int32)}

    @property
    def output_exemplar(self):
        return {"input_ids": np.zeros((0,), dtype=np.int32), "sources_len": np.zeros((0,), dtype=np.int32)}

    @property
    def num_cpus(self) -> int:
        return num_cpus_used_by_tokenizer(self.tokenizer)

    @property
    def metadata(self) -> Dict[str, Any]:
        return {"tokenizer": self.tokenizer.name_or_path, "vocab_size": len(self.tokenizer), "input_field": self.input_field,
                "output_field": self.output_field, "separate_with": self.separate_with}


class SingleTurnChatProcessor(BatchProcessor[dict, dict]):
    """First user message -> prompt, first assistant message -> response; later turns are dropped."""

    def __init__(self, tokenizer, messages_field: str = "messages"):
        self.tokenizer = tokenizer
        self.messages_field = messages_field
        self.supervised_processor = SupervisedProcessor(tokenizer, CANONICAL_INPUT_FIELD, CANONICAL_OUTPUT_FIELD)

    def __call__(self, batch: Sequence[dict]):
        convs = [ex[self.messages_field] for ex in batch]
        inp = [next(m["content"] for m in c if m["role"] == "user") for c in convs]
        out = [next(m["content"] for m in c if m["role"] == "assistant") for c in convs]
        return self.supervised_processor([{CANONICAL_INPUT_FIELD: i, CANONICAL_OUTPUT_FIELD: o} for i, o in zip(inp, out)])

    @property
    def output_exemplar(self):
        return self.supervised_processor.output_exemplar

    @property
    def num_cpus(self) -> int:
        return self.supervised_processor.num_cpus

    @property
    def metadata(self) -> Dict[str, Any]:
        return {**self.supervised_processor.metadata, "tokenizer": self.tokenizer.name_or_path,
                "vocab_size": len(self.tokenizer), "messages_field": self.messages_field}


def preprocessor_for_format(format: LmDatasetFormatBase, tokenizer, *, enforce_eos: bool = True, enforce_bos: bool = True) -> BatchProcessor:
    if isinstance(format, TextLmDatasetFormat):
        return BatchTokenizer(tokenizer, enforce_bos=enforce_bos, enforce_eos=enforce_eos, text_field=format.text_key)
    if isinstance(format, ChatLmDatasetFormat):
        if format.single_turn:
            if format.chat_template is not None:
                raise NotImplementedError("Don't currently support chat templates for single turn chat")
            return SingleTurnChatProcessor(tokenizer, messages_field=format.messages_field)
        return ChatProcessor(tokenizer, messages_field=format.messages_field, chat_template=format.chat_template,
                             mask_user_turns=format.mask_user_turns)
    if isinstance(format, SupervisedLmDatasetFormat):
        return SupervisedProcessor(tokenizer, input_field=format.input_field, output_field=format.output_field,
                                   separate_with=format.separate_with)
    raise ValueError(f"Unknown format {format}")


# ------------------------------------------------------------------------------------------- packed datasets
def _named_stores(cache: TreeCache) -> Dict[str, JaggedArrayStore]:
    return {p[0]: s for p, s in cache.store.tree.items()}


class MultiturnChatDataset(MappedAsyncDataset):
    """Packed chat examples: loss on assistant tokens only (the assistant mask rolled back by one, since position ``t``
    predicts token ``t + 1``), segment ids keep conversations apart."""

    def __init__(self, cache: TreeCache, Pos, max_segments_per_example: int = 64, slice_strategy: str = "left", mask_user_turns: bool = True):
        cache.await_finished()
        self.packed = GreedyPrepackedDataset(_named_stores(cache), _seq_len(Pos), max_segments_per_example=max_segments_per_example,
                                             slice_strategy=slice_strategy)
        self.Pos = Pos
        self.mask_user_turns = mask_user_turns

        def _create_lm_example(e) -> LmExample:
            ex, seg = e
            tokens = torch.from_numpy(ex["input_ids"].astype(np.int32))
            lm = torch.from_numpy(np.roll(ex["assistant_masks"], -1, axis=-1).astype(np.int32)) if mask_user_turns else None
            seg_ids = torch.from_numpy(seg["input_ids"].astype(np.int32))
            return LmExample.causal(tokens=tokens, loss_mask=lm, segment_ids=seg_ids)

        super().__init__(self.packed, _create_lm_example)


class SupervisedDataset(MappedAsyncDataset):
    """Packed prompt/response examples; with ``mask_inputs`` the first ``sources_len`` tokens of every segment carry no loss."""

    def __init__(self, cache: TreeCache, Pos, max_segments_per_example: Optional[int] = 64, mask_inputs: bool = True, slice_strategy: str = "right"):
        self.mask_inputs = mask_inputs
        cache.await_finished()
        S = _seq_len(Pos)
        # ``sources_len`` has one element per document, so at most ``max_segments`` of them land in a pack
        max_len = {"input_ids": S, "sources_len": max_segments_per_example or S}
        self.packed = GreedyPrepackedDataset(_named_stores(cache), max_len, max_segments_per_example=max_segments_per_example,
                                             slice_strategy=slice_strategy)

        def _create_lm_example(pair) -> LmExample:
            ex, seg = pair
            tokens = torch.from_numpy(ex["input_ids"].astype(np.int32))
            segment_ids = seg["input_ids"]
            lm = None
            if self.mask_inputs:
                # ``is_response[t]`` marks response *tokens*; the loss at position ``t`` scores token ``t + 1``, so it is on
                # when the next token is a response token of the same segment.  (The reference passes the unshifted mask,
                # src/levanter/data/text.py:1676-1683, which scores the first token of the following segment instead of
                # the first response token.)
                is_resp = self._make_sequence_mask(segment_ids, ex["sources_len"])
                nxt = np.roll(is_resp, -1)
                nxt[-1] = 0
                same = np.roll(segment_ids, -1) == segment_ids
                lm = torch.from_numpy((nxt * same).astype(np.int32))
            return LmExample.causal(tokens, loss_mask=lm, segment_ids=torch.from_numpy(segment_ids.astype(np.int32)))

        super().__init__(self.packed, _create_lm_example)

    @staticmethod
    def _make_sequence_mask(segment_ids: np.ndarray, segment_source_len: np.ndarray) -> np.ndarray:
        """1 where a token belongs to the response part of its segment, 0 on prompt tokens and padding (segment -1).
        ``segment_source_len[j]`` is the prompt length of the j-th distinct segment in order of appearance."""
        segment_ids = np.asarray(segment_ids)
        n = len(segment_ids)
        if n == 0:
            return np.zeros(0, dtype=np.int32)
        starts = np.nonzero(np.concatenate([[True], segment_ids[1:] != segment_ids[:-1]]))[0]
        run_idx = np.cumsum(np.concatenate([[0], (segment_ids[1:] != segment_ids[:-1]).astype(np.int64)]))
        pos_in_seg = np.arange(n) - starts[run_idx]
        src = np.asarray(segment_source_len).reshape(-1)
        src_per_run = np.zeros(len(starts), dtype=np.int64)
        k = min(len(starts), len(src))
        src_per_run[:k] = src[:k]
        mask = (pos_in_seg >= src_per_run[run_idx]).astype(np.int32)
        mask[segment_ids == -1] = 0
        return mask


def dataset_for_format(format: LmDatasetFormatBase, Pos, cache: TreeCache, *, eos_id: Optional[int], ignore_index: Optional[int]) -> AsyncDataset:
    if isinstance(format, TextLmDatasetFormat):
        return CausalLmDataset(TokenSeqDataset(cache, _seq_len(Pos)), Pos, eos_id=eos_id, ignore_index=ignore_index)
    if isinstance(format, ChatLmDatasetFormat):
        if format.single_turn:
            return SupervisedDataset(cache, Pos, max_segments_per_example=64 if format.pack else 1, mask_inputs=format.mask_user_turns)
        return MultiturnChatDataset(cache, Pos, max_segments_per_example=64 if format.pack else 1, mask_user_turns=format.mask_user_turns)
    if isinstance(format, SupervisedLmDatasetFormat):
        return SupervisedDataset(cache, Pos, max_segments_per_example=64 if format.pack else 1, mask_inputs=format.mask_inputs)
    raise ValueError(f"Unknown format {format}")


# ------------------------------------------------------------------------------------------------ cache helpers
def build_lm_dataset_cache(cache_dir: str, source: Optional[ShardedDataSource], format: LmDatasetFormatBase, tokenizer,
                           options: CacheOptions = CacheOptions.default(), enforce_eos=True,
                           monitors: Union[bool, List[MetricsMonitor]] = True) -> Optional[TreeCache]:
    """Load the cache at ``cache_dir`` or start building it (returns at once; readers wait for the rows they need)."""
    name = os.path.join(*cache_dir.rstrip("/").split("/")[-2:])
    processor = preprocessor_for_format(format, tokenizer, enforce_bos=True, enforce_eos=enforce_eos)
    try:
        return TreeCache.load(cache_dir, exemplar=processor.output_exemplar, options=CacheMetadata(preprocessor_metadata=processor.metadata))
    except FileNotFoundError:
        pass
    if source is None:
        logger.info(f"No data for {name}")
        return None
    logger.info(f"Building cache for {name}...")
    if monitors is True:
        monitors = [LoggingMetricsMonitor(prefix=f"preprocessing/{name}", commit=False), LoggerMetricsMonitor(f"preprocessing.{name}")]
    elif monitors is False:
        monitors = []
    return build_or_load_cache(cache_dir, source, processor, monitors=monitors, await_finished=False, options=options)


def load_lm_dataset_cache(cache_dir: str, format: LmDatasetFormatBase, tokenizer, enforce_eos=True) -> TreeCache:
    """Open a finished cache; raises FileNotFoundError when it does not exist."""
    processor = preprocessor_for_format(format, tokenizer, enforce_bos=True, enforce_eos=enforce_eos)
    return TreeCache.load(cache_dir, exemplar=processor.output_exemplar, options=CacheMetadata(preprocessor_metadata=processor.metadata))


def cached_token_count(cache_path: str, field: str = "input_ids") -> int:
    """Total number of tokens in a finished cache (the last entry of the field's offsets array)."""
    cache = TreeCache.load(cache_path, {field: np.zeros((0,), dtype=np.int32)})
    return cache.store.tree[(field,)].data_size


def _split_key(key, n: int) -> List[int]:
    return [_fold_in(key, i) for i in range(n)]


# ------------------------------------------------------------------------------------------------- task configs
@dataclass(frozen=True)
class LMTaskConfig(abc.ABC):
    tokenizer: str = "gpt2"
    vocab_size: Optional[int] = None  # required for the passthrough tokenizer
    cache_dir: Optional[str] = "cache/"
    cache_options: CacheOptions = field(default_factory=CacheOptions)
    enforce_eos: bool = True
    chat_template: Optional[str] = None
    ignore_token_id: Optional[int] = DEFAULT_IGNORE_INDEX
    shuffle: Union[bool, int] = False
    """True: shuffle the whole dataset; an int: shuffle within eras of that many examples; False: keep order."""
    permutation_type: Optional[str] = None  # "feistel" | "linear"; None means linear

    @cached_property
    def the_tokenizer(self):
        if self.tokenizer == "passthrough":
            return PassthroughTokenizer(self.vocab_size)
        from ..compat.hf_checkpoints import load_tokenizer

        return load_tokenizer(self.tokenizer)

    @abc.abstractmethod
    def train_set(self, Pos, batch_schedule: BatchSchedule, monitors=True, *, key, epochs: Optional[int] = None) -> AsyncDataset:
        ...

    @abc.abstractmethod
    def train_sets(self, Pos, monitors=True, *, key, epochs: Optional[int] = None) -> Mapping[str, AsyncDataset]:
        ...

    @abc.abstractmethod
    def validation_sets(self, Pos, monitors=True) -> Mapping[str, AsyncDataset]:
        ...

    @abc.abstractmethod
    def build_caches(self, split: str, monitors=True) -> Mapping[str, TreeCache]:
        ...

    @property
    @abc.abstractmethod
    def sources(self) -> Mapping[str, LmDatasetSourceConfigBase]:
        ...

    def tagged_eval_sets(self, Pos, monitors=True) -> List[Tuple[AsyncDataset, List[str]]]:
        tags = {name: (cfg.tags or []) + [name] for name, cfg in self.sources.items()}
        eval_sets = self.validation_sets(Pos, monitors)
        return [(eval_sets[name], tags[name]) for name in eval_sets]

    def _perm_type(self) -> str:
        if self.permutation_type is None:
            if self.shuffle is not False:
                logger.warning("Defaulting to linear permutation for shuffling. This will change to Feistel in the future.")
            return "linear"
        return self.permutation_type

    def _shuffle(self, ds: AsyncDataset, key) -> AsyncDataset:
        if self.shuffle is True:
            return ds.shuffle(key, perm_type=self._perm_type())
        if isinstance(self.shuffle, int) and not isinstance(self.shuffle, bool) and self.shuffle > 0:
            return ds.era_shuffle(self.shuffle, key=key, perm_type=self._perm_type())
        return ds


@dataclass(frozen=True)
class SingleDatasetLMConfigBase(LmDatasetSourceConfigBase, LMTaskConfig):
    """One dataset, from URLs or from the Hugging Face hub."""
    cache_dir: Optional[str] = "cache/"

    def train_set(self, Pos, batch_schedule=None, monitors=True, *, key, epochs: Optional[int] = None) -> AsyncDataset:
        cache = self.build_or_load_cache("train", monitors=monitors)
        if cache is None:
            raise ValueError("No training set!")
        ds = dataset_for_format(self.format, Pos, cache, eos_id=self.the_tokenizer.eos_token_id, ignore_index=self.ignore_token_id)
        ds = self._shuffle(ds, key)
        if epochs:
            ds = EpochDataset(ds, max_epochs=epochs)
        return ds

    def train_sets(self, Pos, monitors=True, *, key, epochs: Optional[int] = None) -> Mapping[str, AsyncDataset]:
        return {"": self.train_set(Pos, BatchSchedule(32), monitors, key=key, epochs=epochs)}

    def validation_set(self, Pos, monitors=True) -> Optional[AsyncDataset]:
        cache = self.build_or_load_cache("validation", monitors=monitors)
        if cache is None:
            return None
        return dataset_for_format(self.format, Pos, cache, eos_id=self.the_tokenizer.eos_token_id, ignore_index=self.ignore_token_id)

    def validation_sets(self, Pos, monitors=True) -> Mapping[str, AsyncDataset]:
        v = self.validation_set(Pos, monitors)
        return {} if v is None else {"": v}

    @property
    def sources(self) -> Mapping[str, LmDatasetSourceConfigBase]:
        return {"": self}

    def build_caches(self, split: str, monitors=True) -> Mapping[str, TreeCache]:
        cache = self.build_or_load_cache(split, monitors)
        return {} if cache is None else {"": cache}

    def build_or_load_cache(self, split: str, monitors=True) -> Optional[TreeCache]:
        if self.cache_dir is None:
            raise ValueError("cache_dir cannot be None")
        cache_dir = os.path.join(self.cache_dir, split)
        if fsspec_utils.exists(cache_dir):
            try:
                return load_lm_dataset_cache(cache_dir, self.format, self.the_tokenizer, self.enforce_eos)
            except FileNotFoundError:
                pass
        source = self.get_shard_source(split)
        if source is None:
            logger.warning(f"Skipping {split} because no source was provided")
            return None
        return build_lm_dataset_cache(cache_dir, source, self.format, self.the_tokenizer, self.cache_options, self.enforce_eos, monitors)


@dataclass(frozen=True)
class UrlSingleDatasetLMConfig(SingleDatasetLMConfigBase, UrlDatasetSourceConfig):
    pass


@dataclass(frozen=True)
class HfSingleDatasetLMConfig(SingleDatasetLMConfigBase, HfDatasetSourceConfig):
    pass


# Unions are decoded by trying the members in order: a mapping with ``id`` does not fit the URL config (unknown key) and
# falls through to the hub config; a mapping with neither is a URL config without urls (cache-only).
SingleDatasetLMConfig = Union[UrlSingleDatasetLMConfig, HfSingleDatasetLMConfig]
LMDatasetSourceConfig = Union[UrlDatasetSourceConfig, HfDatasetSourceConfig]


@dataclass(frozen=True)
class LMMixtureDatasetConfig(LMTaskConfig):
    """A weighted mixture of datasets; ``train_weights`` is one mapping or a list of ``(start step, weights)`` stages."""
    cache_dir: Optional[str] = "cache/"
    configs: Dict[str, LMDatasetSourceConfig] = field(default_factory=dict)
    train_weights: Union[Dict[str, float], List[Tuple[int, Dict[str, float]]]] = field(default_factory=dict)
    stop_strategy: str = field(default=StopStrategy.RESTART_STRATEGY)
    # simulated epoching: pretend the run has ``target_budget`` tokens while training on ``experiment_budget``
    target_budget: Optional[int] = None
    experiment_budget: Optional[int] = None
    mixture_block_size: int = 2048
    max_train_batches: Optional[Dict[str, int]] = None
    num_validation_sequences: Optional[Dict[str, int]] = None

    def __post_init__(self):
        if len(self.configs) == 0:
            raise ValueError("At least one dataset must be provided")
        if isinstance(self.train_weights, dict):
            stages = [(0, self.train_weights)]
        elif isinstance(self.train_weights, (list, tuple)):
            stages = list(self.train_weights)
        else:
            raise ValueError(f"Invalid train_weights type: {type(self.train_weights)}")
        for _, w in stages:
            if not all(name in self.configs for name in w):
                raise ValueError(f"Weight keys {list(w.keys())} must be subset of config keys {list(self.configs.keys())}")
        if self.max_train_batches is not None or self.num_validation_sequences is not None:
            assert self.experiment_budget is None and self.target_budget is None, \
                "max_train_batches and num_validation_sequences and simulated data budget cannot all be set"

    def build_token_datasets(self, caches: Mapping[str, TreeCache], Pos) -> Dict[str, AsyncDataset]:
        return {name: dataset_for_format(self.configs[name].format, Pos, cache, eos_id=self.the_tokenizer.eos_token_id,
                                         ignore_index=self.ignore_token_id) for name, cache in caches.items()}

    def train_set(self, Pos, batch_schedule: BatchSchedule, monitors=True, *, key, epochs: Optional[int] = None) -> AsyncDataset:
        mix_key, shuffle_key = _split_key(key, 2)
        weights = self.train_weights
        if isinstance(weights, (list, tuple)):
            weights = rescale_mixture_schedule_for_batch_schedule(weights, batch_schedule)
        initial_batch_size = batch_schedule.batch_size_at_step(0)
        datasets = self.train_sets(Pos, monitors, key=shuffle_key, epochs=epochs, initial_batch_size=initial_batch_size)
        if isinstance(weights, dict):
            weights = {k: v for k, v in weights.items() if k in datasets}
        else:
            weights = [(s, {k: v for k, v in w.items() if k in datasets}) for s, w in weights]
        return MixtureDataset(datasets=datasets, weights=weights, stop_strategy=self.stop_strategy, key=mix_key,
                              block_size=self.mixture_block_size)

    def train_sets(self, Pos, monitors=True, *, initial_batch_size: Optional[int] = None, epochs: Optional[int] = None,
                   key=None) -> Mapping[str, AsyncDataset]:
        if epochs:
            raise ValueError("Epochs are not supported for mixture datasets")
        caches = self.build_caches("train", monitors=monitors)
        datasets = self.build_token_datasets(caches, Pos)
        if key is None:
            key = 0
        # the components are shuffled, not the mixture, so that a block always has the same composition
        if self.shuffle:
            keys = _split_key(key, len(datasets))
            datasets = {name: self._shuffle(ds, k) for (name, ds), k in zip(datasets.items(), keys)}
        if self.experiment_budget is not None and self.target_budget is not None:
            if self.experiment_budget > self.target_budget:
                raise ValueError(f"Experiment budget should be smaller than target budget, got {self.experiment_budget} > {self.target_budget}")
            ratio = self.experiment_budget / self.target_budget
            datasets = {name: ds.slice_dataset(end_index=int(len(ds.as_sync_dataset()) * ratio)) for name, ds in datasets.items()}
        if self.num_validation_sequences is not None:
            for name, ds in list(datasets.items()):
                if name in self.num_validation_sequences:
                    n = len(ds.as_sync_dataset())
                    datasets[name] = ds.slice_dataset(start_index=0, end_index=n - self.num_validation_sequences[name])
        if self.max_train_batches is not None:
            assert initial_batch_size is not None, "initial_batch_size must be provided if max_train_batches is provided"
            for name, ds in list(datasets.items()):
                if name in self.max_train_batches:
                    num = self.max_train_batches[name] * initial_batch_size
                    n = len(ds.as_sync_dataset())
                    assert num <= n, f"Max sequences for {name} ({num}) is greater than the dataset size ({n})"
                    datasets[name] = ds.slice_dataset(end_index=num)
        return datasets

    def validation_sets(self, Pos, monitors=True) -> Mapping[str, AsyncDataset]:
        caches = self.build_caches("validation", monitors=monitors)
        out = self.build_token_datasets(caches, Pos)
        if self.num_validation_sequences is not None:
            train = self.build_token_datasets(self.build_caches("train", monitors=monitors), Pos)
            for name, num in self.num_validation_sequences.items():
                n = len(train[name].as_sync_dataset())
                if name in out:
                    logger.warning(f"Validation dataset {name} already exists, overwriting")
                out[name] = train[name].slice_dataset(start_index=n - num, end_index=n)
        return out

    def build_caches(self, split: str, monitors=True) -> Dict[str, TreeCache]:
        caches: Dict[str, TreeCache] = {}
        stages = [(0, self.train_weights)] if isinstance(self.train_weights, dict) else list(self.train_weights)
        for name, cfg in self.configs.items():
            if split == "train" and not any(w.get(name, 0) > 0 for _, w in stages):
                continue  # never sampled
            if cfg.cache_dir is None:
                if self.cache_dir is None:
                    raise ValueError(f"If the 'main' cache_dir is None, then all component cache_dirs must be non-None, but {name}'s cache_dir is None.")
                cache_dir = os.path.join(self.cache_dir, name)
            else:
                cache_dir = cfg.cache_dir
            source = cfg.get_shard_source(split)
            if source is None:
                try:
                    caches[name] = load_lm_dataset_cache(os.path.join(cache_dir, split), cfg.format, self.the_tokenizer, self.enforce_eos)
                except FileNotFoundError:
                    logger.warning(f"No source for {name} in {split} split and no cache either, skipping")
                continue
            caches[name] = build_lm_dataset_cache(os.path.join(cache_dir, split), source, cfg.format, self.the_tokenizer,
                                                  self.cache_options, self.enforce_eos, monitors)
        if split == "validation":
            for c in caches.values():
                c.await_finished()
        return caches

    @property
    def sources(self) -> Mapping[str, LmDatasetSourceConfigBase]:
        return self.configs


# ------------------------------------------------------------------------------------------------ legacy SFT paths
class SingleTurnChatJsonlDataSource(JsonlDataSource):
    """OpenAI-style chat jsonl -> ``{"input", "output"}`` rows taken from the first ``input_role`` / ``output_role`` messages."""

    def __init__(self, urls: Sequence[str], messages_field: str, input_role: str, output_role: str):
        super().__init__(urls)
        self.messages_field, self.input_role, self.output_role = messages_field, input_role, output_role

    def open_shard_at_row(self, shard_name: str, row: int) -> Iterator[dict]:
        for data in super().open_shard_at_row(shard_name, row):
            msgs = data[self.messages_field]
            inp = next((m["content"] for m in msgs if m["role"] == self.input_role), None)
            out = next((m["content"] for m in msgs if m["role"] == self.output_role), None)
            if inp is None or out is None:
                raise ValueError(f"Conversation is missing a {self.input_role} or {self.output_role} message: {msgs}")
            yield {"input": inp, "output": out}


def datasource_from_chat_jsonl_single_turn(urls: Sequence[str], messages_field: str = "messages", input_role: str = "user",
                                           output_role: str = "assistant") -> ShardedDataSource[dict]:
    return SingleTurnChatJsonlDataSource(urls, messages_field, input_role, output_role)


@dataclass(frozen=True)
class ChatUrlDataSourceConfig:
    cache_dir: str
    train_urls: List[str] = field(default_factory=list)
    validation_urls: List[str] = field(default_factory=list)
    messages_field: str = "messages"
    input_role: str = "user"
    output_role: str = "assistant"

    def get_shard_source(self, split: str) -> Optional[ShardedDataSource[dict]]:
        urls = self.validation_urls if split == "validation" else self.train_urls
        if not urls:
            return None
        return datasource_from_chat_jsonl_single_turn(urls, self.messages_field, self.input_role, self.output_role)


@dataclass(frozen=True)
class SupervisedUrlSourceConfig:
    cache_dir: str
    train_urls: List[str] = field(default_factory=list)
    validation_urls: List[str] = field(default_factory=list)
    input_field: str = CANONICAL_INPUT_FIELD
    output_field: str = CANONICAL_OUTPUT_FIELD
    tags: Optional[List[str]] = None

    def get_shard_source(self, split: str) -> Optional[ShardedDataSource[dict]]:
        urls = self.validation_urls if split == "validation" else self.train_urls
        return UrlDataSource(urls, columns=[self.input_field, self.output_field]) if urls else None


@dataclass(frozen=True)
class SupervisedHfSourceConfig:
    cache_dir: str
    id: str
    name: Optional[str] = None
    streaming: bool = True
    input_field: str = CANONICAL_INPUT_FIELD
    output_field: str = CANONICAL_OUTPUT_FIELD
    tags: Optional[List[str]] = None

    def get_shard_source(self, split: str) -> Optional[ShardedDataSource[dict]]:
        return WrappedHFDataSource(self.id, split=split, name=self.name, streaming=self.streaming).map(
            lambda x: {self.input_field: x[self.input_field], self.output_field: x[self.output_field]})


def _preprocess_supervised_example(batch, tokenizer, input_field: str, output_field: str) -> dict:
    return SupervisedProcessor(tokenizer, input_field, output_field)(batch)


def preprocess_legacy_chat_template(batch, tokenizer, should_append_eos: bool) -> dict:
    sources = [ex["input"] for ex in batch]
    targets = [ex["output"] + (tokenizer.eos_token if should_append_eos else "") for ex in batch]
    src_tok = tokenizer(sources, padding=False, truncation=True)
    ex_tok = tokenizer([f"{s}{t}" for s, t in zip(sources, targets)], padding=False, truncation=True)
    return {"input_ids": [np.array(e, dtype=np.int32) for e in ex_tok["input_ids"]],
            "sources_len": np.array([len(s) for s in src_tok["input_ids"]], dtype=np.int32)}


def _prepare_supervised_examples(exs: Sequence[dict], tokenizer, Pos) -> List[LmExample]:
    """Right-pad (or keep the last ``Pos`` tokens of) each example; loss only on response tokens that are not padding."""
    S = _seq_len(Pos)
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else tokenizer.eos_token_id
    out = []
    for ex in exs:
        ids = np.asarray(ex["input_ids"], dtype=np.int32)[-S:]
        src_len = int(np.asarray(ex["sources_len"]).reshape(-1)[0])
        toks = np.full(S, pad, dtype=np.int32)
        toks[:len(ids)] = ids
        t = torch.from_numpy(toks)
        lm = (torch.arange(S) >= src_len - 1) & (torch.roll(t, -1) != pad)
        out.append(LmExample.causal(t, loss_mask=lm.to(torch.int32), eos_id=tokenizer.eos_token_id))
    return out


def _legacy_sft_cache(config, tokenizer) -> TreeCache:
    source = config.get_shard_source("train")
    if source is None:
        raise ValueError("No training data source found")
    exemplar = {"input_ids": np.zeros((0,), dtype=np.int32), "sources_len": np.zeros((0,), dtype=np.int32)}
    should_append_eos = tokenizer("1 2" if isinstance(tokenizer, PassthroughTokenizer) else "hi there")["input_ids"][-1] != tokenizer.eos_token_id
    ds = source.map_batches(lambda ex: preprocess_legacy_chat_template(ex, tokenizer, should_append_eos), batch_size=128,
                            num_cpus=num_cpus_used_by_tokenizer(tokenizer), output_exemplar=exemplar)
    return ds.build_or_load_cache(config.cache_dir, await_finished=True)


def mk_single_turn_cached_sft_dataset(config: ChatUrlDataSourceConfig, tokenizer, Pos) -> AsyncDataset:
    return _legacy_sft_cache(config, tokenizer)


def mk_chat_sft_dataset(config: ChatUrlDataSourceConfig, tokenizer, Pos) -> AsyncDataset:
    cached = _legacy_sft_cache(config, tokenizer)
    return cached.map_batches(lambda ex: _prepare_supervised_examples(ex, tokenizer, Pos))


def mk_supervised_dataset(config, split: str, tokenizer, Pos) -> AsyncDataset:
    source = config.get_shard_source(split)
    if source is None:
        raise ValueError(f"No data source for split {split}")
    exemplar = {"input_ids": np.zeros((0,), dtype=np.int32), "sources_len": np.zeros((0,), dtype=np.int32)}
    ds = source.map_batches(lambda ex: _preprocess_supervised_example(ex, tokenizer, config.input_field, config.output_field),
                            batch_size=128, num_cpus=num_cpus_used_by_tokenizer(tokenizer), output_exemplar=exemplar)
    cached = ds.build_or_load_cache(os.path.join(config.cache_dir, split), await_finished=True)
    return cached.map_batches(lambda ex: _prepare_supervised_examples(ex, tokenizer, Pos))


def count_corpus_sizes(config, prefix: str = "data/stats/", seq_len: int = 4096) -> dict:
    """Token/document/sequence counts of every training cache (and the mixture weights), for logging at start-up."""
    stats: Dict[str, Any] = {}
    caches = config.build_caches("train")
    weights = None
    if isinstance(config, LMMixtureDatasetConfig):
        weights = config.train_weights if isinstance(config.train_weights, dict) else config.train_weights[0][1]
    for name, cache in caches.items():
        cache.await_finished()
        tag = f"{prefix}train/{name}/" if name else f"{prefix}train/"
        toks = cache.store.tree[("input_ids",)]
        stats[f"{tag}total_tokens"] = toks.data_size
        stats[f"{tag}total_docs"] = toks.num_rows
        stats[f"{tag}total_seqs"] = toks.data_size // seq_len
        if weights is not None:
            stats[f"{tag}weight"] = weights.get(name, 0.0)
    return stats
