"""Tagged evaluation of language models (src/levanter/eval.py): several validation sets, each with hierarchical tags
(``"web/wiki"``), evaluated in one pass; logs the micro average (token weighted) as ``eval/loss``, the macro average over
leaf tags, per-tag losses, and bits-per-byte when a tokenizer is given.

Per-batch work stays on the device: the per-token losses come from the fused cross-entropy path with ``reduction=None`` and
are folded into ``[1 + 2T]`` running sums (loss, tokens, bytes per tag) by two small matmuls, so a pass over the validation
data synchronises with the host once, at the end (plus one all-reduce across data-parallel ranks)."""
from __future__ import annotations

import asyncio
import dataclasses
import logging
import math
import time
import warnings
from collections import defaultdict
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import tracker as trk
from .callbacks import StepInfo
from .data.dataset import AsyncDataset
from .data.loader import DataLoader
from .models.lm_model import LmExample, LmHeadModel, compute_next_token_loss
from .utils.hf_utils import byte_length_of_token

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class EvalResult:
    micro_avg_loss: float  # per token across all datasets
    macro_avg_loss: float  # mean of the per-leaf-tag losses
    tag_macro_losses: Dict[str, float]  # per parent tag: mean over its children
    tag_micro_losses: Dict[str, float]  # per tag: token weighted
    total_eval_loading_time: float
    micro_bpb: Optional[float] = None
    macro_bpb: Optional[float] = None
    tag_macro_bpb: Optional[Dict[str, float]] = None
    tag_micro_bpb: Optional[Dict[str, float]] = None


class DomainTaggedDataset(AsyncDataset):
    """Concatenation of datasets; item ``i`` is ``(example, multi-hot tag vector of its dataset)``."""

    def __init__(self, datasets: Sequence[Tuple[AsyncDataset, Sequence[str]]], max_examples_per_dataset: Optional[int] = None):
        super().__init__()
        self.datasets: List[Tuple[AsyncDataset, Sequence[str]]] = []
        self._max = max_examples_per_dataset
        tag_index: Dict[str, int] = {}
        for i, (ds, tags) in enumerate(datasets):
            if not tags and len(datasets) > 1:
                warnings.warn("Dataset has no tags. Giving it an index")
                tags = [f"domain_{i}"]
            for t in tags:
                tag_index.setdefault(t, len(tag_index))
            if self._max:
                ds = ds.take(self._max)
            self.datasets.append((ds, list(tags)))
        self.tag_to_index = tag_index
        self.num_tags = len(tag_index)
        self._tag_arrays = []
        for _, tags in self.datasets:
            v = np.zeros(max(self.num_tags, 1), dtype=np.float32)
            for t in tags:
                v[tag_index[t]] = 1
            self._tag_arrays.append(v)
        self._offsets: Optional[np.ndarray] = None

    @property
    def tags(self):
        return self.tag_to_index.keys()

    async def _get_offsets(self) -> np.ndarray:
        if self._offsets is None:
            lengths = [await ds.async_len() for ds, _ in self.datasets]
            if self._max is not None:
                lengths = [min(n, self._max) for n in lengths]
            self._offsets = np.cumsum([0] + lengths)
        return self._offsets

    async def async_len(self) -> int:
        return int((await self._get_offsets())[-1])

    async def final_length_is_known(self) -> bool:
        return all([await ds.final_length_is_known() for ds, _ in self.datasets])

    def is_finite(self) -> bool:
        return all(ds.is_finite() for ds, _ in self.datasets)

    async def current_len(self) -> Optional[int]:
        return await self.async_len()

    async def getitem_async(self, item: int):
        return (await self.get_batch([item]))[0]

    async def get_batch(self, indices: Sequence[int]):
        offsets = await self._get_offsets()
        which = np.searchsorted(offsets, np.asarray(indices), side="right") - 1
        grouped: Dict[int, List[Tuple[int, int]]] = defaultdict(list)
        for out_pos, (idx, d) in enumerate(zip(indices, which)):
            grouped[int(d)].append((out_pos, int(idx - offsets[d])))
        out: list = [None] * len(indices)
        for d, items in grouped.items():
            ds, _ = self.datasets[d]
            got = await ds.get_batch([i for _, i in items])
            for (p, _), ex in zip(items, got):
                out[p] = (ex, self._tag_arrays[d])
        return out


def _join_prefix(prefix: str, tag: str) -> str:
    return f"{prefix}/{tag}" if prefix else tag


class TaggedEvaluator:
    def __init__(self, EvalBatch, tagged_eval_sets: Sequence[Tuple[AsyncDataset, Sequence[str]]], tokenizer=None, device_mesh=None,
                 axis_mapping=None, max_examples_per_dataset: Optional[int] = None, mp=None, device=None):
        self.EvalBatch = EvalBatch
        batch_size = int(getattr(EvalBatch, "size", EvalBatch))
        self.dataset = DomainTaggedDataset(tagged_eval_sets, max_examples_per_dataset)
        self.loader = DataLoader(self.dataset, batch_size, mesh=device_mesh, max_buffered_batches=100,
                                 allow_nondivisible_batch_size=True)
        self.mesh = device_mesh
        self.mp = mp
        self.device = device
        self.tokenizer = tokenizer
        self.bytes_per_token = self._calculate_bytes_per_token_type(tokenizer)
        hierarchy: Dict[str, List[int]] = {}
        for tag, index in self.dataset.tag_to_index.items():
            parts = tag.split("/")
            for i in range(1, len(parts)):
                hierarchy.setdefault("/".join(parts[:i]), []).append(index)
        self.hierarchy = hierarchy

    def _calculate_bytes_per_token_type(self, tokenizer) -> Optional[torch.Tensor]:
        from .data.passthrough_tokenizer import PassthroughTokenizer

        if tokenizer is None or isinstance(tokenizer, PassthroughTokenizer):  # token ids without text have no byte length
            return None
        n = len(tokenizer.get_vocab())
        return torch.tensor([byte_length_of_token(tokenizer, i) for i in range(n)], dtype=torch.float32)

    @torch.no_grad()
    def evaluate(self, m: LmHeadModel) -> EvalResult:
        device = self.device or next(m.parameters()).device
        T = max(self.dataset.num_tags, 1)
        # sums: [0]=loss, [1]=tokens, [2]=bytes, then per tag loss / tokens / bytes
        sums = torch.zeros(3 + 3 * T, dtype=torch.float64, device=device)
        bpt = self.bytes_per_token.to(device) if self.bytes_per_token is not None else None
        was_training = m.training
        m.eval()
        load_time = 0.0
        it = iter(self.loader)
        try:
            while True:
                t0 = time.time()
                try:
                    batch, tags = next(it)
                except StopIteration:
                    break
                load_time += time.time() - t0
                batch = batch.to(device, non_blocking=True)
                tags = tags.to(device, non_blocking=True).float()  # [B, T]
                losses = compute_next_token_loss(m, batch, reduction=None).float()  # [B, S]
                mask = batch.loss_mask.float()
                loss_per_ex = (losses * mask).sum(-1)
                tok_per_ex = mask.sum(-1)
                if bpt is not None:
                    nxt = torch.roll(batch.tokens, -1, dims=-1).long().clamp_(0, bpt.numel() - 1)
                    bytes_per_ex = (bpt[nxt] * mask).sum(-1)
                else:
                    bytes_per_ex = torch.zeros_like(tok_per_ex)
                per_ex = torch.stack([loss_per_ex, tok_per_ex, bytes_per_ex], dim=0).double()  # [3, B]
                sums[:3] += per_ex.sum(-1)
                sums[3:] += (per_ex @ tags.double()).reshape(-1)
        finally:
            m.train(was_training)
        if self.mesh is not None and torch.distributed.is_available() and torch.distributed.is_initialized() \
                and torch.distributed.get_world_size() > 1:
            torch.distributed.all_reduce(sums)
        s = sums.cpu().numpy()
        loss_sum, tokens, nbytes = s[0], s[1], s[2]
        tag_loss, tag_tok, tag_bytes = s[3:3 + T], s[3 + T:3 + 2 * T], s[3 + 2 * T:3 + 3 * T]
        log2e = math.log2(math.e)
        mean_per_tag = np.divide(tag_loss, tag_tok, out=np.zeros_like(tag_loss), where=tag_tok > 0)
        bpb_per_tag = np.divide(tag_loss * log2e, tag_bytes, out=np.zeros_like(tag_loss), where=tag_bytes > 0)
        has = tag_tok > 0
        micro = float(loss_sum / max(tokens, 1.0))
        macro = float(mean_per_tag[has].mean()) if has.any() else micro
        tag_macro, tag_micro, tag_macro_bpb, tag_micro_bpb = {}, {}, {}, {}
        for parent, children in self.hierarchy.items():
            ch = np.array([c for c in children if has[c]], dtype=np.int64)
            if len(ch) == 0:
                continue
            tag_macro[parent] = float(mean_per_tag[ch].mean())
            tag_micro[parent] = float(tag_loss[ch].sum() / tag_tok[ch].sum())
            if bpt is not None:
                tag_macro_bpb[parent] = float(bpb_per_tag[ch].mean())
                tag_micro_bpb[parent] = float(tag_loss[ch].sum() * log2e / max(tag_bytes[ch].sum(), 1.0))
        for tag, idx in self.dataset.tag_to_index.items():
            tag_micro[tag] = float(mean_per_tag[idx])
            if bpt is not None:
                tag_micro_bpb[tag] = float(bpb_per_tag[idx])
        if bpt is not None:
            return EvalResult(micro, macro, tag_macro, tag_micro, load_time, float(loss_sum * log2e / max(nbytes, 1.0)),
                              float(bpb_per_tag[has].mean()) if has.any() else 0.0, tag_macro_bpb, tag_micro_bpb)
        return EvalResult(micro, macro, tag_macro, tag_micro, load_time)


def _construct_log_dict(evaluator: TaggedEvaluator, r: EvalResult, total_time: float, prefix: str) -> Dict[str, float]:
    d = {_join_prefix(prefix, "loss"): r.micro_avg_loss, _join_prefix(prefix, "loading_time"): r.total_eval_loading_time,
         _join_prefix(prefix, "total_time"): total_time}
    logger.info(f"{prefix} loss: {r.micro_avg_loss:.3f}")
    leaf = evaluator.dataset.tag_to_index
    has_tags = len(leaf) > 1
    if has_tags:
        d[_join_prefix(prefix, "macro_loss")] = r.macro_avg_loss
        for tag, loss in r.tag_macro_losses.items():
            if tag and tag not in leaf:
                d[_join_prefix(prefix, tag) + "/macro_loss"] = loss
    for tag, loss in r.tag_micro_losses.items():
        if not tag:
            continue
        d[_join_prefix(prefix, tag) + ("/loss" if tag in leaf else "/micro_loss")] = loss
    if evaluator.bytes_per_token is not None and r.micro_bpb is not None:
        d[_join_prefix(prefix, "bpb")] = r.micro_bpb
        if has_tags:
            d[_join_prefix(prefix, "macro_bpb")] = r.macro_bpb
            for tag, b in (r.tag_macro_bpb or {}).items():
                d[_join_prefix(prefix, tag) + "/macro_bpb"] = b
        for tag, b in (r.tag_micro_bpb or {}).items():
            if tag:
                d[_join_prefix(prefix, tag) + "/bpb"] = b
    return d


def eval_model(evaluator: TaggedEvaluator, model: LmHeadModel, prefix: str = "") -> Dict[str, float]:
    t0 = time.time()
    result = evaluator.evaluate(model)
    return _construct_log_dict(evaluator, result, time.time() - t0, prefix=prefix)


def cb_tagged_lm_evaluate(EvalBatch, tagged_eval_sets, tokenizer=None, device_mesh=None, axis_mapping=None,
                          max_examples_per_dataset: Optional[int] = None, eval_current: bool = True, eval_ema: bool = True,
                          prefix: str = "eval", mp=None) -> Callable[[StepInfo], None]:
    """Hook evaluating the current weights (and the averaged weights when model averaging is on, under ``<prefix>/ema``)."""
    if not eval_current and not eval_ema:
        raise ValueError("At least one of eval_current or eval_ema should be True")
    evaluator = TaggedEvaluator(EvalBatch, tagged_eval_sets, tokenizer, device_mesh, axis_mapping, max_examples_per_dataset, mp=mp)

    def eval_callback(step: StepInfo):
        if eval_current:
            trk.log(eval_model(evaluator, step.model, prefix=prefix), step=step.step)
        if not eval_current and step.state.model_averaging is None:
            raise ValueError("Cannot evaluate EMA model without model averaging, but you only want to evaluate EMA")
        if eval_ema and step.state.model_averaging is not None:
            trk.log(eval_model(evaluator, step.eval_model, prefix=_join_prefix(prefix, "ema")), step=step.step)

    return eval_callback
