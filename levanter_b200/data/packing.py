"""Sequence packing (src/levanter/data/packing.py): several short documents share one ``seq_len`` row, kept apart in attention
by segment ids; padding has segment id -1 and loss mask 0.

* :class:`SequencePacker`, :func:`pack_prompt_completions` (:52-165): online first-fit packing of prompt/completion pairs
  for evaluation harnesses.
* :func:`pack_documents` (:335-430): greedy *contiguous* packing from document lengths alone.  The reference recomputes the
  token sum of a pack for every candidate document; this version carries running sums, so it is linear in the number of
  documents.
* :class:`GreedyPrepackedDataset` (:433-580): a packed view over a tree of jagged stores; one range read per pack and leaf.
* :func:`per_segment_loss`, :func:`per_segment_correct` (:167-255): scatter-reduce per-position values by segment id.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..layers.attention import AttentionMask
from ..models.lm_model import LmExample
from .dataset import AsyncDataset


def _seq_len(Pos) -> int:
    return int(getattr(Pos, "size", Pos))


class SequencePacker:
    """Accumulates (ids, loss mask) pairs into one row of ``Pos`` tokens."""

    def __init__(self, Pos, max_pack_size: int, pad_token: int):
        if pad_token is None:
            raise ValueError("pad_token must be set")
        self.Pos = Pos
        self.seq_len = _seq_len(Pos)
        self._ids: List[int] = []
        self._segment_ids: List[int] = []
        self._loss_mask: List[int] = []
        self.num_segments = 0
        self.pad_token = pad_token
        self.max_pack_size = max_pack_size

    def can_pack(self, ids: Sequence[int]) -> bool:
        return len(ids) + len(self._ids) <= self.seq_len and self.num_segments < self.max_pack_size

    def add_example(self, ids: Sequence[int], loss_mask, segment_id: Optional[int] = None) -> None:
        if len(ids) != len(loss_mask):
            raise ValueError("ids and loss_mask must have the same length")
        if len(ids) == 0:
            return
        if len(ids) + len(self._ids) > self.seq_len:
            raise ValueError("Too many tokens")
        if self.num_segments >= self.max_pack_size:
            raise ValueError("Too many segments")
        self._ids.extend(int(i) for i in ids)
        if segment_id is None:
            segment_id = self.num_segments
        self.num_segments += 1
        self._segment_ids.extend([segment_id] * len(ids))
        self._loss_mask.extend(int(m) for m in loss_mask)

    def pack(self) -> LmExample:
        pad = self.seq_len - len(self._ids)
        tokens = torch.tensor(self._ids + [self.pad_token] * pad, dtype=torch.int32)
        seg = torch.tensor(self._segment_ids + [-1] * pad, dtype=torch.int32)
        lm = torch.tensor(self._loss_mask + [0] * pad, dtype=torch.int32)
        return LmExample(tokens=tokens, loss_mask=lm, attn_mask=AttentionMask.causal().with_segment_ids(seg))


@dataclass(frozen=True)
class PromptCompletion:
    ids: List[int]
    prompt_length: int
    segment_id: Optional[int] = None

    def __post_init__(self):
        if len(self.ids) == 0:
            raise ValueError("PromptCompletion must have at least one token")
        if len(self.ids) <= self.prompt_length:
            raise ValueError(f"PromptCompletion must have strictly more tokens than the prompt length. Got {len(self.ids)} tokens"
                             f" and prompt length {self.prompt_length}")


def _prompt_loss_mask(n: int, prompt_length: int) -> np.ndarray:
    m = np.arange(n) >= prompt_length - 1
    m[-1] = False
    return m


def pack_prompt_completions(Pos, sequences: Iterable[PromptCompletion], pad_token: int, max_segments_per_example: int = 64,
                            max_buffered_examples: int = 64) -> Iterator[LmExample]:
    """First-fit packing with at most ``max_buffered_examples`` open rows; the oldest row is emitted when the buffer fills."""
    packers = [SequencePacker(Pos, max_segments_per_example, pad_token)]
    for seq in sequences:
        lm = _prompt_loss_mask(len(seq.ids), seq.prompt_length)
        for packer in packers:
            if packer.can_pack(seq.ids):
                packer.add_example(seq.ids, lm, seq.segment_id)
                if packer.num_segments == max_segments_per_example:
                    yield packer.pack()
                    packers.remove(packer)
                break
        else:
            packer = SequencePacker(Pos, max_segments_per_example, pad_token)
            packer.add_example(seq.ids, lm, seq.segment_id)
            packers.append(packer)
        while len(packers) >= max_buffered_examples:
            yield packers.pop(0).pack()
    for packer in packers:
        yield packer.pack()


def _leaves(tree, prefix=()) -> List[Tuple[tuple, object]]:
    if isinstance(tree, dict):
        out = []
        for k in tree:
            out.extend(_leaves(tree[k], prefix + (k,)))
        return out
    return [(prefix, tree)]


def _broadcast(value, like) -> Dict[tuple, int]:
    if isinstance(value, dict):
        return {p: int(v) for p, v in _leaves(value)}
    return {p: int(value) for p, _ in _leaves(like)}


def pack_documents(lengths, max_length, max_segments_per_example: Optional[int] = None,
                   slice_too_long_examples: bool = False) -> List[range]:
    """Greedy contiguous packing.  ``lengths``: an array (or dict tree of arrays) of per-document lengths; ``max_length``: the
    capacity per leaf.  Returns the document-index range of every pack; a document longer than the capacity raises unless
    ``slice_too_long_examples``, in which case it gets a pack of its own."""
    if max_segments_per_example is not None and (not isinstance(max_segments_per_example, int) or max_segments_per_example <= 0):
        raise ValueError(f"max_segments_per_example must be a positive integer, got {max_segments_per_example}")
    leaves = _leaves(lengths)
    caps = _broadcast(max_length, lengths)
    if set(caps) != {p for p, _ in leaves}:
        raise ValueError("Lengths and max_length PyTrees must have the same number of leaves.")
    n_docs = None
    for _, lens in leaves:
        if n_docs is None:
            n_docs = len(lens)
        elif len(lens) != n_docs:
            raise ValueError("All leaves must have the same number of documents.")
    if n_docs is None:
        raise ValueError("Could not determine the number of documents from lengths.")
    arrs = [np.asarray(lens, dtype=np.int64) for _, lens in leaves]
    cap = np.array([caps[p] for p, _ in leaves], dtype=np.int64)
    if not slice_too_long_examples:
        for (p, _), a, c in zip(leaves, arrs, cap):
            bad = np.nonzero(a > c)[0]
            if len(bad):
                raise ValueError(f"Document {int(bad[0])} in leaf '{'.'.join(map(str, p))}' has length {int(a[bad[0]])} which exceeds "
                                 f"maximum allowed length {int(c)}. Consider setting slice_too_long_examples=True or increasing max_length.")
    lens2d = np.stack(arrs, axis=1) if arrs else np.zeros((n_docs, 0), dtype=np.int64)  # [docs, leaves]
    out: List[range] = []
    start = 0
    sums = np.zeros(len(arrs), dtype=np.int64)
    segs = 0
    max_segs = max_segments_per_example if max_segments_per_example is not None else 1 << 62
    for i in range(n_docs):
        row = lens2d[i]
        if segs > 0 and (segs + 1 > max_segs or np.any(sums + row > cap)):
            out.append(range(start, i))
            start, segs = i, 0
            sums[:] = 0
        sums += row
        segs += 1
    if segs > 0:
        out.append(range(start, n_docs))
    return out


def greedy_pack_prompt_completions(Pos, sequences: Iterable[PromptCompletion], pad_token: int,
                                   max_segments_per_example: int = 64) -> List[LmExample]:
    """Contiguous packing of prompt/completions; segment ids are the positions of the sequences in the input."""
    S = _seq_len(Pos)
    sequences = list(sequences)
    packs = pack_documents(np.array([len(s.ids) for s in sequences]), S, max_segments_per_example, slice_too_long_examples=True)
    out = []
    for docs in packs:
        ids: List[int] = []
        lm: List[int] = []
        seg: List[int] = []
        for d in docs:
            s = sequences[d]
            ids.extend(s.ids)
            lm.extend(_prompt_loss_mask(len(s.ids), s.prompt_length).astype(np.int32).tolist())
            seg.extend([d] * len(s.ids))
        pad = S - len(ids)
        if pad > 0:
            ids += [pad_token] * pad
            lm += [0] * pad
            seg += [-1] * pad
        elif pad < 0:
            if len(docs) != 1:
                raise ValueError("Too many tokens in a pack with more than one document")
            ids, lm, seg = ids[-S:], lm[-S:], seg[-S:]
        out.append(LmExample(tokens=torch.tensor(ids, dtype=torch.int32), loss_mask=torch.tensor(lm, dtype=torch.int32),
                             attn_mask=AttentionMask.causal().with_segment_ids(torch.tensor(seg, dtype=torch.int32))))
    return out


def _segment_ids_of(example: LmExample) -> torch.Tensor:
    seg = example.attn_mask.segment_ids
    if seg is None:
        raise ValueError("segment_ids must be set in the AttentionMask")
    if isinstance(seg, tuple):
        seg = seg[0]
    if seg.dim() != 1:
        raise ValueError(f"Expected segment_ids to be 1D, got {seg.dim()}")
    return seg


def _unique_segment_ids(max_segments: int, segment_ids: torch.Tensor) -> torch.Tensor:
    """Sorted unique ids padded with -1 to a fixed ``max_segments`` (static shape: no host sync on the count)."""
    uniq = torch.unique(segment_ids)
    out = torch.full((max_segments,), -1, dtype=segment_ids.dtype, device=segment_ids.device)
    n = min(max_segments, uniq.numel())
    out[:n] = uniq[:n]
    return out


def per_segment_loss(packed_example: LmExample, losses: torch.Tensor, max_Segments) -> Tuple[torch.Tensor, torch.Tensor]:
    """(segment ids ``[max_segments]`` padded with -1, summed masked loss per segment)."""
    seg = _segment_ids_of(packed_example)
    masked = losses.float() * packed_example.loss_mask.to(losses.device).float()
    uniq = _unique_segment_ids(_seq_len(max_Segments), seg)
    onehot = (uniq[:, None] == seg[None, :]).float()
    return uniq, onehot @ masked


def per_segment_correct(packed_example: LmExample, correct: torch.Tensor, max_Segments) -> Tuple[torch.Tensor, torch.Tensor]:
    """(segment ids, whether every loss-bearing token of the segment is correct)."""
    seg = _segment_ids_of(packed_example)
    ok = correct.bool() | ~packed_example.loss_mask.to(correct.device).bool()
    uniq = _unique_segment_ids(_seq_len(max_Segments), seg)
    member = uniq[:, None] == seg[None, :]
    return uniq, torch.where(member, ok[None, :], torch.ones_like(member)).all(dim=1)


class GreedyPrepackedDataset(AsyncDataset):
    """Packed view over ``dataset`` = {leaf: JaggedArrayStore}.  Item ``i`` is ``(data, segment_ids)``: two dicts with the
    structure of ``dataset``, each leaf padded to its ``max_length`` (data with 0, segment ids with -1).

    ``slice_strategy`` for documents longer than the capacity: ``left`` keeps the first tokens, ``right`` the last, ``raise``
    rejects them."""

    def __init__(self, dataset, max_length, max_segments_per_example: Optional[int] = None, pad_with_zeros: bool = True,
                 slice_strategy: str = "raise"):
        super().__init__()
        if slice_strategy not in ("left", "right", "raise"):
            raise ValueError(f"slice_strategy must be one of 'left', 'right', or 'raise', got {slice_strategy}")
        self._single = not isinstance(dataset, dict)
        self.dataset = {(): dataset} if self._single else {p: s for p, s in _leaves(dataset)}
        self.max_length = {(): int(max_length)} if self._single else _broadcast(max_length, dataset)
        self.max_segments_per_example = max_segments_per_example
        self.pad_with_zeros = pad_with_zeros
        self.slice_strategy = slice_strategy
        self._offsets: Dict[tuple, np.ndarray] = {}
        lengths = {}
        for p, store in self.dataset.items():
            n = store.num_rows
            offs = store.offsets.read([0], [n + 1]).astype(np.int64)
            offs[0] = 0
            self._offsets[p] = offs
            lengths[p] = np.diff(offs)
        self._pack_indices = pack_documents(lengths if not self._single else lengths[()],
                                            self.max_length if not self._single else self.max_length[()],
                                            max_segments_per_example, slice_strategy != "raise")

    def is_finite(self) -> bool:
        return True

    async def async_len(self) -> int:
        return len(self._pack_indices)

    async def final_length_is_known(self) -> bool:
        return True

    async def current_len(self) -> Optional[int]:
        return len(self._pack_indices)

    def _leaf_batch(self, p, ranges: List[range]):
        store, offs, allowed = self.dataset[p], self._offsets[p], self.max_length[p]
        data, segs = [], []
        for dr in ranges:
            t0, t1 = int(offs[dr.start]), int(offs[dr.stop])
            if t1 - t0 > allowed:
                if self.slice_strategy == "raise":
                    raise ValueError(f"Token count {t1 - t0} exceeds allowed maximum {allowed} for documents {list(dr)}.")
                assert len(dr) == 1, "a document longer than the capacity is always alone in its pack"
                if self.slice_strategy == "right":
                    t0 = t1 - allowed
                else:
                    t1 = t0 + allowed
            x = store.data.read([t0], [t1])
            doc_lens = np.minimum(np.diff(offs[dr.start:dr.stop + 1]), allowed)
            s = np.repeat(np.arange(dr.start, dr.stop, dtype=np.int64), doc_lens)
            if self.pad_with_zeros:
                x = np.pad(x, (0, allowed - len(x)))
                s = np.pad(s, (0, allowed - len(s)), constant_values=-1)
            data.append(x)
            segs.append(s)
        return data, segs

    async def get_batch(self, indices: Sequence[int]):
        ranges = [self._pack_indices[int(i)] for i in indices]
        per_leaf = {p: self._leaf_batch(p, ranges) for p in self.dataset}
        out = []
        for i in range(len(ranges)):
            if self._single:
                out.append((per_leaf[()][0][i], per_leaf[()][1][i]))
            else:
                out.append((_unflatten({p: v[0][i] for p, v in per_leaf.items()}), _unflatten({p: v[1][i] for p, v in per_leaf.items()})))
        return out


def _unflatten(flat: Dict[tuple, object]):
    out: dict = {}
    for p, v in flat.items():
        d = out
        for k in p[:-1]:
            d = d.setdefault(k, {})
        d[p[-1]] = v
    return out
