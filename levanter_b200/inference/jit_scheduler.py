"""Scheduler state of the generation engine (src/levanter/inference/jit_scheduler.py:19-682): the per-slot token buffers and
decoding parameters (``DecodeState``), the queue of sampled tokens waiting to be fed back (``TokenQueue``) and the stream of
outputs handed to the host loop (``_DecodeOutputs``).

The reference runs this bookkeeping inside compiled device loops.  Here it is host state (numpy) updated between kernel
launches; the device only ever sees packed token/slot/position arrays and a ``PageBatchInfo``.  Methods return the updated
object (``state = state.update_tokens(...)``) like the reference; ``TokenQueue`` and ``_DecodeOutputs`` are values,
``DecodeState`` updates its large token buffers in place and returns itself."""
from __future__ import annotations

import ctypes
import dataclasses
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

from .page_table import _I32P, PageTable, _lib, _np, _p
from .utils import INVALID, is_stop_signal, is_valid, purge_raw


@dataclass
class PackedSequence:
    """Tokens dequeued for one forward pass, sorted by slot (stable), padded with INVALID."""
    tokens: np.ndarray
    slot_ids: np.ndarray
    pos_ids: np.ndarray
    num_tokens: int

    def token_counts_per_slot(self, max_slots: int) -> np.ndarray:
        s = self.slot_ids[:self.num_tokens]
        return np.bincount(s[(s >= 0) & (s < max_slots)], minlength=max_slots).astype(np.int32)


@dataclass
class SeqDecodingParams:
    max_num_tokens: int  # prompt included
    stop_tokens: Optional[np.ndarray]  # i32[stop_seq, position], left padded with INVALID
    temperature: float
    key: int  # seed of the per-sequence counter-based generator

    @staticmethod
    def default() -> "SeqDecodingParams":
        return SeqDecodingParams(max_num_tokens=np.iinfo(np.int32).max - 100000, stop_tokens=None, temperature=0.0, key=0)


@dataclass
class TokenQueue:
    queued_tokens: np.ndarray
    queued_slot_ids: np.ndarray
    queued_pos_ids: np.ndarray
    num_queued_tokens: int

    @property
    def max_queued_tokens(self) -> int:
        return self.queued_tokens.shape[0]

    @property
    def empty_queue_space(self) -> int:
        return self.max_queued_tokens - self.num_queued_tokens

    @staticmethod
    def init(max_queued_tokens: int) -> "TokenQueue":
        f = lambda: np.full(max_queued_tokens, INVALID, dtype=np.int32)  # noqa: E731
        return TokenQueue(f(), f(), f(), 0)

    def _copy(self) -> "TokenQueue":
        return TokenQueue(self.queued_tokens.copy(), self.queued_slot_ids.copy(), self.queued_pos_ids.copy(), self.num_queued_tokens)

    def enqueue_tokens(self, new_tokens, new_slot_ids, new_pos_ids, num_new_tokens: int) -> "TokenQueue":
        """Append the first ``num_new_tokens`` entries; what does not fit is dropped (callers size the queue so it fits)."""
        q = self._copy()
        n = int(min(num_new_tokens, q.empty_queue_space))
        a = q.num_queued_tokens
        q.queued_tokens[a:a + n] = _np(new_tokens)[:n]
        q.queued_slot_ids[a:a + n] = _np(new_slot_ids)[:n]
        q.queued_pos_ids[a:a + n] = _np(new_pos_ids)[:n]
        q.num_queued_tokens = a + n
        return q

    def pack_next_sequence(self, max_tokens: int) -> Tuple["TokenQueue", PackedSequence]:
        q = self._copy()
        out_t = np.empty(max_tokens, np.int32)
        out_s = np.empty(max_tokens, np.int32)
        out_p = np.empty(max_tokens, np.int32)
        lib = _lib()
        if lib is not None:
            nq = ctypes.c_int(q.num_queued_tokens)
            n = lib.lvb_tq_pack_next(_p(q.queued_tokens), _p(q.queued_slot_ids), _p(q.queued_pos_ids), ctypes.byref(nq),
                                     q.max_queued_tokens, max_tokens, _p(out_t), _p(out_s), _p(out_p))
            q.num_queued_tokens = nq.value
        else:
            n = min(q.num_queued_tokens, max_tokens)
            order = np.argsort(q.queued_slot_ids[:n], kind="stable")
            for dst, src in ((out_t, q.queued_tokens), (out_s, q.queued_slot_ids), (out_p, q.queued_pos_ids)):
                dst[:] = INVALID
                dst[:n] = src[:n][order]
                rest = src[n:q.num_queued_tokens].copy()
                src[:] = INVALID
                src[:len(rest)] = rest
            q.num_queued_tokens -= n
        return q, PackedSequence(out_t, out_s, out_p, int(n))

    def purge_queue_of_slot(self, slot_id) -> "TokenQueue":
        ids = np.atleast_1d(_np(slot_id))
        drop = np.isin(self.queued_slot_ids, ids)
        s = purge_raw(self.queued_slot_ids, drop)
        return TokenQueue(purge_raw(self.queued_tokens, drop), s, purge_raw(self.queued_pos_ids, drop), int((s != INVALID).sum()))

    def cleared(self) -> "TokenQueue":
        return TokenQueue.init(self.max_queued_tokens)


@dataclass
class DecodeState:
    """The hot set of sequences being decoded.  ``tokens[slot]`` holds prompt and generated tokens; ``seq_lens[slot]`` how
    many of them exist.  ``max_num_tokens`` counts the prompt.  ``clone_sources[slot]`` names the slot a pending clone will
    copy its prefix from (INVALID otherwise)."""
    tokens: np.ndarray  # i32[seq, position]
    logprobs: Optional[np.ndarray]  # f32[seq, position], nan where unknown (prompt)
    seq_lens: np.ndarray  # i32[seq]
    clone_sources: np.ndarray  # i32[seq]
    kv_pages: np.ndarray  # i32[seq, page]
    page_size: int
    page_table: PageTable
    max_num_tokens: np.ndarray  # i32[seq]
    stop_tokens: Optional[np.ndarray]  # i32[seq, stop_seq, position]
    temperature: np.ndarray  # f32[seq]
    prng_keys: np.ndarray  # u64[seq]
    tqueue: TokenQueue
    finished: np.ndarray  # bool[seq]

    @staticmethod
    def init(page_table: PageTable, pad_token_id: int = INVALID, max_stop_seqs: int = 0, max_stop_tokens: int = 16,
             max_queued_tokens: int = 0, enable_logprobs: bool = False) -> "DecodeState":
        S, P, L = page_table.max_seqs, page_table.pages_per_seq, page_table.max_len_per_seq
        return DecodeState(
            tokens=np.full((S, L), pad_token_id, dtype=np.int32),
            logprobs=np.full((S, L), np.nan, dtype=np.float32) if enable_logprobs else None,
            seq_lens=np.zeros(S, dtype=np.int32), clone_sources=np.full(S, INVALID, dtype=np.int32),
            kv_pages=np.full((S, P), INVALID, dtype=np.int32), page_size=page_table.page_size, page_table=page_table,
            max_num_tokens=np.zeros(S, dtype=np.int32),
            stop_tokens=np.full((S, max_stop_seqs, max_stop_tokens), INVALID, dtype=np.int32) if max_stop_tokens > 0 else None,
            temperature=np.ones(S, dtype=np.float32), prng_keys=np.zeros(S, dtype=np.uint64),
            tqueue=TokenQueue.init(max(max_queued_tokens, 0)), finished=np.zeros(S, dtype=bool))

    # -- sizes ------------------------------------------------------------------------------------------------
    @property
    def max_seqs(self) -> int:
        return self.tokens.shape[0]

    @property
    def max_tokens(self) -> int:
        return self.tokens.shape[1]

    @property
    def max_stop_seq_len(self) -> int:
        return 0 if self.stop_tokens is None else self.stop_tokens.shape[2]

    @property
    def empty_queue_space(self) -> int:
        return self.tqueue.empty_queue_space

    @property
    def max_queued_tokens(self) -> int:
        return self.tqueue.max_queued_tokens

    @property
    def num_queued_tokens(self) -> int:
        return self.tqueue.num_queued_tokens

    # -- per-sequence RNG -------------------------------------------------------------------------------------
    def prng_key_for(self, slot_id: int, pos_id: int) -> int:
        return int(self.prng_keys_for(np.array([slot_id]), np.array([pos_id]))[0])

    def prng_keys_for(self, slot_ids, pos_ids) -> np.ndarray:
        """One 63-bit seed per (sequence key, position): sampling a position twice gives the same token whatever else is
        in the batch (src/levanter/inference/jit_scheduler.py:141-156)."""
        s = np.clip(_np(slot_ids).astype(np.int64), 0, self.max_seqs - 1)
        k = self.prng_keys[s].astype(np.uint64)
        p = _np(pos_ids).astype(np.uint64)
        with np.errstate(over="ignore"):
            z = k * np.uint64(0x9E3779B97F4A7C15) + p * np.uint64(0xBF58476D1CE4E5B9) + np.uint64(0x94D049BB133111EB)
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            z = z ^ (z >> np.uint64(31))
        return (z & np.uint64(0x7FFFFFFFFFFFFFFF)).astype(np.int64)

    # -- queue passthrough ------------------------------------------------------------------------------------
    def enqueue_tokens(self, new_tokens, new_slot_ids, new_pos_ids, num_new_tokens: int) -> "DecodeState":
        self.tqueue = self.tqueue.enqueue_tokens(new_tokens, new_slot_ids, new_pos_ids, num_new_tokens)
        return self

    def purge_queue_of_slot(self, slot_id) -> "DecodeState":
        self.tqueue = self.tqueue.purge_queue_of_slot(slot_id)
        return self

    def pack_next_sequence(self, max_tokens: int) -> Tuple["DecodeState", PackedSequence]:
        self.tqueue, packed = self.tqueue.pack_next_sequence(max_tokens)
        return self, packed

    # -- slots ------------------------------------------------------------------------------------------------
    def invalidate_finished(self) -> "DecodeState":
        m = self.finished
        self.seq_lens[m] = INVALID
        self.clone_sources[m] = INVALID
        self.kv_pages[m] = INVALID
        self.finished = np.zeros_like(self.finished)
        return self

    def discharge_clone(self, target_slot_ids, num_targets: int) -> "DecodeState":
        for t in _np(target_slot_ids)[:int(num_targets)]:
            if is_valid(t):
                self.clone_sources[int(t)] = INVALID
        return self

    def assign_seq(self, local_slot_id: int, tokens, seq_len: int, kv_pages=None, seq_params: Optional[SeqDecodingParams] = None) -> "DecodeState":
        s = int(local_slot_id)
        toks = _np(tokens).astype(np.int32)
        self.tokens[s, :len(toks)] = toks
        self.kv_pages[s] = INVALID if kv_pages is None else _np(kv_pages)
        if self.logprobs is not None:
            self.logprobs[s, :] = np.nan
        self.seq_lens[s] = int(seq_len)
        self.finished[s] = False
        if seq_params is not None:
            self.max_num_tokens[s] = int(min(seq_params.max_num_tokens, np.iinfo(np.int32).max))
            self.temperature[s] = float(seq_params.temperature)
            self.prng_keys[s] = np.uint64(int(seq_params.key) & 0xFFFFFFFFFFFFFFFF)
            if self.stop_tokens is None:
                if seq_params.stop_tokens is not None:
                    raise ValueError("DecodeState was initialized without stop token storage")
            else:
                self.stop_tokens[s] = INVALID
                if seq_params.stop_tokens is not None:
                    st = np.atleast_2d(_np(seq_params.stop_tokens)).astype(np.int32)
                    n, L = st.shape
                    if n > self.stop_tokens.shape[1] or L > self.stop_tokens.shape[2]:
                        raise ValueError(f"stop sequences [{n}, {L}] exceed the configured capacity {self.stop_tokens.shape[1:]}")
                    if n and L:
                        self.stop_tokens[s, :n, -L:] = st
        return self

    def update_tokens(self, new_tokens, local_slot_ids, new_log_probs, num_new_tokens: int, enqueue: bool = True) -> "DecodeState":
        """Append sampled tokens to their sequences, detect stop sequences / length limits, and queue the tokens of
        sequences that go on (finished ones are not fed back).  ``enqueue=False`` is for tokens the device has already fed
        into its next round."""
        toks, slots = _np(new_tokens), _np(local_slot_ids)
        lps = None if new_log_probs is None else _np(new_log_probs)
        n = int(num_new_tokens)
        pos_ids = np.full(len(toks), INVALID, dtype=np.int32)
        purge_mask = np.ones(len(toks), dtype=bool)
        sl = np.asarray(slots[:n]).astype(np.int64)
        in_range = (sl >= 0) & (sl < self.max_seqs)
        if n > 0 and len(np.unique(sl[in_range])) == int(in_range.sum()):
            # one token per sequence (every decode round): all sequences at once
            idx = np.nonzero(in_range)[0]
            sid = sl[idx]
            pos = self.seq_lens[sid].astype(np.int64)
            over = pos >= self.max_tokens
            self.finished[sid[over]] = True
            idx, sid, pos = idx[~over], sid[~over], pos[~over]
            self.tokens[sid, pos] = toks[idx]
            if self.logprobs is not None and lps is not None:
                self.logprobs[sid, pos] = lps[idx]
            self.seq_lens[sid] = pos + 1
            done = (pos + 1) >= self.max_num_tokens[sid]
            if self.stop_tokens is not None and self.stop_tokens.shape[1] > 0 and len(sid):
                stops = self.stop_tokens[sid]                      # [m, stop_seq, L], left padded with INVALID
                valid = is_valid(stops)
                if valid.any():
                    L = stops.shape[2]
                    at = pos[:, None] + 1 - L + np.arange(L)[None, :]
                    tail = np.where(at >= 0, self.tokens[sid[:, None], np.clip(at, 0, None)], INVALID)[:, None, :]
                    match = ((tail == stops) & (tail != INVALID)).sum(axis=-1) == valid.sum(axis=-1)
                    done = done | (valid.any(axis=-1) & match).any(axis=-1)
            self.finished[sid] = done
            purge_mask[idx] = done
            pos_ids[idx] = pos
        else:
            for i in range(n):
                sid = int(slots[i])
                if not (0 <= sid < self.max_seqs):
                    continue
                pos = int(self.seq_lens[sid])
                if pos >= self.max_tokens:
                    self.finished[sid] = True
                    continue
                self.tokens[sid, pos] = toks[i]
                if self.logprobs is not None and lps is not None:
                    self.logprobs[sid, pos] = lps[i]
                self.seq_lens[sid] = pos + 1
                done = (pos + 1) >= int(self.max_num_tokens[sid])
                if not done and self.stop_tokens is not None and self.stop_tokens.shape[1] > 0:
                    L = self.stop_tokens.shape[2]
                    row = self.tokens[sid, max(0, pos + 1 - L):pos + 1]
                    tail = np.concatenate([np.full(L - len(row), INVALID, dtype=np.int32), row])
                    done = is_stop_signal(tail, self.stop_tokens[sid])
                self.finished[sid] = done
                purge_mask[i] = done
                pos_ids[i] = pos
        if enqueue:
            keep = ~purge_mask
            self.tqueue = self.tqueue.enqueue_tokens(toks[keep], slots[keep], pos_ids[keep], int(keep.sum()))
        return self

    def is_finished(self, slot_id) -> np.ndarray:
        return self.finished[np.atleast_1d(_np(slot_id))]


@dataclass
class _DecodeOutputs:
    """Flat stream of (token, slot, logprob) produced by a decode call, plus the finished flags seen so far."""
    tokens: np.ndarray
    slot_ids: np.ndarray
    logprobs: Optional[np.ndarray]
    num_tokens: int
    finished: np.ndarray

    @property
    def max_queued_tokens(self) -> int:
        return self.tokens.shape[0]

    @property
    def empty_queue_space(self) -> int:
        return self.tokens.shape[0] - self.num_tokens

    @staticmethod
    def init(max_tokens: int, max_seqs: int, with_logprobs: bool = True) -> "_DecodeOutputs":
        return _DecodeOutputs(np.full(max_tokens, INVALID, np.int32), np.full(max_tokens, INVALID, np.int32),
                              np.full(max_tokens, np.nan, np.float32) if with_logprobs else None, 0, np.zeros(max_seqs, dtype=bool))

    def append(self, new_tokens, new_slot_ids, new_logprobs, num_new_tokens: int, finished_snapshot) -> "_DecodeOutputs":
        n = int(min(num_new_tokens, self.empty_queue_space))
        a = self.num_tokens
        self.tokens[a:a + n] = _np(new_tokens)[:n]
        self.slot_ids[a:a + n] = _np(new_slot_ids)[:n]
        if self.logprobs is not None and new_logprobs is not None:
            self.logprobs[a:a + n] = _np(new_logprobs)[:n]
        self.num_tokens = a + n
        self.finished = self.finished | _np(finished_snapshot).astype(bool)
        return self
