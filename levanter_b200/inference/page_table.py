"""KV page table (src/levanter/inference/page_table.py:27-542): which pages belong to which sequence slot, with reference
counts so that clones can share full pages.

The table lives in host memory as int32 numpy arrays and is updated by the host C++ routines of ``csrc/page_table.cpp`` (a
numpy implementation with the same results is used when the native library is not available, and as the test oracle).  The
methods keep the reference's value semantics: they return a new ``PageTable`` and leave ``self`` untouched.  What the GPU
needs for one forward pass is the :class:`PageBatchInfo`, moved to the device in one pinned copy by ``to(device)``."""
from __future__ import annotations

import ctypes
import dataclasses
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from .utils import INVALID, is_valid

__all__ = ["PageTable", "PageBatchInfo"]

_I32P = ctypes.POINTER(ctypes.c_int32)
_U8P = ctypes.POINTER(ctypes.c_uint8)
_native = None
_native_tried = False


def _lib():
    """The native library, or None (no compiler / load failure): callers then use the numpy path."""
    global _native, _native_tried
    if not _native_tried:
        _native_tried = True
        try:
            from ..ops import lib as L

            l = L.load()
            l.lvb_pt_allocate.restype = ctypes.c_int
            l.lvb_pt_clone.restype = ctypes.c_int
            l.lvb_pt_free_finished.restype = None
            l.lvb_tq_pack_next.restype = ctypes.c_int
            _native = l
        except Exception:  # noqa: BLE001
            _native = None
    return _native


def _p(a: np.ndarray, tp=_I32P):
    return a.ctypes.data_as(tp)


def _relative_positions(seg_ids: np.ndarray) -> np.ndarray:
    """0, 1, 2, ... inside each run of equal ids."""
    seg_ids = np.asarray(seg_ids)
    idx = np.arange(len(seg_ids))
    is_start = np.concatenate([[True], seg_ids[1:] != seg_ids[:-1]])
    return idx - np.maximum.accumulate(idx * is_start)


@dataclass
class PageBatchInfo:
    """Pages and lengths of the sequences that have tokens in one forward pass.  Row ``i`` describes the ``i``-th distinct
    sequence of the packed tokens, not slot ``i``; ``slot_ids`` maps rows back to slots."""
    slot_ids: torch.Tensor  # i32[seq]
    page_indices: torch.Tensor  # i32[seq, page]
    seq_lens: torch.Tensor  # i32[seq]   (INVALID for unused rows)
    cu_q_lens: torch.Tensor  # i32[seq + 1]
    num_seqs: torch.Tensor  # i32[]
    new_token_dests: torch.Tensor  # i32[position]: page * page_size + slot of every packed token, or INVALID
    page_size: int
    prefill_segment_ids: Optional[torch.Tensor] = None
    """i32[position], set only when every packed sequence starts at position 0 (a pure prefill): the index of the sequence each
    token belongs to, -1 for padding.  Attention then needs no cached context and can run as dense causal attention over the
    packed tokens with these segment ids."""

    def pages_and_slots(self) -> Tuple[torch.Tensor, torch.Tensor]:
        d = self.new_token_dests
        ok = is_valid(d)
        inv = torch.full_like(d, INVALID)
        return torch.where(ok, d // self.page_size, inv), torch.where(ok, d % self.page_size, inv)

    def to(self, device, non_blocking: bool = True) -> "PageBatchInfo":
        mv = lambda t: t.to(device, non_blocking=non_blocking)  # noqa: E731
        return PageBatchInfo(mv(self.slot_ids), mv(self.page_indices), mv(self.seq_lens), mv(self.cu_q_lens), mv(self.num_seqs),
                             mv(self.new_token_dests), self.page_size,
                             None if self.prefill_segment_ids is None else mv(self.prefill_segment_ids))


@dataclass
class PageTable:
    page_indices: np.ndarray  # i32[seq, page]
    page_ref_counts: np.ndarray  # i32[page]
    seq_lens: np.ndarray  # i32[seq]
    used_mask: np.ndarray  # bool[seq]
    page_size: int

    # -- properties -------------------------------------------------------------------------------------------
    @property
    def num_pages(self) -> int:
        return self.page_ref_counts.shape[0]

    @property
    def pages_per_seq(self) -> int:
        return self.page_indices.shape[1]

    @property
    def max_seqs(self) -> int:
        return self.page_indices.shape[0]

    @property
    def max_len_per_seq(self) -> int:
        return self.page_size * self.pages_per_seq

    @property
    def current_num_seqs(self) -> int:
        return int(self.used_mask.sum())

    @property
    def num_free_pages(self) -> int:
        return int((self.page_ref_counts == 0).sum())

    @staticmethod
    def init(max_pages: int, max_seqs: int, page_size: int, max_pages_per_seq: int) -> "PageTable":
        return PageTable(np.full((max_seqs, max_pages_per_seq), INVALID, dtype=np.int32), np.zeros(max_pages, dtype=np.int32),
                         np.zeros(max_seqs, dtype=np.int32), np.zeros(max_seqs, dtype=bool), page_size)

    def _copy(self) -> "PageTable":
        return PageTable(self.page_indices.copy(), self.page_ref_counts.copy(), self.seq_lens.copy(), self.used_mask.copy(), self.page_size)

    # -- slots ------------------------------------------------------------------------------------------------
    def assign_seq_id_to_seq(self, seq_id: Optional[int] = None) -> Tuple["PageTable", int]:
        """Mark a slot used and return it: the given one when it is free, the lowest free one when ``seq_id`` is None or out
        of range.  Returns ``INVALID`` (table unchanged) when the requested slot is taken or none is free."""
        sid = INVALID if seq_id is None else int(seq_id)
        if 0 <= sid < self.max_seqs:
            if self.used_mask[sid]:
                return self, INVALID
        else:
            free = np.nonzero(~self.used_mask)[0]
            if len(free) == 0:
                return self, INVALID
            sid = int(free[0])
        new = self._copy()
        new.seq_lens[sid] = 0
        new.used_mask[sid] = True
        return new, sid

    # -- allocation -------------------------------------------------------------------------------------------
    def allocate_for_seq(self, token_slot_ids, token_pos_ids) -> Tuple["PageTable", PageBatchInfo]:
        """Reserve pages for packed tokens (tokens of a sequence contiguous) and describe the batch."""
        slots = np.ascontiguousarray(_np(token_slot_ids), dtype=np.int32)
        pos = np.ascontiguousarray(_np(token_pos_ids), dtype=np.int32)
        new = self._copy()
        S, P, n = self.max_seqs, self.pages_per_seq, len(slots)
        o_slot = np.empty(S, np.int32)
        o_pages = np.empty((S, P), np.int32)
        o_lens = np.empty(S, np.int32)
        o_cu = np.empty(S + 1, np.int32)
        o_dest = np.empty(n, np.int32)
        o_num = ctypes.c_int(0)
        lib = _lib()
        if lib is not None:
            used8 = new.used_mask.astype(np.uint8)
            rc = lib.lvb_pt_allocate(_p(new.page_indices), _p(new.page_ref_counts), _p(new.seq_lens), _p(used8, _U8P), S, P,
                                     self.num_pages, self.page_size, _p(slots), _p(pos), n, _p(o_slot), _p(o_pages), _p(o_lens),
                                     _p(o_cu), ctypes.byref(o_num), _p(o_dest))
            if rc != 0:
                raise RuntimeError("Out of free pages during allocation")
            num = o_num.value
        else:
            num = _allocate_numpy(new, slots, pos, o_slot, o_pages, o_lens, o_cu, o_dest)
        info = PageBatchInfo(torch.from_numpy(o_slot), torch.from_numpy(o_pages), torch.from_numpy(o_lens), torch.from_numpy(o_cu),
                             torch.tensor(num, dtype=torch.int32), torch.from_numpy(o_dest), self.page_size)
        return new, info

    # -- release ----------------------------------------------------------------------------------------------
    def free_pages(self, seq_id: int) -> "PageTable":
        if seq_id is None or seq_id < 0 or seq_id >= self.max_seqs:
            return self
        mask = np.zeros(self.max_seqs, dtype=bool)
        mask[int(seq_id)] = True
        return self.free_pages_for_finished(mask)

    def free_pages_for_finished(self, finished_mask) -> "PageTable":
        fm = np.ascontiguousarray(_np(finished_mask)).astype(np.uint8)
        assert fm.ndim == 1
        new = self._copy()
        lib = _lib()
        if lib is not None:
            used8 = new.used_mask.astype(np.uint8)
            lib.lvb_pt_free_finished(_p(new.page_indices), _p(new.page_ref_counts), _p(new.seq_lens), _p(used8, _U8P), self.max_seqs,
                                     self.pages_per_seq, _p(fm, _U8P))
            new.used_mask = used8.astype(bool)
        else:
            for s in np.nonzero(fm)[0]:
                for p in new.page_indices[s]:
                    if is_valid(p):
                        new.page_ref_counts[p] = max(new.page_ref_counts[p] - 1, 0)
                new.page_indices[s] = INVALID
                new.seq_lens[s] = 0
                new.used_mask[s] = False
        return new

    # -- clones -----------------------------------------------------------------------------------------------
    def increment_ref_counts_for_pages(self, pages, count: int = 1) -> "PageTable":
        new = self._copy()
        for p in _np(pages):
            if is_valid(p):
                new.page_ref_counts[int(p)] += count
        return new

    def clone_pages_from(self, src_seq_id: int, dst_seq_id: int) -> "PageTable":
        """``dst`` shares every full page of ``src``; if ``src`` ends inside a page, ``dst`` gets a fresh last page (its K/V
        must be copied by the caller, see :meth:`last_clone_copy`) so later writes of the two do not collide."""
        new = self._copy()
        lib = _lib()
        if lib is not None:
            used8 = new.used_mask.astype(np.uint8)
            rc = lib.lvb_pt_clone(_p(new.page_indices), _p(new.page_ref_counts), _p(new.seq_lens), _p(used8, _U8P), self.pages_per_seq,
                                  self.num_pages, self.page_size, int(src_seq_id), int(dst_seq_id))
            if rc == -5:
                raise RuntimeError("Out of free pages during clone_pages_from")
            new.used_mask = used8.astype(bool)
            return new
        src_len = int(new.seq_lens[src_seq_id])
        used_pages = (src_len + self.page_size - 1) // self.page_size
        boundary = src_len % self.page_size == 0
        new.page_indices[dst_seq_id] = new.page_indices[src_seq_id]
        for p in new.page_indices[src_seq_id][:used_pages - (0 if boundary else 1)]:
            if is_valid(p):
                new.page_ref_counts[p] += 1
        if not boundary:
            free = np.nonzero(new.page_ref_counts == 0)[0]
            if len(free) == 0:
                raise RuntimeError("Out of free pages during clone_pages_from")
            new.page_indices[dst_seq_id, max(used_pages - 1, 0)] = free[0]
            new.page_ref_counts[free[0]] += 1
        new.seq_lens[dst_seq_id] = src_len
        new.used_mask[dst_seq_id] = True
        return new

    def bump_seq_len_to_next_page(self, seq_id: int) -> "PageTable":
        new = self._copy()
        cur = int(new.seq_lens[seq_id])
        new.seq_lens[seq_id] = ((cur + self.page_size - 1) // self.page_size) * self.page_size
        return new


def _np(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    return np.asarray(x)


def _allocate_numpy(t: PageTable, slots, pos, o_slot, o_pages, o_lens, o_cu, o_dest) -> int:
    S, P = t.max_seqs, t.pages_per_seq
    o_slot[:] = INVALID
    o_pages[:] = INVALID
    o_lens[:] = INVALID
    o_dest[:] = INVALID
    order, counts, max_pos = [], {}, {}
    pad = 0
    for s, p in zip(slots.tolist(), pos.tolist()):
        if s < 0 or s >= S:
            pad += 1
            continue
        if s not in counts:
            order.append(s)
            counts[s], max_pos[s] = 0, -1
        counts[s] += 1
        if is_valid(p):
            max_pos[s] = max(max_pos[s], p)
    num = len(order)
    cu = [0]
    for d in range(S):
        cu.append(cu[-1] + (counts[order[d]] if d < num else (pad if d == num else 0)))
    o_cu[:] = cu
    for d, s in enumerate(order):
        o_slot[d] = s
        if not t.used_mask[s]:
            continue
        old = int(t.seq_lens[s])
        new = max(old, max_pos[s] + 1)
        t.seq_lens[s] = new
        for p in range((old + t.page_size - 1) // t.page_size, min((new + t.page_size - 1) // t.page_size, P)):
            free = np.nonzero(t.page_ref_counts == 0)[0]
            if len(free) == 0:
                raise RuntimeError("Out of free pages during allocation")
            t.page_ref_counts[free[0]] += 1
            t.page_indices[s, p] = free[0]
    for d, s in enumerate(order):
        o_pages[d] = t.page_indices[s]
        o_lens[d] = t.seq_lens[s]
    for i, (s, p) in enumerate(zip(slots.tolist(), pos.tolist())):
        if 0 <= s < S and is_valid(p) and p // t.page_size < P:
            page = t.page_indices[s, p // t.page_size]
            if is_valid(page):
                o_dest[i] = page * t.page_size + p % t.page_size
    return num
