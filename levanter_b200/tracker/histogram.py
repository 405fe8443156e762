"""Histogram summaries of tensors (src/levanter/tracker/histogram.py:20-150).

``Histogram.from_array`` bins on the device; ``sharded_histogram`` bins a tensor whose shards live on several ranks: each
rank counts its shard against shared edges and the counts are summed with one all-reduce (the reference's only explicit
device collective, :119)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

NUM_BINS = 31


@dataclass
class Histogram:
    min: float
    max: float
    num: int
    sum: float
    sum_squares: float
    bucket_limits: np.ndarray
    bucket_counts: np.ndarray

    @staticmethod
    def from_array(array: torch.Tensor, num_bins: int = NUM_BINS, group: Optional[dist.ProcessGroup] = None,
                   sharded: bool = False) -> "Histogram":
        if array.is_cuda and array.numel() > 0 and num_bins <= 256 and not (sharded and dist.is_initialized()):
            from ..ops import analysis_kernels as ak
            from ..ops import lib

            if lib.available():
                # two reads of the tensor (summary, then bins over the range the summary left on the device), one read-back
                a = array.detach().reshape(-1)
                a = a if a.dtype in (torch.float32, torch.bfloat16) else a.float()
                summary, counts = ak.summary_and_histogram(a, num_bins)
                mn, mx, total, total_sq = summary.tolist()
                edges = np.linspace(mn, mx if mx > mn else mn + 1.0, num_bins + 1, dtype=np.float32)
                return Histogram(mn, mx, a.numel(), total, total_sq, edges, counts.cpu().numpy().astype(np.float32))
        a = array.detach().float().reshape(-1)
        stats = torch.stack([a.min() if a.numel() else torch.tensor(float("inf"), device=a.device),
                             -(a.max() if a.numel() else torch.tensor(-float("inf"), device=a.device))])
        sums = torch.stack([a.sum(), (a * a).sum(), torch.tensor(float(a.numel()), device=a.device)])
        if sharded and dist.is_initialized():
            dist.all_reduce(stats, op=dist.ReduceOp.MIN, group=group)
            dist.all_reduce(sums, group=group)
        mn, mx = float(stats[0]), float(-stats[1])
        counts, edges = sharded_histogram(a, bins=num_bins, range=(mn, mx), group=group if sharded else None, reduce=sharded)
        return Histogram(mn, mx, int(sums[2]), float(sums[0]), float(sums[1]), edges.cpu().numpy(), counts.cpu().numpy())

    def to_numpy_histogram(self):
        return np.asarray(self.bucket_counts), np.asarray(self.bucket_limits)


def sharded_histogram(a: torch.Tensor, bins: int = NUM_BINS, range=None, group=None, reduce: bool = True):
    """Counts of ``a`` in ``bins`` equal-width buckets over ``range``; counts are all-reduced over ``group``."""
    a = a.detach().float().reshape(-1)
    if range is None:
        lo, hi = (float(a.min()), float(a.max())) if a.numel() else (0.0, 1.0)
    else:
        lo, hi = range
    if not (hi > lo):
        hi = lo + 1.0
    edges = torch.linspace(lo, hi, bins + 1, device=a.device)
    if a.is_cuda and a.numel() > 0 and bins <= 256:
        from ..ops import analysis_kernels as ak
        from ..ops import lib

        if lib.available():
            counts = ak.histogram_counts(a, lo, hi, bins).to(torch.float32)
            if reduce and dist.is_available() and dist.is_initialized():
                dist.all_reduce(counts, group=group)
            return counts, edges
    idx = torch.clamp(((a - lo) / (hi - lo) * bins).floor().long(), 0, bins - 1)
    inside = (a >= lo) & (a <= hi)
    counts = torch.bincount(idx[inside], minlength=bins).to(torch.float32)
    if reduce and dist.is_available() and dist.is_initialized():
        dist.all_reduce(counts, group=group)
    return counts, edges
