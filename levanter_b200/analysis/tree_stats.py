"""Per-parameter norms and histograms of a parameter-shaped tree (src/levanter/analysis/tree_stats.py:17-102)."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..optim.config import levanter_path
from ..tracker.histogram import Histogram


def summary_statistics_for_tree(prefix: str, tree: Dict[str, Optional[torch.Tensor]], split_scan_layers: bool = True,
                                include_histogram: bool = False, include_norms: bool = True,
                                include_per_parameter_norms: bool = True, group=None, sharded: bool = False,
                                all_names=None) -> Dict[str, Any]:
    """Metrics ``<prefix>/norm/<path>``, ``<prefix>/norm/total`` and ``<prefix>/hist/<path>``.  With
    ``split_scan_layers`` every layer gets its own entry (``.../layers/3/...``); otherwise layers are aggregated under
    the stacked path.  ``sharded`` trees hold local slices: squared norms and histogram counts are summed over ``group``.
    A rank of a sharded run holds slices of only some leaves, so ``all_names`` (the same list, in the same order, on every
    rank) fixes what the collectives range over; a leaf this rank has no part of contributes zero."""
    out: Dict[str, Any] = {}
    if sharded and all_names is not None:
        names = list(all_names)
        proto = next((v for v in tree.values() if v is not None), None)
        empty = torch.zeros(0, device=proto.device if proto is not None else None)
        tree = {k: (tree[k] if tree.get(k) is not None else empty) for k in names}
    else:
        names = [k for k, v in tree.items() if v is not None]
    if not names:
        return out
    if include_norms:
        sq = torch.stack([(tree[k].float() ** 2).sum() for k in names])
        if sharded and dist.is_initialized():
            dist.all_reduce(sq, group=group)
        keyed: Dict[str, torch.Tensor] = {}
        for k, v in zip(names, sq):
            key = k if split_scan_layers else levanter_path(k)
            keyed[key] = keyed.get(key, 0) + v
        if include_per_parameter_norms:
            for key, v in keyed.items():
                out[f"{prefix}/norm/{key.replace('.', '/')}"] = torch.sqrt(v)
        out[f"{prefix}/norm/total"] = torch.sqrt(sq.sum())
    if include_histogram:
        for k in names:
            key = k if split_scan_layers else levanter_path(k)
            out[f"{prefix}/hist/{key.replace('.', '/')}"] = Histogram.from_array(tree[k], group=group, sharded=sharded)
    return out
