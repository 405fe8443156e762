"""Watch hook: norms and histograms of gradients, parameters, updates and optimizer state every ``interval`` steps
(src/levanter/callbacks/watch.py:24-175)."""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from .. import tracker as trk
from ..analysis.tree_stats import summary_statistics_for_tree
from ._core import JitCallback, StepInfo

VALID_TARGETS = ("grads", "params", "opt_state", "updates")


class WatchCallback(JitCallback):
    def __init__(self, config):
        targets = config.watch_targets
        if isinstance(targets, str):
            targets = [t.strip() for t in targets.split(",")]
        for t in targets:
            if t not in VALID_TARGETS:
                raise ValueError(f"Invalid watch target: {t}. Valid targets are: {VALID_TARGETS}")
        self.watch_targets: List[str] = list(targets)
        self.include_norms = config.include_norms
        self.include_per_parameter_norms = config.include_per_parameter_norms
        self.include_histogram = config.include_histograms
        self.split_scan_layers = config.split_scan_layers

    @property
    def wants_updates(self) -> bool:
        return "updates" in self.watch_targets

    def _stats_kwargs(self, engine) -> Dict[str, Any]:
        group = engine.data_group if (engine.world > 1 and engine.shard_optimizer) else None
        sharded = group is not None
        return dict(split_scan_layers=self.split_scan_layers, include_histogram=self.include_histogram,
                    include_norms=self.include_norms, include_per_parameter_norms=self.include_per_parameter_norms,
                    group=group, sharded=sharded, all_names=[s.name for s in engine.slots] if sharded else None)

    def after_update(self, state, engine, cb_info: Dict[str, Any]) -> Dict[str, Any]:
        # the change the optimizer made to the weights in this step: learning rate and weight decay included
        cb_info.update(summary_statistics_for_tree("updates", engine.last_updates, **self._stats_kwargs(engine)))
        return cb_info

    def inside_step(self, state, engine) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        kw = self._stats_kwargs(engine)
        if "grads" in self.watch_targets:
            # gradients in the accumulator are not yet reduced over data ranks at this point; use local full grads
            g = {s.name: s.param.main_grad for s in engine.slots if getattr(s.param, "main_grad", None) is not None}
            out.update(summary_statistics_for_tree("grad", g, **{**kw, "group": None, "sharded": False, "all_names": None}))
        if "params" in self.watch_targets:
            out.update(summary_statistics_for_tree("params", engine.master_tree(), **kw))
        if "opt_state" in self.watch_targets and engine.opt_state is not None:
            from ..parallel.engine import _is_param_tree

            def walk(x, p):
                if _is_param_tree(x):
                    out.update(summary_statistics_for_tree(f"opt_state/{p}" if p else "opt_state", x, **kw))
                elif isinstance(x, tuple) and hasattr(x, "_fields"):
                    for f in x._fields:
                        walk(getattr(x, f), f"{p}/{f}" if p else f)
                elif isinstance(x, (tuple, list)):
                    for i, v in enumerate(x):
                        walk(v, f"{p}/{i}" if p else str(i))
                elif isinstance(x, dict):
                    for k, v in x.items():
                        walk(v, f"{p}/{k}" if p else str(k))

            walk(engine.opt_state, "")
        return out

    def on_step(self, step_info: StepInfo, cb_info: Dict[str, Any]):
        trk.log(cb_info, step=step_info.step)
