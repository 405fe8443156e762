"""Distributions of the model's predictive entropy and of the gap between its two most likely tokens
(src/levanter/analysis/entropy.py:31-232), logged as histograms."""
from __future__ import annotations

import logging
from typing import Callable, Optional

import torch

from .. import tracker as trk
from ..callbacks import StepInfo
from ..tracker.histogram import Histogram

logger = logging.getLogger(__name__)


def entropy_from_logits(logits: torch.Tensor, axis: int = -1) -> torch.Tensor:
    """``H = logsumexp(z) - sum(softmax(z) * z)`` in fp32 (one streaming pass over the logits on a B200)."""
    if logits.is_cuda and axis in (-1, logits.dim() - 1):
        from ..ops.analysis_kernels import entropy_top2

        return entropy_top2(logits)[0]
    z = logits.float()
    lse = torch.logsumexp(z, dim=axis, keepdim=True)
    p = torch.exp(z - lse)
    return lse.squeeze(axis) - (p * z).sum(dim=axis)


def top2_gap_from_logits(logits: torch.Tensor, axis: int = -1) -> torch.Tensor:
    """Difference between the largest and the second largest logit."""
    if logits.is_cuda and axis in (-1, logits.dim() - 1):
        from ..ops.analysis_kernels import entropy_top2

        return entropy_top2(logits)[1]
    top = torch.topk(logits.float(), 2, dim=axis).values
    a, b = top.unbind(dim=axis)
    return a - b


def _histogram_over(model, logit_fn: Callable, test_data, reduce_fn: Callable, max_tokens: int, num_bins: int) -> Histogram:
    vals = []
    total = 0
    device = next(model.parameters()).device
    was_training = model.training
    model.eval()
    try:
        with torch.no_grad():
            for batch in test_data:
                batch = batch.to(device) if hasattr(batch, "to") else batch
                v = reduce_fn(logit_fn(model, batch)).reshape(-1)
                vals.append(v)
                total += v.numel()
                if total >= max_tokens:
                    break
    finally:
        model.train(was_training)
    if not vals or total == 0:
        raise ValueError("No tokens processed")
    return Histogram.from_array(torch.cat(vals), num_bins=num_bins)


def compute_entropy_histogram(model, Vocab, logit_fn, test_data, max_tokens: int = 1024 * 1024, num_bins: int = 64) -> Histogram:
    return _histogram_over(model, logit_fn, test_data, entropy_from_logits, max_tokens, num_bins)


def compute_top2_gap_histogram(model, Vocab, logit_fn, test_data, max_tokens: int = 1024 * 1024, num_bins: int = 64) -> Histogram:
    return _histogram_over(model, logit_fn, test_data, top2_gap_from_logits, max_tokens, num_bins)


def _cb(kind: str, fn, logit_fn, Vocab, test_data, prefix: Optional[str], batch_size: int, mapping, num_tokens: int):
    prefix = prefix or "analysis"

    def hook(step: StepInfo):
        from ..data.loader import DataLoader

        loader = DataLoader(test_data, batch_size, pad_final_batch=False, max_buffered_batches=0)
        try:
            hist = fn(model=step.eval_model, Vocab=Vocab, logit_fn=logit_fn, test_data=loader, max_tokens=num_tokens)
        except ValueError as e:
            if "No tokens processed" in str(e):
                logger.warning(f"{prefix} is too small to compute {kind} with batch size {batch_size}")
                return
            raise
        trk.log({f"{prefix}/{kind}": hist}, step=step.step)

    return hook


def cb_compute_entropies(logit_fn, Vocab, test_data, prefix: Optional[str], batch_size: int, mapping=None, num_tokens: int = 10 * 1024 * 1024):
    return _cb("entropy", compute_entropy_histogram, logit_fn, Vocab, test_data, prefix, batch_size, mapping, num_tokens)


def cb_compute_top2_gap(logit_fn, Vocab, test_data, prefix: Optional[str], batch_size: int, mapping=None, num_tokens: int = 10 * 1024 * 1024):
    return _cb("top2_gap", compute_top2_gap_histogram, logit_fn, Vocab, test_data, prefix, batch_size, mapping, num_tokens)
