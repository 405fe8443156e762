"""Activation-checkpointing policy accepted by ``gradient_checkpointing:`` in model configs
(bool | str | mapping; the reference's ``ScanCheckpointPolicy`` codec, src/levanter/config.py:56-70)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Union


@dataclass(frozen=True)
class ScanCheckpointPolicy:
    """``save_carries``: keep each layer's input and recompute the inside of the layer in backward.
    ``disable``: keep everything (no recompute).  ``nested``/``offload`` variants of the reference are accepted and
    map onto per-layer recompute; ``save_block_internals`` names activations to keep anyway."""

    save_carries: Union[bool, str] = True
    save_inputs: Union[bool, str] = False
    save_block_internals: Union[bool, list] = False
    prevent_cse: bool = False
    disable: bool = False
    simple: bool = False
    nested: Union[bool, int] = False
    recompute_attention: bool = False
    """by default the flash-attention outputs of a checkpointed layer are kept (see ``checkpoint_layer``); True recomputes them too"""

    @staticmethod
    def from_bool_or_str(remat) -> "ScanCheckpointPolicy":
        if isinstance(remat, ScanCheckpointPolicy):
            return remat
        if remat is True:
            return ScanCheckpointPolicy(save_carries=True)
        if remat == "full":  # recompute everything inside the layer, attention included
            return ScanCheckpointPolicy(save_carries=True, save_block_internals=False, recompute_attention=True)
        if remat is False or remat is None:
            return ScanCheckpointPolicy(disable=True)
        if isinstance(remat, str):
            key = remat.lower()
            if key in ("true", "recompute", "simple"):
                return ScanCheckpointPolicy(save_carries=True, simple=key == "simple")
            if key in ("false", "none", "disable"):
                return ScanCheckpointPolicy(disable=True)
            if key == "offload":
                return ScanCheckpointPolicy(save_carries="offload")
            if key in ("save_all", "everything"):
                return ScanCheckpointPolicy(disable=True)
            if key == "nested":
                return ScanCheckpointPolicy(nested=True)
            raise ValueError(f"unknown gradient_checkpointing policy {remat!r}")
        raise ValueError(f"cannot interpret gradient_checkpointing={remat!r}")

    @staticmethod
    def from_config_value(v):
        return ScanCheckpointPolicy.from_bool_or_str(v)

    @property
    def recompute(self) -> bool:
        return not self.disable


def keeps_attention(gc) -> bool:
    """Whether checkpointed layers keep their attention outputs (the default) under the policy ``gc``."""
    if isinstance(gc, dict):
        return not gc.get("recompute_attention", False)
    try:
        return not ScanCheckpointPolicy.from_bool_or_str(gc).recompute_attention
    except ValueError:
        return True


def should_recompute(gc) -> bool:
    if isinstance(gc, ScanCheckpointPolicy):
        return gc.recompute
    if isinstance(gc, dict):
        return not gc.get("disable", False)
    return ScanCheckpointPolicy.from_bool_or_str(gc).recompute


# --------------------------------------------------------------------------------------------- layer checkpointing
def checkpoint_layer(fn, *args, keep_attention: bool = True):
    """Run ``fn(*args)`` keeping only its inputs and recompute its inside during backward, like
    ``torch.utils.checkpoint``, except that the outputs of the flash-attention kernel (attention output and log-sum-exp)
    of the first pass are kept and handed to the recomputation instead of being computed again.  Attention is the one part
    of a transformer layer whose recomputation is expensive relative to what it would cost to keep: its output is one
    ``[tokens, hidden]`` tensor per layer, its forward is a quarter of the layer's FLOPs at long sequence lengths.
    ``keep_attention=False`` (or a pass in which nothing requires gradients) gives plain recomputation."""
    import torch

    if not torch.is_grad_enabled():
        return fn(*args)
    if not keep_attention or not any(isinstance(a, torch.Tensor) and a.requires_grad for a in args):
        # (a custom autograd function only produces a differentiable output when one of its tensor inputs requires gradients;
        # with frozen embeddings, as under LoRA, the first layer's input does not, although parameters inside the layer do)
        from torch.utils.checkpoint import checkpoint

        return checkpoint(fn, *args, use_reentrant=False)
    return _KeepAttentionCheckpoint.apply(fn, *args)


def _rng_snapshot():
    import torch

    cuda = torch.cuda.get_rng_state() if torch.cuda.is_available() and torch.cuda.is_initialized() else None
    return torch.get_rng_state(), cuda


class _RestoredRng:
    """Run a block under a saved RNG state and put the current one back afterwards (dropout masks repeat in the recomputation)."""

    def __init__(self, snap):
        self.snap = snap

    def __enter__(self):
        import torch

        self.outer = _rng_snapshot()
        torch.set_rng_state(self.snap[0])
        if self.snap[1] is not None:
            torch.cuda.set_rng_state(self.snap[1])

    def __exit__(self, *exc):
        import torch

        torch.set_rng_state(self.outer[0])
        if self.outer[1] is not None:
            torch.cuda.set_rng_state(self.outer[1])
        return False


def _make_checkpoint_function():
    import torch

    from ..ops import _flash_impl

    class KeepAttentionCheckpoint(torch.autograd.Function):
        @staticmethod
        def forward(ctx, fn, *args):
            ctx.fn = fn
            ctx.is_tensor = [isinstance(a, torch.Tensor) for a in args]
            ctx.other = [None if t else a for a, t in zip(args, ctx.is_tensor)]
            ctx.save_for_backward(*[a for a in args if isinstance(a, torch.Tensor)])
            ctx.rng = _rng_snapshot()
            kept = []
            with torch.no_grad(), _flash_impl.keeping_outputs(kept):
                out = fn(*args)
            ctx.kept = kept
            if not isinstance(out, torch.Tensor):
                raise TypeError("checkpoint_layer expects a function that returns one tensor")
            return out

        @staticmethod
        def backward(ctx, grad_out):
            saved = list(ctx.saved_tensors)
            inputs = []
            for t, other in zip(ctx.is_tensor, ctx.other):
                if t:
                    x = saved.pop(0)
                    x = x.detach().requires_grad_(x.is_floating_point())
                    inputs.append(x)
                else:
                    inputs.append(other)
            with torch.enable_grad(), _RestoredRng(ctx.rng), _flash_impl.replaying_outputs(ctx.kept):
                out = ctx.fn(*inputs)
            ctx.kept = None
            torch.autograd.backward(out, grad_out)
            grads = [x.grad if (t and isinstance(x, torch.Tensor) and x.requires_grad) else None for x, t in zip(inputs, ctx.is_tensor)]
            return (None, *grads)

    return KeepAttentionCheckpoint


class _LazyFunction:
    """Defers the import of torch and of the kernel bindings until the first use."""

    _cls = None

    @classmethod
    def apply(cls, *args):
        if cls._cls is None:
            cls._cls = _make_checkpoint_function()
        return cls._cls.apply(*args)


_KeepAttentionCheckpoint = _LazyFunction
