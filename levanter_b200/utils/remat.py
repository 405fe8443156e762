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

    @staticmethod
    def from_bool_or_str(remat) -> "ScanCheckpointPolicy":
        if isinstance(remat, ScanCheckpointPolicy):
            return remat
        if remat is True or remat == "full":
            return ScanCheckpointPolicy(save_carries=True)
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


def should_recompute(gc) -> bool:
    if isinstance(gc, ScanCheckpointPolicy):
        return gc.recompute
    if isinstance(gc, dict):
        return not gc.get("disable", False)
    return ScanCheckpointPolicy.from_bool_or_str(gc).recompute
