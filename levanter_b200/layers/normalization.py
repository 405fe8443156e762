"""Normalisation configs selectable by ``type:`` (``rms`` | ``layer``; Gemma registers ``gemma``)
(src/levanter/layers/normalization.py:15-48)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..config import ChoiceRegistry


@dataclass(frozen=True)
class LayerNormConfigBase(ChoiceRegistry):
    eps: float = 1e-6
    use_weight: bool = True
    use_bias: bool = False

    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return "rms"

    def build(self, dim: int):
        raise NotImplementedError


@LayerNormConfigBase.register_subclass("rms")
@dataclass(frozen=True)
class RmsNormConfig(LayerNormConfigBase):
    def build(self, dim: int):
        from ..nn import RmsNorm

        return RmsNorm(dim, eps=self.eps, use_weight=self.use_weight, use_bias=self.use_bias)


@LayerNormConfigBase.register_subclass("layer")
@dataclass(frozen=True)
class LayerNormConfig(LayerNormConfigBase):
    eps: float = 1e-5
    use_bias: bool = True

    def build(self, dim: int):
        from ..nn import LayerNorm

        return LayerNorm(dim, eps=self.eps, use_weight=self.use_weight, use_bias=self.use_bias)
