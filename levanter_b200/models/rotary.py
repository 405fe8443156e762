"""Former home of the rotary embeddings; they live in :mod:`levanter_b200.layers.rotary` (src/levanter/models/rotary.py)."""
import warnings

from ..layers.rotary import *  # noqa: F401,F403

warnings.warn("levanter_b200.models.rotary is deprecated; import levanter_b200.layers.rotary", DeprecationWarning, stacklevel=2)
