"""JSON encoder for config trees (src/levanter/utils/json_utils.py:9-17)."""
import enum
import json
from dataclasses import asdict, is_dataclass
from datetime import timedelta

import torch


class ConfigJSONEncoder(json.JSONEncoder):
    def default(self, o):
        if isinstance(o, enum.Enum):
            return o.name
        if isinstance(o, torch.dtype):
            return str(o).replace("torch.", "")
        if isinstance(o, timedelta):
            return o.total_seconds()
        if is_dataclass(o) and not isinstance(o, type):
            return asdict(o)
        if isinstance(o, (set, frozenset)):
            return sorted(o)
        try:
            return super().default(o)
        except TypeError:
            return str(o)
