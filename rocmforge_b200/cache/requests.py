"""What a mixer asks of the cache."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class KVRequest:
    """Keys and values of every position (window None) or of the last ``window`` positions."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self):
        return ("kv", self.n_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateRequest:
    """Per-sequence state of fixed size: {name: (shape, dtype)}; zero when a slot is handed out.

    dtype None means the model's compute dtype.
    """
    tensors: Tuple[Tuple[str, Tuple[int, ...], Optional[torch.dtype]], ...]

    @staticmethod
    def of(**named) -> "StateRequest":
        items = []
        for name, v in named.items():
            shape, dtype = v if isinstance(v, tuple) and len(v) == 2 and not isinstance(v[0], int) else (v, None)
            items.append((name, tuple(shape), dtype))
        return StateRequest(tuple(items))
