"""What a mixer asks of the cache."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class KVRequest:
    """Keys and values of every position (window and chunk None), of the last ``window`` positions, or of the chunk of
    ``chunk`` positions that the newest position lies in (chunks counted from position 0).  ``keep_first``: with a window,
    the sequence's first ``keep_first`` positions are kept for good as well.  ``values_are_keys``: the mixer's values are
    its keys as cached, so the pages hold keys alone and the view's value pages are the key pages."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None      # size of a value head where it differs from a key head's
    chunk: Optional[int] = None
    keep_first: int = 0
    values_are_keys: bool = False

    def __post_init__(self):
        if self.values_are_keys and self.v_head_dim is not None and self.v_head_dim != self.head_dim:
            raise ValueError("keys that serve as values have one size")
        if self.window and self.chunk:
            raise ValueError("a cache request keeps a window or a chunk, not both")
        if self.keep_first < 0 or (self.keep_first and not self.window):
            raise ValueError("a cache request keeps first positions beside a window only")

    def group_key(self):
        return ("kv", self.n_kv_heads, self.head_dim, self.window, self.v_head_dim, self.chunk, self.keep_first,
                self.values_are_keys)

    def first_needed(self, position: int) -> int:
        """The first key position that a query at ``position`` (and therefore any later one) can see."""
        if self.window:
            return max(position - self.window + 1, 0)
        if self.chunk:
            return position // self.chunk * self.chunk
        return 0


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
