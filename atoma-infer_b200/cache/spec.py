"""What the parts and the cache tell each other: a mixer's need, a group of layers, a layer's view."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

FULL_KEYS, WINDOW_KEYS = 0, 1


@dataclass(frozen=True)
class CacheNeed:
    """What one mixer keeps per cached token: keys and values of ``num_kv_heads`` heads of
    ``head_dim``; ``window`` = how many keys a query looks back over (itself included),
    None for all of them."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    @property
    def kind(self) -> int:
        return FULL_KEYS if self.window is None else WINDOW_KEYS


@dataclass
class CacheGroup:
    need: CacheNeed
    layers: List[int] = field(default_factory=list)  # model layer indices that own a cache here
    num_pages: int = 0  # pool size, page 0 (never handed out) included


@dataclass
class LayerCache:
    """What one layer run sees of the cache."""

    group: int = -1                            # cache group of the layer, -1: none
    pages: Optional[torch.Tensor] = None       # [num_pages, 2, kv_heads, page_size, head_dim]
    num_pages: int = 0
    page_size: int = 0
    writes: bool = True                        # False when the run reads another layer's cache
    state: Optional[torch.Tensor] = None       # [max_seqs, state_bytes] uint8, the layer's per-request state


