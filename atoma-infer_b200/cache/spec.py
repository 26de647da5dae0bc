"""What the parts and the cache tell each other: a mixer's need, a group of layers, a layer's view."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

FULL_KEYS, WINDOW_KEYS = 0, 1


@dataclass(frozen=True)
class CachedTensor:
    """One thing a mixer keeps per cached token: ``heads`` vectors of ``width`` elements."""

    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class CacheNeed:
    """What one mixer keeps per cached token: a tuple of named tensors, each ``[heads, width]``.  Keys and
    values of attention are the instance ``CacheNeed.kv(num_kv_heads, head_dim)``; a mixer that caches one
    latent vector, or keys and values of different widths, names its own.  ``window`` = how many cached tokens
    a query looks back over (itself included), None for all of them; pages a window has passed go back to
    the pool."""

    tensors: Tuple[CachedTensor, ...]
    window: Optional[int] = None

    @staticmethod
    def kv(num_kv_heads: int, head_dim: int, window: Optional[int] = None) -> "CacheNeed":
        return CacheNeed((CachedTensor("k", num_kv_heads, head_dim), CachedTensor("v", num_kv_heads, head_dim)), window)

    @property
    def kind(self) -> int:
        return FULL_KEYS if self.window is None else WINDOW_KEYS

    @property
    def elements_per_token(self) -> int:
        return sum(t.heads * t.width for t in self.tensors)

    @property
    def is_kv(self) -> bool:
        """Keys and values of one shape: the layout the attention kernels read."""
        t = self.tensors
        return len(t) == 2 and (t[0].name, t[1].name) == ("k", "v") and (t[0].heads, t[0].width) == (t[1].heads, t[1].width)

    # the two sizes of a keys-and-values need, as the attention kernels name them
    @property
    def num_kv_heads(self) -> int:
        return self.tensors[0].heads

    @property
    def head_dim(self) -> int:
        return self.tensors[0].width


@dataclass
class CacheGroup:
    need: CacheNeed
    layers: List[int] = field(default_factory=list)  # model layer indices that own a cache here
    num_pages: int = 0  # pool size, page 0 (never handed out) included


@dataclass
class LayerCache:
    """What one layer run sees of the cache."""

    group: int = -1                            # cache group of the layer, -1: none
    pages: Optional[torch.Tensor] = None       # keys and values: [num_pages, 2, kv_heads, page_size, head_dim];
                                               # any other need: [num_pages, elements of a page], see ``tensors``
    num_pages: int = 0
    page_size: int = 0
    writes: bool = True                        # False when the run reads another layer's cache
    state: Optional[torch.Tensor] = None       # [max_seqs, state_bytes] uint8, the layer's per-request state
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)  # name -> view [num_pages, heads, page_size, width]
