"""Device memory of the cache: pages of keys and values per group, state slots per layer.

One tensor per cache group, ``[layers_in_group, num_pages, 2, kv_heads, page_size,
head_dim]``: a page id addresses the same page in every layer of its group (a layer here is
a run of the model's schedule that owns a cache), and the
(page, K|V, head) block of page_size * head_dim elements is contiguous.  The
reference keeps ``[2, num_blocks, block_size, kv_heads, head_dim]`` per layer
(backends/vllm/src/worker.rs:592-595, models/src/flash_attention.rs:239-246); the
layout is private to the cache and the kernels.  The number of pages follows the
reference's arithmetic: memory budget / bytes per page over all layers
(backends/vllm/src/config.rs:626-641, 708-718).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .spec import CacheGroup, LayerCache


def page_bytes(group: CacheGroup, page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page id costs in its group, all layers of the group together."""
    elem = torch.empty((), dtype=dtype).element_size()
    return 2 * group.need.num_kv_heads * page_size * group.need.head_dim * elem * len(group.layers)


def pages_for_memory(groups: List[CacheGroup], page_size: int, dtype: torch.dtype, budget_bytes: int) -> int:
    """Pages per pool (the same for every pool) that fit the budget."""
    per = sum(page_bytes(g, page_size, dtype) for g in groups)
    return max(0, budget_bytes // per) if per else 0


class KVCache:
    def __init__(self, model, groups: List[CacheGroup], page_size: int, max_seqs: int, rt,
                 poison: bool = False):
        self.model, self.groups, self.page_size, self.rt = model, groups, page_size, rt
        self.pages: List[torch.Tensor] = []
        for g in groups:
            shape = (len(g.layers), g.num_pages, 2, g.need.num_kv_heads, page_size, g.need.head_dim)
            t = torch.empty(shape, dtype=rt.dtype, device=rt.device)
            # Poison: a key or value that is read without having been written shows as NaN.
            t.fill_(float("nan")) if poison else t.zero_()
            self.pages.append(t)
        self.state: Dict[int, torch.Tensor] = {  # by run of the model's schedule
            run: torch.zeros((max_seqs, nbytes), dtype=torch.uint8, device=rt.device)
            for run, nbytes in enumerate(model.state_bytes) if nbytes
        }

    def layer_view(self, owner: int, writes: bool = True, state_run: Optional[int] = None) -> LayerCache:
        """What a run sees: the pages of the run that owns its cache, and its own state."""
        state = self.state.get(owner if state_run is None else state_run)
        where = self.model.run_group.get(owner)
        if where is None:
            return LayerCache(group=-1, page_size=self.page_size, writes=False, state=state)
        gi, idx = where
        return LayerCache(group=gi, pages=self.pages[gi][idx], num_pages=self.groups[gi].num_pages,
                          page_size=self.page_size, writes=writes, state=state)

    def reset_state(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()
