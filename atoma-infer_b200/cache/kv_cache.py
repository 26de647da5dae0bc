"""Device memory of the cache: pages per group, state slots per layer.

One tensor per cache group, ``[layers_in_group, num_pages, elements of a page]``: a page id addresses
the same page in every layer of its group (a layer here is a run of the model's schedule that owns a
cache).  Inside a page the named tensors of the group's need follow one another, each as
``[heads, page_size, width]``, so that a (page, tensor, head) block of page_size * width elements is
contiguous; for keys and values that is ``[num_pages, 2, kv_heads, page_size, head_dim]``, which the
attention kernels read.  The
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
    return group.need.elements_per_token * page_size * elem * len(group.layers)


def state_bytes_total(model, max_seqs: int) -> int:
    """Bytes of the fixed-size per-request state of all layer runs, for ``max_seqs`` slots."""
    return max_seqs * sum(int(n) for n in model.state_bytes)


def pages_for_memory(groups: List[CacheGroup], page_size: int, dtype: torch.dtype, free_bytes: int,
                     gpu_memory_utilization: float, state_bytes: int = 0, workspace_bytes: int = 0):
    """Pages per pool (the same for every pool) from the memory that is free once the weights are loaded:
    floor(free * utilization) / bytes per page over all layers, the reference's arithmetic
    (backends/vllm/src/config.rs:626-641, 708-718), after the state slots and the step's working memory
    have been taken out of the budget.  Returns (pages, budget in bytes)."""
    per = sum(page_bytes(g, page_size, dtype) for g in groups)
    budget = int(free_bytes * gpu_memory_utilization) - int(state_bytes) - int(workspace_bytes)
    return (max(0, budget // per) if per else 0), budget


class KVCache:
    def __init__(self, model, groups: List[CacheGroup], page_size: int, max_seqs: int, rt,
                 poison: bool = False):
        self.model, self.groups, self.page_size, self.rt = model, groups, page_size, rt
        self.pages: List[torch.Tensor] = []
        for g in groups:
            shape = (len(g.layers), g.num_pages, g.need.elements_per_token * page_size)
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
        need, flat, ps = self.groups[gi].need, self.pages[gi][idx], self.page_size
        named, at = {}, 0
        for t in need.tensors:
            n = t.heads * ps * t.width
            named[t.name] = flat[:, at:at + n].unflatten(1, (t.heads, ps, t.width))
            at += n
        pages = flat.view(flat.shape[0], 2, need.num_kv_heads, ps, need.head_dim) if need.is_kv else flat
        return LayerCache(group=gi, pages=pages, num_pages=self.groups[gi].num_pages, page_size=ps, writes=writes,
                          state=state, tensors=named)

    def reset_state(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()
