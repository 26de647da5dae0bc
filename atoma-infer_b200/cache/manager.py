"""Python face of the native cache manager (csrc/host/cache_manager.cpp).

``CacheNeed`` is what a mixer asks of the cache; layers with equal needs form a
``CacheGroup`` that has a page pool and block tables of its own.  The reference
has one pool for all layers and a global sliding window
(backends/vllm/src/block_manager.rs:37-50, 61); groups are this engine's way to
let layers of one model differ.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..csrc.build import host_library
from .spec import FULL_KEYS, WINDOW_KEYS, CacheGroup, CacheNeed

_ERRORS = {
    -20: "an entry brings no tokens", -21: "a request appears twice in one step",
    -22: "a wanted place lies outside the entry's tokens", -23: "token ids must lie in the vocabulary",
    -1: "out of pages", -2: "no free state slot", -3: "unknown request (or freed twice)",
    -4: "request already exists", -5: "advance beyond what was reserved",
    -6: "the request would not fit an empty cache", -7: "bad argument",
}


class CacheError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(f"{what}: {_ERRORS.get(code, code)}")


class OutOfPages(CacheError):
    pass


def _bind(lib):
    if getattr(lib, "_bound", False):
        return lib
    c = ctypes
    i64, i32p, i64p = c.c_int64, c.POINTER(c.c_int32), c.POINTER(c.c_int64)
    sig = {
        "cm_create": (c.c_void_p, [c.c_int, c.c_int, c.POINTER(c.c_int), c.POINTER(c.c_int), c.POINTER(c.c_int), c.c_int]),
        "cm_destroy": (None, [c.c_void_p]),
        "cm_add_request": (c.c_int, [c.c_void_p, i64]),
        "cm_has_request": (c.c_int, [c.c_void_p, i64]),
        "cm_can_reserve": (c.c_int, [c.c_void_p, i64, i64]),
        "cm_reserve": (c.c_int, [c.c_void_p, i64, i64]),
        "cm_advance": (c.c_int, [c.c_void_p, i64, i64]),
        "cm_free_request": (c.c_int, [c.c_void_p, i64]),
        "cm_num_tokens": (i64, [c.c_void_p, i64]),
        "cm_state_slot": (c.c_int, [c.c_void_p, i64]),
        "cm_table_len": (c.c_int, [c.c_void_p, i64, c.c_int]),
        "cm_table": (c.c_int, [c.c_void_p, i64, c.c_int, c.c_void_p, c.c_int]),
        "cm_pages_needed": (c.c_int, [c.c_void_p, i64, c.c_int, i64]),
        "cm_num_free_pages": (c.c_int, [c.c_void_p, c.c_int]),
        "cm_num_usable_pages": (c.c_int, [c.c_void_p, c.c_int]),
        "cm_num_free_slots": (c.c_int, [c.c_void_p]),
        "cm_num_requests": (c.c_int, [c.c_void_p]),
        "cm_audit": (c.c_int, [c.c_void_p, c.c_char_p, c.c_int]),
        # arrays go as addresses (numpy's .ctypes.data)
        "cm_step_begin": (c.c_int, [c.c_void_p, c.c_int] + [c.c_void_p] * 5 + [c.c_int] + [c.c_void_p] * 5),
        "cm_step_fill": (None, [c.c_void_p, c.c_int] + [c.c_void_p] * 8 + [c.c_int] * 11 + [c.c_void_p] * 2 + [c.c_int] * 5),
        "sched_create": (c.c_void_p, [c.c_void_p, c.c_int, c.c_int, i64, c.c_int]),
        "sched_destroy": (None, [c.c_void_p]),
        "sched_add_request": (c.c_int, [c.c_void_p, i64, i64]),
        "sched_schedule": (c.c_int, [c.c_void_p, i32p]),
        "sched_plan": (c.c_int, [c.c_void_p, i64p, i64p, i32p, i32p, i32p, i64p, i64p]),
        "sched_step_done": (None, [c.c_void_p]),
        "sched_append_token": (c.c_int, [c.c_void_p, i64]),
        "sched_finish": (c.c_int, [c.c_void_p, i64]),
        "sched_status": (c.c_int, [c.c_void_p, i64]),
        "sched_length": (i64, [c.c_void_p, i64]),
        "sched_num_computed": (i64, [c.c_void_p, i64]),
        "sched_num_waiting": (c.c_int, [c.c_void_p]),
        "sched_num_running": (c.c_int, [c.c_void_p]),
        "sched_num_preemptions": (i64, [c.c_void_p]),
        "sched_prompt_limit": (i64, [c.c_void_p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    lib._bound = True
    return lib


def native():
    return _bind(host_library())


class CacheManager:
    """Pages, block tables and state slots of all live requests (host bookkeeping only)."""

    def __init__(self, page_size: int, groups: Sequence[CacheGroup], max_seqs: int):
        self._lib = native()
        self.page_size = page_size
        self.groups = list(groups)
        self.max_seqs = max_seqs
        n = len(self.groups)
        arr = ctypes.c_int * max(n, 1)
        kinds = arr(*[g.need.kind for g in self.groups])
        windows = arr(*[(g.need.window or 0) for g in self.groups])
        pages = arr(*[g.num_pages for g in self.groups])
        self._h = self._lib.cm_create(page_size, n, kinds, windows, pages, max_seqs)
        if not self._h:
            raise ValueError("cache manager: bad geometry (page size, pool sizes, windows and max_seqs must be positive)")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.cm_destroy(h)

    @property
    def handle(self):
        return self._h

    def _check(self, code: int, what: str) -> int:
        if code < 0:
            raise (OutOfPages if code in (-1, -6) else CacheError)(code, what)
        return code

    def add_request(self, req: int) -> int:
        """Claims a state slot for a new request; returns the slot."""
        return self._check(self._lib.cm_add_request(self._h, req), f"add_request({req})")

    def has_request(self, req: int) -> bool:
        return bool(self._lib.cm_has_request(self._h, req))

    def can_reserve(self, req: int, upto: int) -> int:
        """0 if the pools can cover ``upto`` tokens of ``req`` now, -1 not now, -6 never."""
        return self._lib.cm_can_reserve(self._h, req, upto)

    def reserve(self, req: int, upto: int) -> None:
        self._check(self._lib.cm_reserve(self._h, req, upto), f"reserve({req}, {upto})")

    def advance(self, req: int, n: int) -> int:
        """``req`` holds ``n`` more tokens; returns how many pages a window gave back."""
        return self._check(self._lib.cm_advance(self._h, req, n), f"advance({req}, {n})")

    def free_request(self, req: int) -> int:
        return self._check(self._lib.cm_free_request(self._h, req), f"free_request({req})")

    def num_tokens(self, req: int) -> int:
        return self._check(self._lib.cm_num_tokens(self._h, req), f"num_tokens({req})")

    def state_slot(self, req: int) -> int:
        return self._check(self._lib.cm_state_slot(self._h, req), f"state_slot({req})")

    def table(self, req: int, group: int = 0) -> List[int]:
        n = self._check(self._lib.cm_table_len(self._h, req, group), f"table({req})")
        buf = (ctypes.c_int32 * max(n, 1))()
        self._lib.cm_table(self._h, req, group, buf, n)
        return list(buf[:n])

    def table_into(self, req: int, group: int, address: int, cap: int) -> int:
        """Writes the block table to int32 memory at ``address``; returns its full length."""
        return self._check(self._lib.cm_table(self._h, req, group, address, cap), f"table({req})")

    def step_begin(self, reqs, ntok, tokens, want_count, wants, vocab: int):
        """Admits and checks the entries of a step and claims their pages, in one native call.
        Arguments are numpy arrays: request ids (int64), tokens each entry brings, the tokens
        themselves one entry after the other, wanted places each entry has, and those places (all
        int32).  Returns (tokens cached, state slot, starts-now flag) per entry and the longest block
        table per group.  Raises ValueError for a malformed entry, CacheError/OutOfPages when the
        cache refuses; the refused entry leaves nothing behind."""
        n = len(reqs)
        ctx, slot, new = np.empty(n, np.int64), np.empty(n, np.int32), np.empty(n, np.int32)
        lens = np.ones(max(len(self.groups), 1), np.int32)
        bad = ctypes.c_int32(-1)
        code = self._lib.cm_step_begin(self._h, n, reqs.ctypes.data, ntok.ctypes.data, tokens.ctypes.data,
                                       want_count.ctypes.data, wants.ctypes.data, vocab, ctx.ctypes.data, slot.ctypes.data,
                                       new.ctypes.data, lens.ctypes.data, ctypes.addressof(bad))
        if code <= -20:
            k = bad.value
            raise ValueError(f"request {int(reqs[k])} (entry {k} of the step, {int(ntok[k])} tokens): {_ERRORS[code]}"
                             + (f" [0, {vocab})" if code == -23 else ""))
        if code < 0:
            self._check(code, f"step entry {bad.value} (request {int(reqs[bad.value])})")
        return ctx, slot, new, lens

    def step_fill(self, *args) -> None:
        """Writes the step's metadata buffer (csrc/host/step_meta.cpp gives the arguments)."""
        self._lib.cm_step_fill(self._h, *args)

    def table_len(self, req: int, group: int = 0) -> int:
        return self._check(self._lib.cm_table_len(self._h, req, group), f"table_len({req})")

    def pages_needed(self, req: int, group: int, upto: int) -> int:
        return self._check(self._lib.cm_pages_needed(self._h, req, group, upto), f"pages_needed({req})")

    def num_free_pages(self, group: int = 0) -> int:
        return self._lib.cm_num_free_pages(self._h, group)

    def num_usable_pages(self, group: int = 0) -> int:
        return self._lib.cm_num_usable_pages(self._h, group)

    def num_free_slots(self) -> int:
        return self._lib.cm_num_free_slots(self._h)

    def num_requests(self) -> int:
        return self._lib.cm_num_requests(self._h)

    def audit(self) -> str:
        """Empty when no page or slot is lost, held twice or free twice."""
        buf = ctypes.create_string_buffer(4096)
        self._lib.cm_audit(self._h, buf, 4096)
        return buf.value.decode()
