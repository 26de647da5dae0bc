"""Python face of the native scheduler (csrc/host/scheduler.cpp)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List

from ..cache.manager import CacheError, CacheManager, native

WAITING, RUNNING, FINISHED, IGNORED, UNKNOWN = 0, 1, 2, 3, -1


@dataclass(frozen=True)
class PlannedEntry:
    req: int
    context_len: int  # tokens already in the cache
    num_tokens: int   # tokens to run in this step
    samples: bool     # the portion reaches the end of the request: sample after it
    is_prompt: bool   # nothing sampled yet since (re)admission


@dataclass
class StepPlan:
    entries: List[PlannedEntry]
    preempted: List[int]
    ignored: List[int]


class Scheduler:
    """Admits requests, cuts prompts into portions under a token budget, plans decodes,
    preempts by recompute when pages run out.  Works on lengths; the caller keeps tokens."""

    def __init__(self, cache: CacheManager, *, max_num_batched_tokens: int, max_num_seqs: int,
                 max_model_len: int, enable_chunked_prefill: bool = True):
        self._lib = native()
        self.cache = cache  # keeps the native cache manager alive
        self._cap = max(max_num_seqs, 1) + 8
        self._h = self._lib.sched_create(cache.handle, max_num_batched_tokens, max_num_seqs, max_model_len,
                                         int(enable_chunked_prefill))
        if not self._h:
            raise ValueError("scheduler: budgets and max_model_len must be positive")
        c = ctypes
        self._req = (c.c_int64 * self._cap)()
        self._ctx = (c.c_int64 * self._cap)()
        self._n = (c.c_int32 * self._cap)()
        self._samples = (c.c_int32 * self._cap)()
        self._is_prompt = (c.c_int32 * self._cap)()
        self._pre = (c.c_int64 * self._cap)()
        self._ign = (c.c_int64 * self._cap)()
        self._counts = (c.c_int32 * 3)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.sched_destroy(h)

    def add_request(self, req: int, prompt_len: int) -> None:
        code = self._lib.sched_add_request(self._h, req, prompt_len)
        if code < 0:
            raise CacheError(code, f"scheduler.add_request({req}, {prompt_len})")

    def schedule(self) -> StepPlan:
        code = self._lib.sched_schedule(self._h, self._cap, self._req, self._ctx, self._n, self._samples,
                                        self._is_prompt, self._pre, self._ign, self._counts)
        if code < 0:
            raise CacheError(code, "scheduler.schedule")
        ne, npre, nign = self._counts[0], self._counts[1], self._counts[2]
        entries = [PlannedEntry(self._req[i], self._ctx[i], self._n[i], bool(self._samples[i]), bool(self._is_prompt[i]))
                   for i in range(ne)]
        return StepPlan(entries, list(self._pre[:npre]), list(self._ign[:nign]))

    def step_done(self) -> None:
        self._lib.sched_step_done(self._h)

    def append_token(self, req: int) -> None:
        code = self._lib.sched_append_token(self._h, req)
        if code < 0:
            raise CacheError(code, f"scheduler.append_token({req})")

    def finish(self, req: int) -> None:
        code = self._lib.sched_finish(self._h, req)
        if code < 0:
            raise CacheError(code, f"scheduler.finish({req})")

    def status(self, req: int) -> int:
        return self._lib.sched_status(self._h, req)

    def length(self, req: int) -> int:
        return self._lib.sched_length(self._h, req)

    def num_computed(self, req: int) -> int:
        return self._lib.sched_num_computed(self._h, req)

    @property
    def num_waiting(self) -> int:
        return self._lib.sched_num_waiting(self._h)

    @property
    def num_running(self) -> int:
        return self._lib.sched_num_running(self._h)

    @property
    def num_preemptions(self) -> int:
        return self._lib.sched_num_preemptions(self._h)

    @property
    def prompt_limit(self) -> int:
        return self._lib.sched_prompt_limit(self._h)

    def has_unfinished(self) -> bool:
        return self.num_waiting + self.num_running > 0
