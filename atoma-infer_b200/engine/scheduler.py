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
        self._h = self._lib.sched_create(cache.handle, max_num_batched_tokens, max_num_seqs, max_model_len,
                                         int(enable_chunked_prefill))
        if not self._h:
            raise ValueError("scheduler: budgets and max_model_len must be positive")
        self._counts = (ctypes.c_int32 * 3)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.sched_destroy(h)

    def add_request(self, req: int, prompt_len: int) -> None:
        code = self._lib.sched_add_request(self._h, req, prompt_len)
        if code < 0:
            raise CacheError(code, f"scheduler.add_request({req}, {prompt_len})")

    def schedule(self) -> StepPlan:
        """Plans one step.  Planning changes the queues, so it cannot be allowed to fail afterwards: the
        native side keeps the plan and says how long its three lists are, then fills arrays of that size."""
        code = self._lib.sched_schedule(self._h, self._counts)
        if code < 0:
            raise CacheError(code, "scheduler.schedule")
        ne, npre, nign = self._counts[0], self._counts[1], self._counts[2]
        c = ctypes
        i64 = lambda n: (c.c_int64 * max(n, 1))()  # noqa: E731
        i32 = lambda n: (c.c_int32 * max(n, 1))()  # noqa: E731
        req, ctx, num, samples, is_prompt, pre, ign = i64(ne), i64(ne), i32(ne), i32(ne), i32(ne), i64(npre), i64(nign)
        self._lib.sched_plan(self._h, req, ctx, num, samples, is_prompt, pre, ign)
        entries = [PlannedEntry(req[i], ctx[i], num[i], bool(samples[i]), bool(is_prompt[i])) for i in range(ne)]
        return StepPlan(entries, list(pre[:npre]), list(ign[:nign]))

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
