"""The engine: requests in, generated token ids out.

``Engine(model_dir, ...)`` loads a model folder; ``generate(prompts, params)`` runs
requests to their end; ``add_request`` / ``step`` drive it one step at a time.  One
step = the scheduler's plan -> the step function -> sampling -> stop rules, as the
reference's LlmEngine::step and process_generated_outputs do
(backends/vllm/src/llm_engine.rs:216-245, 264-342).  Stop rules in the reference's
order (:438-501): an end-of-sequence id of config.json unless ``ignore_eos_token``,
the model length, ``max_new_tokens``; stop strings become ``stop_token_ids`` since
text is outside this engine.  A finished request's pages are given back at once.
"""
from __future__ import annotations

import contextlib
import os
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..config.engine_config import EngineConfig
from ..sampling import ResolvedParams, Sampler, SamplingParams
from .runtime import LoadedModel, load_model
from .scheduler import Scheduler
from .step import StepEntry


@dataclass
class RequestMetrics:
    """Times in seconds since the epoch (backends/vllm/src/sequence.rs:142-160)."""

    arrival_time: float
    first_scheduled_time: Optional[float] = None
    first_token_time: Optional[float] = None
    finished_time: Optional[float] = None
    num_preemptions: int = 0


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str  # "stop" (end-of-sequence or stop id), "length", "ignored", "error"
    metrics: RequestMetrics
    error: Optional[str] = None  # with "error": what the kernels reported for the step that spoilt the request


@dataclass
class _Request:
    req: int
    prompt: List[int]
    params: ResolvedParams
    metrics: RequestMetrics
    output: List[int] = field(default_factory=list)
    pending: int = 0             # tokens sampled on the device that the host has not read yet
    ends_by_count: bool = False  # the token in flight is the request's last, whatever it is

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def token_span(self, start: int, n: int) -> List[int]:
        """Tokens start .. start+n-1 of prompt + output, without building the whole list."""
        p = len(self.prompt)
        if start >= p:
            return self.output[start - p:start - p + n]
        if start + n <= p:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.output[:start + n - p]


class Engine:
    def __init__(self, model_dir: str, config: Optional[EngineConfig] = None, *, ops=None, **overrides):
        """``ops``: another kernel table than the CUDA one (tests drive the host side with a stand-in)."""
        cfg = config or EngineConfig(**overrides)
        if config is not None and overrides:
            for k, v in overrides.items():
                setattr(cfg, k, v)
            cfg.__post_init__()
        self.config = cfg
        self.lm: LoadedModel = load_model(
            model_dir, dtype=cfg.dtype, device=getattr(ops, "device", None) or f"cuda:{cfg.device_id}", ops=ops,
            page_size=cfg.block_size,
            num_pages=cfg.num_gpu_blocks_override, max_seqs=cfg.max_num_sequences,
            gpu_memory_utilization=cfg.gpu_memory_utilization, cuda_graphs=cfg.cuda_graphs,
            max_model_len=cfg.max_model_len, max_batched_tokens=cfg.max_num_batched_tokens,
            random_weights_seed=cfg.random_weights_seed, random_weights_std=cfg.random_weights_std)
        spec = self.lm.model.spec
        self.max_model_len = min(cfg.max_model_len or spec.max_position or 2 ** 31, spec.max_position or 2 ** 31)
        self.scheduler = Scheduler(self.lm.manager, max_num_batched_tokens=cfg.max_num_batched_tokens,
                                   max_num_seqs=cfg.max_num_sequences, max_model_len=self.max_model_len,
                                   enable_chunked_prefill=cfg.enable_chunked_prefill)
        self.sampler = Sampler(self.lm.rt)
        self.eos_token_ids = tuple(spec.eos_token_ids)
        self._requests: Dict[int, _Request] = {}
        self._inflight = None  # (requests sampled, their tokens on the way to the host, all requests) of the last step
        self.num_device_errors = 0
        self._next_id = 0
        self.num_steps = 0
        self.num_generated = 0
        # Optional tracing (the reference has `tracing` spans around its worker and layers,
        # backends/vllm/src/worker.rs:110): ATOMA_INFER_TRACE=1 prints every step's batch composition and, one step
        # late so that nothing waits, its device time from a pair of CUDA events; ATOMA_INFER_NVTX=1 wraps plan,
        # launch and read-back of a step in NVTX ranges for a timeline profiler.
        self.trace = os.environ.get("ATOMA_INFER_TRACE", "0") not in ("", "0")
        self.nvtx = os.environ.get("ATOMA_INFER_NVTX", "0") not in ("", "0") and torch.cuda.is_available()
        self._trace_events = None

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        prompt = [int(t) for t in prompt_token_ids]
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        vocab = self.lm.model.spec.vocab_size
        if min(prompt) < 0 or max(prompt) >= vocab:
            raise ValueError(f"prompt token ids must lie in [0, {vocab})")
        resolved = (params or SamplingParams()).validated()
        if self.config.max_input_length is not None and len(prompt) > self.config.max_input_length:
            raise ValueError(f"the prompt has {len(prompt)} tokens, max_input_length is {self.config.max_input_length}")
        if self.config.max_total_tokens is not None:
            want = len(prompt) + (resolved.max_new_tokens or 0)
            if want > self.config.max_total_tokens:
                raise ValueError(f"prompt + max_new_tokens = {want} exceeds max_total_tokens {self.config.max_total_tokens}")
        req = self._next_id
        self._next_id += 1
        self._requests[req] = _Request(req, prompt, resolved, RequestMetrics(arrival_time=time.time()))
        self.scheduler.add_request(req, len(prompt))
        return req

    def abort_request(self, req: int) -> None:
        """Drops a request from whichever queue it is in; its pages go back (backends/vllm/src/scheduler.rs:390-443)."""
        if req in self._requests:
            self.scheduler.finish(req)
            del self._requests[req]

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    # ------------------------------------------------------------------ tracing
    def _range(self, name: str):
        return torch.cuda.nvtx.range(name) if self.nvtx else contextlib.nullcontext()

    def _trace_step(self, plan, entries) -> None:
        """One line per step on stderr: what ran, the pool, and the device time of the step before."""
        last = ""
        if self._trace_events is not None:
            n, a, b = self._trace_events
            if b.query():
                last = f"; step {n} took {a.elapsed_time(b):.3f} ms on the device"
        prompt = sum(len(e.tokens) for e in entries if len(e.tokens) > 1)
        decode = sum(1 for e in entries if len(e.tokens) == 1)
        mgr = self.lm.manager
        pools = ",".join(f"{mgr.num_free_pages(g)}/{mgr.num_usable_pages(g)}" for g in range(len(mgr.groups)))
        print(f"[trace] step {self.num_steps}: {len(entries)} requests, {prompt} prompt tokens, {decode} decode tokens, "
              f"{sum(1 for e in entries if e.want)} sampled; waiting {self.scheduler.num_waiting}, running "
              f"{self.scheduler.num_running}, preempted {len(plan.preempted)}, ignored {len(plan.ignored)}; free pages {pools}"
              f"{last}", file=sys.stderr, flush=True)

    def stats(self) -> dict:
        """Counters of the engine so far (the reference keeps such figures in its metrics registry,
        backends/vllm/src/llm_engine.rs:314-318)."""
        mgr = self.lm.manager
        return {"steps": self.num_steps, "generated_tokens": self.num_generated, "graph_replays": self.lm.step.graph_replays,
                "preemptions": self.scheduler.num_preemptions, "device_errors": self.num_device_errors,
                "waiting": self.scheduler.num_waiting, "running": self.scheduler.num_running,
                "free_pages": [mgr.num_free_pages(g) for g in range(len(mgr.groups))],
                "usable_pages": [mgr.num_usable_pages(g) for g in range(len(mgr.groups))],
                "kernel_launches": getattr(self.lm.rt.ops, "launches", 0)}

    # ------------------------------------------------------------------ one step
    def step(self) -> List[RequestOutput]:
        """Plans and launches one step, then reads the tokens of the step before it; returns the
        requests that ended.

        The host runs one step ahead of the device: a decode step is launched with "the token
        last sampled for this request" left on the device by the sampler, so the device never
        waits for the host to read tokens, plan and build the next step.  Stop rules that need
        the token's value (end-of-sequence, stop ids) therefore act one step late; the extra
        token such a request computes meanwhile is dropped.  Rules that only count (max_new_tokens,
        the model length) act at once.  Requests with a repetition penalty need their history on
        the host, so steps that sample for one are read back before the next is launched.
        """
        with self._range("plan"):
            plan = self.scheduler.schedule()
        now = time.time()
        finished: List[RequestOutput] = []
        for req in plan.ignored:
            r = self._requests.pop(req)
            r.metrics.finished_time = now
            finished.append(RequestOutput(req, r.prompt, r.output, "ignored", r.metrics))
        for req in plan.preempted:
            self._requests[req].metrics.num_preemptions += 1
        if not plan.entries:
            finished += self._resolve()
            return finished
        # a portion that needs the value of a token still on the device (a request sent back to
        # prefill right after sampling): read the tokens first
        for e in plan.entries:
            r = self._requests[e.req]
            known = len(r.prompt) + len(r.output)
            if r.pending and e.context_len + e.num_tokens > known and not (e.num_tokens == 1 and e.context_len == known):
                finished += self._resolve()
                break
        entries, sampled, taking_part = [], [], []
        for e in plan.entries:
            r = self._requests.get(e.req)
            if r is None:  # ended while the tokens were read just above
                continue
            if r.metrics.first_scheduled_time is None:
                r.metrics.first_scheduled_time = now
            if r.pending and e.num_tokens == 1 and e.context_len == len(r.prompt) + len(r.output):
                toks = [-1 - self.lm.manager.state_slot(e.req)]  # the token the sampler left on the device
            else:
                toks = r.token_span(e.context_len, e.num_tokens)
            entries.append(StepEntry(e.req, toks, [e.num_tokens - 1] if e.samples else []))
            taking_part.append(r)
            if e.samples:
                sampled.append(r)
        if not entries:
            self.scheduler.step_done()
            return finished
        if self.trace:
            self._trace_step(plan, entries)
        timed = self.trace and torch.cuda.is_available() and self.lm.rt.device.type == "cuda"
        if timed:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        with self._range("launch"):
            logits = self.lm.step.run(entries)
        if timed:
            b.record()
            self._trace_events = (self.num_steps, a, b)
        self.scheduler.step_done()
        self.num_steps += 1
        previous, self._inflight = self._inflight, None
        if sampled:
            slots = [self.lm.manager.state_slot(r.req) for r in sampled]
            tokens = self.sampler.sample(
                logits, [r.params for r in sampled], [len(r.output) + r.pending for r in sampled],
                [r.tokens if r.params.repetition_penalty != 1.0 else () for r in sampled], slots=slots, defer=True)
            for r in sampled:
                r.pending += 1
                n_out = len(r.output) + r.pending
                p = r.params
                if len(r.prompt) + n_out >= self.max_model_len or (p.max_new_tokens is not None and n_out >= p.max_new_tokens):
                    r.ends_by_count = True       # whatever the token is, the request ends with it
                else:
                    self.scheduler.append_token(r.req)
            self._inflight = (sampled, tokens, taking_part)
        finished += self._resolve(previous)
        if self._inflight and any(r.params.repetition_penalty != 1.0 for r in self._inflight[0]):
            finished += self._resolve()
        return finished

    def _resolve(self, inflight="current") -> List[RequestOutput]:
        """Reads the tokens of a launched step (waits for them if need be) and applies the stop rules."""
        if inflight == "current":
            inflight, self._inflight = self._inflight, None
        if not inflight:
            return []
        sampled, deferred, taking_part = inflight
        tokens, status = deferred.wait()
        now = time.time()
        finished = []
        ops = self.lm.rt.ops
        what = ops.describe_status(status) if status and hasattr(ops, "describe_status") else None
        if what:
            # A kernel reported a fault (a wait it gave up, a page or token id out of range) instead of
            # hanging or trapping: what this step computed, and left in the cache, cannot be trusted.  Its
            # requests end with reason "error"; the word is cleared for the steps that follow.
            ops.clear_status()
            self.num_device_errors += 1
            print(f"[engine] device status: {what}; {len(taking_part)} requests of the step end with an error",
                  file=sys.stderr, flush=True)
            for r in taking_part:
                if self._requests.get(r.req) is not r:
                    continue
                self.scheduler.finish(r.req)
                r.metrics.finished_time = now
                del self._requests[r.req]
                finished.append(RequestOutput(r.req, r.prompt, r.output, "error", r.metrics, error=what))
            return finished
        for r, tok in zip(sampled, tokens):
            if self._requests.get(r.req) is not r:
                continue  # ended or aborted since: its extra token is dropped
            r.pending -= 1
            r.output.append(tok)
            self.num_generated += 1
            if r.metrics.first_token_time is None:
                r.metrics.first_token_time = now
            reason = self._stop_reason(r, tok)
            if reason:
                self.scheduler.finish(r.req)
                r.metrics.finished_time = now
                del self._requests[r.req]
                finished.append(RequestOutput(r.req, r.prompt, r.output, reason, r.metrics))
        return finished

    def _stop_reason(self, r: _Request, tok: int) -> Optional[str]:
        p = r.params
        if tok in p.stop_token_ids:
            return "stop"
        if tok in self.eos_token_ids and not p.ignore_eos_token:
            return "stop"
        if len(r.prompt) + len(r.output) >= self.max_model_len:
            return "length"
        if p.max_new_tokens is not None and len(r.output) >= p.max_new_tokens:
            return "length"
        return None

    # ------------------------------------------------------------------ whole requests
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[RequestOutput]:
        """Runs all prompts to their end; results in the order of the prompts."""
        if params is None or isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams for all prompts, or one for each")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        done: Dict[int, RequestOutput] = {}
        while self.has_unfinished():
            for o in self.step():
                done[o.request_id] = o
        return [done[i] for i in ids]
