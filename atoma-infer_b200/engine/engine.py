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
    finish_reason: str  # "stop" (end-of-sequence or stop id), "length", "ignored"
    metrics: RequestMetrics


@dataclass
class _Request:
    req: int
    prompt: List[int]
    params: ResolvedParams
    metrics: RequestMetrics
    output: List[int] = field(default_factory=list)

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
    def __init__(self, model_dir: str, config: Optional[EngineConfig] = None, **overrides):
        cfg = config or EngineConfig(**overrides)
        if config is not None and overrides:
            for k, v in overrides.items():
                setattr(cfg, k, v)
            cfg.__post_init__()
        self.config = cfg
        self.lm: LoadedModel = load_model(
            model_dir, dtype=cfg.dtype, device=f"cuda:{cfg.device_id}", page_size=cfg.block_size,
            num_pages=cfg.num_gpu_blocks_override, max_seqs=cfg.max_num_sequences,
            gpu_memory_utilization=cfg.gpu_memory_utilization, cuda_graphs=cfg.cuda_graphs,
            max_model_len=cfg.max_model_len)
        spec = self.lm.model.spec
        self.max_model_len = min(cfg.max_model_len or spec.max_position or 2 ** 31, spec.max_position or 2 ** 31)
        self.scheduler = Scheduler(self.lm.manager, max_num_batched_tokens=cfg.max_num_batched_tokens,
                                   max_num_seqs=cfg.max_num_sequences, max_model_len=self.max_model_len,
                                   enable_chunked_prefill=cfg.enable_chunked_prefill)
        self.sampler = Sampler(self.lm.rt)
        self.eos_token_ids = tuple(spec.eos_token_ids)
        self._requests: Dict[int, _Request] = {}
        self._next_id = 0
        self.num_steps = 0
        self.num_generated = 0

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
        return self.scheduler.has_unfinished()

    # ------------------------------------------------------------------ one step
    def step(self) -> List[RequestOutput]:
        """Plans and runs one step; returns the requests that ended in it."""
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
            return finished
        entries, sampled = [], []
        for e in plan.entries:
            r = self._requests[e.req]
            if r.metrics.first_scheduled_time is None:
                r.metrics.first_scheduled_time = now
            toks = r.token_span(e.context_len, e.num_tokens)
            entries.append(StepEntry(e.req, toks, [e.num_tokens - 1] if e.samples else []))
            if e.samples:
                sampled.append(r)
        logits = self.lm.step.run(entries)
        self.scheduler.step_done()
        self.num_steps += 1
        if sampled:
            tokens = self.sampler.sample(logits, [r.params for r in sampled], [len(r.output) for r in sampled],
                                         [r.tokens if r.params.repetition_penalty != 1.0 else () for r in sampled])
            now = time.time()
            for r, tok in zip(sampled, tokens):
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
                else:
                    self.scheduler.append_token(r.req)
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
            outs = self.step()
            for o in outs:
                done[o.request_id] = o
            if not outs and not self.has_unfinished():
                break
        return [done[i] for i in ids]
