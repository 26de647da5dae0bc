"""Request parameters, named and checked as the reference does.

Names and defaults follow GenerateParameters (backends/vllm/src/types.rs:32-95):
temperature, repetition_penalty, repeat_last_n, top_k, top_p, do_sample,
max_new_tokens (default 100), random_seed; the checks follow Validation::validate
(backends/vllm/src/validation.rs:187-380): temperature > 0, repetition_penalty > 0,
0 < top_p < 1 when given, top_k > 0 when given, max_new_tokens != 0; the default
seed is 1_283_768_955 (:11).  Which sampler a request gets follows
backends/vllm/src/llm_service.rs:346-369: ArgMax when ``do_sample`` is false or the
temperature is exactly 1.0, else temperature sampling over all tokens, the top k,
the top-p nucleus, or top-k then top-p.  Text-level options (stop strings,
truncate, return_full_text) belong to the tokenizer side, which is outside this
engine: requests are token ids in, token ids out, with ``stop_token_ids`` instead.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

DEFAULT_RANDOM_SEED = 1_283_768_955


class ValidationError(ValueError):
    pass


@dataclass
class SamplingParams:
    temperature: Optional[float] = None        # None: 1.0
    top_k: Optional[int] = None                # None: no cut
    top_p: Optional[float] = None              # None: no cut
    repetition_penalty: Optional[float] = None # None: 1.0 (off)
    repeat_last_n: Optional[int] = None        # how far back the penalty looks; None: 64
    do_sample: bool = True
    max_new_tokens: Optional[int] = 100
    random_seed: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos_token: bool = False

    def validated(self) -> "ResolvedParams":
        t = 1.0 if self.temperature is None else float(self.temperature)
        if t <= 0.0:
            raise ValidationError("temperature must be greater than 0")
        rp = 1.0 if self.repetition_penalty is None else float(self.repetition_penalty)
        if rp <= 0.0:
            raise ValidationError("repetition_penalty must be greater than 0")
        if self.top_p is not None and not (0.0 < self.top_p < 1.0):
            raise ValidationError("top_p must be between 0.0 and 1.0 (exclusive)")
        if self.top_k is not None and self.top_k <= 0:
            raise ValidationError("top_k must be greater than 0")
        if self.max_new_tokens is not None and self.max_new_tokens <= 0:
            raise ValidationError("max_new_tokens must be greater than 0")
        rl = 64 if self.repeat_last_n is None else int(self.repeat_last_n)
        if rp != 1.0 and rl <= 0:
            raise ValidationError("repeat_last_n must be greater than 0 when a repetition penalty is set")
        greedy = (not self.do_sample) or t == 1.0  # llm_service.rs:346-349
        return ResolvedParams(
            greedy=greedy, temperature=t, top_k=int(self.top_k or 0), top_p=float(self.top_p or 1.0),
            repetition_penalty=rp, repeat_last_n=rl, max_new_tokens=self.max_new_tokens,
            seed=DEFAULT_RANDOM_SEED if self.random_seed is None else int(self.random_seed) & (2 ** 64 - 1),
            stop_token_ids=tuple(self.stop_token_ids), ignore_eos_token=self.ignore_eos_token,
        )


@dataclass(frozen=True)
class ResolvedParams:
    greedy: bool
    temperature: float
    top_k: int
    top_p: float
    repetition_penalty: float
    repeat_last_n: int
    max_new_tokens: Optional[int]
    seed: int
    stop_token_ids: Tuple[int, ...]
    ignore_eos_token: bool
