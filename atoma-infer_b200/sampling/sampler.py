"""Sampling a token for each wanted row of logits, on the device.

One kernel launch samples all rows (csrc/kernels/sampling.cu); per-row parameters
travel in one small buffer, only token ids come back.  The random number of a
request's n-th token depends on its seed and n alone (the reference gives every
request a generator of its own, backends/vllm/src/llm_service.rs:371-372), so a
request's tokens do not depend on who shares its batch, nor on preemption.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .params import ResolvedParams


class Sampler:
    def __init__(self, rt):
        self.rt = rt
        self._pinned = torch.cuda.is_available()
        self.h2d_bytes = self.d2h_bytes = 0  # bytes copied to and from the device so far

    def sample(self, logits: torch.Tensor, params: Sequence[ResolvedParams], steps: Sequence[int],
               histories: Sequence[Sequence[int]], slots: Sequence[int] = (), defer: bool = False):
        """``logits`` [R, vocab] float32 on the device; ``steps[i]``: how many tokens request i
        has sampled before; ``histories[i]``: its tokens so far (for the repetition penalty);
        ``slots[i]``: where to leave the token on the device for the next step's embedding.
        Returns the token ids as a list, or with ``defer`` a ``DeferredTokens``: the ids and the kernels'
        status words on their way to pinned host memory, with the CUDA event that marks their arrival."""
        R = logits.shape[0]
        if R == 0:
            return DeferredTokens(None, None, 0) if defer else []
        ops, dev = self.rt.ops, self.rt.device
        for i, p in enumerate(params):
            if p.repetition_penalty != 1.0:
                ctx = list(histories[i])[-p.repeat_last_n:]
                if ctx:
                    ops.repeat_penalty(logits[i], p.repetition_penalty,
                                       torch.tensor(ctx, dtype=torch.int32).to(dev, non_blocking=True))
        # one buffer: seed u64 | step u64 | temperature f32 | top_k i32 | top_p f32 (64-bit arrays first: aligned)
        S = R if len(slots) else 0
        host = torch.empty(7 * R + S, dtype=torch.int32, pin_memory=self._pinned)
        h = host.numpy()
        if S:
            h[7 * R:8 * R] = list(slots)
        h[0:2 * R].view(np.uint64)[:] = [p.seed for p in params]
        h[2 * R:4 * R].view(np.uint64)[:] = list(steps)
        h[4 * R:5 * R].view(np.float32)[:] = [0.0 if p.greedy else p.temperature for p in params]
        h[5 * R:6 * R] = [p.top_k for p in params]
        h[6 * R:7 * R].view(np.float32)[:] = [p.top_p for p in params]
        d = host.to(dev, non_blocking=True)
        self.h2d_bytes += host.numel() * 4
        out = torch.empty(R, dtype=torch.int32, device=dev)
        ops.sample(logits, d[4 * R:5 * R].view(torch.float32), d[5 * R:6 * R], d[6 * R:7 * R].view(torch.float32),
                   d[0:2 * R], d[2 * R:4 * R], out, slots=d[7 * R:8 * R] if S else None)
        if not defer:
            return out.tolist()
        status = getattr(ops, "status", None)
        ns = status.numel() if status is not None else 0
        back = torch.empty(R + ns, dtype=torch.int32, pin_memory=self._pinned)
        self.d2h_bytes += back.numel() * 4
        back[:R].copy_(out, non_blocking=True)
        if ns:  # the status words ride along: the host sees a kernel's complaint with the tokens it spoilt
            back[R:].copy_(status, non_blocking=True)
        event = None
        if torch.cuda.is_available() and dev.type == "cuda":
            event = torch.cuda.Event()
            event.record()
        return DeferredTokens(back, event, R)


class DeferredTokens:
    """Sampled token ids (and the kernels' status words) whose copy to the host may still be in flight."""

    def __init__(self, host, event, num_rows: int):
        self._host, self._event, self._rows = host, event, num_rows

    def wait(self):
        """(token ids as a list, status words as a list); blocks until the copy has landed."""
        if self._host is None:
            return [], []
        if self._event is not None:
            self._event.synchronize()
        values = self._host.tolist()
        return values[:self._rows], values[self._rows:]
