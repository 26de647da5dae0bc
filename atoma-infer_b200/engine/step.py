"""The step function: one batch of (request, its next tokens) through the model.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere,
runs only those tokens, from the cache that earlier steps left, and returns
float32 logits at the wanted places only.  It claims the pages the tokens need,
builds the step's metadata in one int32 buffer (one host-to-device copy; the
reference uploads about ten small tensors, backends/vllm/src/worker.rs:411-434),
runs the model's forward pass and advances the requests in the cache manager.

The reference's counterpart is ModelWorker::execute_model with
prepare_input_tensors (backends/vllm/src/worker.rs:111-191, 224-460); it returns
the last row of every sequence (:166, 688-698) and cannot run a later portion of a
prompt against its cached part (models/src/flash_attention.rs:384-410).
"""
from __future__ import annotations

import gc
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.kv_cache import KVCache
from ..cache.manager import CacheManager
from ..csrc.ops import (MAX_GROUPS, META_BT_OFFSET, META_BT_STRIDE, META_HEADER_INTS, META_NUM_ENTRIES,
                        META_NUM_ROWS, META_NUM_TOKENS)
from ..parts.base import EntryInfo, Runtime, StepContext


@dataclass
class StepEntry:
    """A request's share of a step: its next tokens and the places (indices into these
    tokens) whose logits are wanted."""

    req: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class MetaLayout:
    """Where each array lies in the metadata buffer, for given capacities."""

    T: int
    S: int
    R: int
    strides: Tuple[int, ...]  # block-table row length per group

    def __post_init__(self):
        o = META_HEADER_INTS
        self.tokens = o; o += self.T
        self.positions = o; o += self.T
        self.token_entry = o; o += self.T
        self.cu = o; o += self.S + 1
        self.ctx = o; o += self.S
        self.slots = o; o += self.S
        self.rows = o; o += max(self.R, 1)
        self.tables = []
        for s in self.strides:
            self.tables.append(o)
            o += self.S * s
        self.size = o


class StepFunction:
    def __init__(self, model, cache: KVCache, manager: CacheManager, rt: Runtime, cuda_graphs: bool = False,
                 max_model_len: int = 0):
        if len(manager.groups) > MAX_GROUPS:
            raise ValueError(f"at most {MAX_GROUPS} cache groups are supported")
        self.model, self.cache, self.manager, self.rt = model, cache, manager, rt
        self.page_size = manager.page_size
        self._pinned = torch.cuda.is_available()
        self.steps = 0
        self.h2d_bytes = 0  # bytes of step metadata copied to the device so far
        # Decode steps (every request brings one token and wants its logits) replay a CUDA graph
        # captured per padded batch size; the reference has no graphs.
        self.cuda_graphs = cuda_graphs and torch.cuda.is_available() and getattr(model, "graph_safe", True)
        self.max_model_len = max_model_len
        self._graphs: Dict[Tuple[int, int], "_DecodeGraph"] = {}  # insertion order = least recently used first
        self._graph_meta: Dict[int, torch.Tensor] = {}  # metadata buffer of a bucket, shared by its graphs
        self._graph_pool = None                          # one memory pool for the activations of all graphs
        self.graph_replays = 0

    # ------------------------------------------------------------------ metadata
    def _host_buffer(self, n: int) -> torch.Tensor:
        return torch.empty(n, dtype=torch.int32, pin_memory=self._pinned)

    def prepare(self, entries: Sequence[StepEntry], pad_to: int = 0):
        """Claims pages, builds the metadata on the host.  Returns (host buffer, layout, infos, R).
        ``pad_to``: lay the arrays out for that many tokens, entries and rows (a captured graph's
        fixed sizes); the header still holds the true counts, which is what the kernels obey."""
        mgr = self.manager
        S = len(entries)
        counts = [len(e.tokens) for e in entries]
        ntok = np.asarray(counts, dtype=np.int32)
        reqs = np.asarray([e.req for e in entries], dtype=np.int64)
        tokens = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=sum(counts))
        if tokens.size and (tokens.max() > 0x7FFFFFFF or tokens.min() < -0x80000000):
            raise ValueError("token ids must fit 32 bits")
        tokens = tokens.astype(np.int32)
        want_count = np.asarray([len(e.want) for e in entries], dtype=np.int32)
        wants = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=int(want_count.sum()))
        ctx, slots, new, strides = mgr.step_begin(reqs, ntok, tokens, want_count, wants, self.model.spec.vocab_size)
        starts = np.cumsum(ntok) - ntok
        infos = [EntryInfo(e.req, int(a), int(n), int(c), int(s), bool(f))
                 for e, a, n, c, s, f in zip(entries, starts, ntok, ctx, slots, new)]
        T, R = int(tokens.size), int(wants.size)
        strides = tuple(int(x) for x in strides[:len(mgr.groups)])
        lay = MetaLayout(max(T, pad_to), max(S, pad_to), max(R, pad_to), strides)
        host = self._host_buffer(lay.size)
        table_off = np.asarray(lay.tables or [0], dtype=np.int32)
        table_stride = np.asarray(strides or (1,), dtype=np.int32)
        mgr.step_fill(S, reqs.ctypes.data, ntok.ctypes.data, ctx.ctypes.data, slots.ctypes.data, tokens.ctypes.data,
                      want_count.ctypes.data, wants.ctypes.data, host.data_ptr(), META_HEADER_INTS, lay.T, lay.S, lay.R,
                      lay.tokens, lay.positions, lay.token_entry, lay.cu, lay.ctx, lay.slots, lay.rows,
                      table_off.ctypes.data, table_stride.ctypes.data, META_NUM_TOKENS, META_NUM_ENTRIES, META_NUM_ROWS,
                      META_BT_STRIDE, META_BT_OFFSET)
        return host, lay, infos, R

    def context(self, dev: torch.Tensor, lay: MetaLayout, infos: List[EntryInfo]) -> StepContext:
        """Views into the step's metadata on the device, for the parts."""
        v = lambda o, n: dev[o:o + n]  # noqa: E731
        return StepContext(
            rt=self.rt, T=lay.T, S=lay.S, meta=dev,
            tokens=v(lay.tokens, lay.T), positions=v(lay.positions, lay.T), token_entry=v(lay.token_entry, lay.T),
            cu_tokens=v(lay.cu, lay.S + 1), context_lens=v(lay.ctx, lay.S), state_slots=v(lay.slots, lay.S),
            entries=infos,
            max_tokens_per_entry=max((i.num_tokens for i in infos), default=0),
            max_context=max((i.context_len + i.num_tokens for i in infos), default=0),
            decode_only=all(i.num_tokens == 1 for i in infos),
            page_size=self.page_size, table_offsets=tuple(lay.tables), table_strides=tuple(lay.strides),
        )

    # ------------------------------------------------------------------ the step
    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the step; returns float32 logits [wanted places, vocab] on the device, in the
        order of the entries and of their ``want`` lists."""
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.rt.device)
        if self._graph_eligible(entries):
            return self._run_graph(entries)
        host, lay, infos, R = self.prepare(entries)
        dev = host.to(self.rt.device, non_blocking=True)
        self.h2d_bytes += host.numel() * 4
        for i in infos:
            if i.is_new:
                self.cache.reset_state(i.state_slot)
        ctx = self.context(dev, lay, infos)
        logits = self.model.forward(ctx, self.cache, dev[lay.rows:lay.rows + max(R, 1)], R)
        for i in infos:
            self.manager.advance(i.req, i.num_tokens)
        self.steps += 1
        return logits

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
    MAX_GRAPHS = 32  # captured (batch bucket, context bound) pairs kept; beyond that the least recently used goes

    def _graph_eligible(self, entries: Sequence[StepEntry]) -> bool:
        if not self.cuda_graphs or len(entries) > self.GRAPH_BUCKETS[-1]:
            return False
        return all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def _run_graph(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        S = len(entries)
        bucket = next(b for b in self.GRAPH_BUCKETS if b >= S)
        # Kernels size their work splits by the longest context; graphs are kept per power-of-two
        # bound on it, so a captured split count stays right while contexts grow.
        longest = max((self.manager.num_tokens(e.req) if self.manager.has_request(e.req) else 0) for e in entries) + 1
        ctx_bound = max(256, 1 << (longest - 1).bit_length())
        key = (bucket, ctx_bound)
        g = self._graphs.pop(key, None)
        if g is None:
            cap_stride = -(-max(self.max_model_len, 1) // self.page_size)
            meta = self._graph_meta.get(bucket)
            if meta is None:
                cap = MetaLayout(bucket, bucket, bucket, (cap_stride,) * len(self.manager.groups)).size
                meta = self._graph_meta[bucket] = torch.zeros(cap, dtype=torch.int32, device=self.rt.device)
            g = _DecodeGraph(meta, cap_stride)
            while len(self._graphs) >= self.MAX_GRAPHS:  # the graph unused for longest goes
                self._graphs.pop(next(iter(self._graphs)))
        self._graphs[key] = g  # most recently used last
        host, lay, infos, R = self.prepare(entries, pad_to=bucket)
        if max(lay.strides, default=0) > g.cap_stride:
            raise RuntimeError(f"a request holds more pages than max_model_len ({self.max_model_len}) allows")
        g.meta[:lay.size].copy_(host, non_blocking=True)
        self.h2d_bytes += host.numel() * 4
        for i in infos:
            if i.is_new:  # a one-token prompt is a decode step too: its state starts from zero
                self.cache.reset_state(i.state_slot)
        if g.graph is None:
            ctx = self.context(g.meta, lay, [])
            # sizes that pick kernels and splits are those of the bucket, not of this batch
            ctx.decode_only, ctx.max_tokens_per_entry, ctx.max_context = True, 1, ctx_bound
            rows = g.meta[lay.rows:lay.rows + bucket]
            if not g.warm:  # the first step of a bucket runs eagerly: libraries load, attributes get set
                logits = self.model.forward(ctx, self.cache, rows, bucket)
                g.warm = True
            else:
                torch.cuda.synchronize(self.rt.device)
                graph = torch.cuda.CUDAGraph()
                before = self.rt.ops.launches
                if self._graph_pool is None:
                    self._graph_pool = torch.cuda.graph_pool_handle()
                # one pool for all graphs: only one replays at a time and its logits are consumed (sampled or
                # copied) on the same stream before the next replay, so their activations may share memory
                # Garbage that holds captured graphs of an engine no longer in use must not be collected while
                # this capture runs (destroying a graph then invalidates the capture): collect it now, and keep the
                # collector off until the capture has ended.
                gc.collect()
                gc_was_on = gc.isenabled()
                gc.disable()
                try:
                    with torch.cuda.graph(graph, pool=self._graph_pool):
                        g.logits = self.model.forward(ctx, self.cache, rows, bucket)
                finally:
                    if gc_was_on:
                        gc.enable()
                g.kernels = self.rt.ops.launches - before  # own kernels in one replay
                g.graph = graph
                graph.replay()
                logits = g.logits
        else:
            g.graph.replay()
            self.graph_replays += 1
            self.rt.ops.launches += g.kernels
            logits = g.logits
        for i in infos:
            self.manager.advance(i.req, i.num_tokens)
        self.steps += 1
        return logits[:S]

    def finish(self, req: int) -> None:
        """The request ends: its pages and its state slot go back to the pools."""
        self.manager.free_request(req)


class _DecodeGraph:
    """A captured decode step for one padded batch size: its metadata buffer (fixed address,
    rewritten before every replay) and its logits buffer."""

    def __init__(self, meta: torch.Tensor, cap_stride: int):
        self.meta, self.cap_stride = meta, cap_stride
        self.graph = None
        self.logits = None
        self.warm = False
        self.kernels = 0
