"""A model as data: layers chosen part by part, and the order in which they run.

``ModelSpec`` is what an architecture's builder returns from its configuration:
per layer the kinds and parameters of block, mixer, feed-forward and norm, and a
``schedule`` — the list of layer runs.  A run names the layer to execute and the
layer whose cache it uses, so a layer may run twice or read another layer's keys
and values.  ``DecoderModel`` turns the spec into bound parts and runs a step:
the embedding part, the scheduled blocks, the final norm at the wanted rows, the head part
(models/src/llama.rs:456-478 has this sequence fixed for one model).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.spec import CacheGroup, CacheNeed
from ..config.registry import part_class
from ..weights.loader import TensorDecl
from .base import LayerCache, Runtime, StepContext
from .decode_stack import MAX_ROWS as STACK_MAX_ROWS, plan_stacks

# the registrations of the built-in parts
from . import attention, block, embedding, feed_forward, head, norm, position  # noqa: F401


@dataclass
class LayerSpec:
    prefix: str              # checkpoint prefix of the layer, e.g. "model.layers.3"
    block: Dict[str, Any]    # {"kind": "prenorm", "norm": {...}, "mixer": {...}, "feed_forward": {...}}


@dataclass
class LayerRun:
    layer: int                       # index into ModelSpec.layers
    cache_of: Optional[int] = None   # layer whose cache this run uses (None: its own)


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: List[LayerSpec]
    final_norm: Dict[str, Any]
    embedding_tensor: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm"
    head_tensor: Optional[str] = "lm_head.weight"   # None: the embedding matrix is the head
    # The two ends of the model as parts, by kind like the rest.  None: the plain ones, a token table named
    # ``embedding_tensor`` and a bias-free linear head on ``head_tensor``.
    embedding: Optional[Dict[str, Any]] = None
    head: Optional[Dict[str, Any]] = None
    schedule: Optional[List[LayerRun]] = None       # None: every layer once, in order
    ignored_tensors: Tuple[str, ...] = ()           # globs a checkpoint may carry unused
    max_position: int = 0
    eos_token_ids: Tuple[int, ...] = ()

    def runs(self) -> List[LayerRun]:
        return self.schedule if self.schedule is not None else [LayerRun(i) for i in range(len(self.layers))]

    def embedding_spec(self) -> Dict[str, Any]:
        return self.embedding or {"kind": "token", "vocab": self.vocab_size, "hidden": self.hidden_size,
                                  "tensor": self.embedding_tensor}

    def head_spec(self) -> Dict[str, Any]:
        return self.head or {"kind": "linear", "vocab": self.vocab_size, "hidden": self.hidden_size,
                             "tensor": self.head_tensor}


def _build_layers(spec: ModelSpec):
    return [part_class("block", ls.block["kind"])(ls.block, ls.prefix) for ls in spec.layers]


def _build_ends(spec: ModelSpec):
    e, h = spec.embedding_spec(), spec.head_spec()
    return part_class("embedding", e["kind"])(e, ""), part_class("head", h["kind"])(h, "")


def declared_tensors(spec: ModelSpec) -> List[TensorDecl]:
    """Every checkpoint tensor the model needs, by name and shape."""
    embedding, head = _build_ends(spec)
    decls = embedding.declare()
    for blk in _build_layers(spec):
        decls += blk.declare()
    decls += part_class("norm", spec.final_norm["kind"])(spec.final_norm, spec.final_norm_prefix).declare()
    return decls + head.declare()


class DecoderModel:
    """Bound parts of one model plus the plan of its cache."""

    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks = _build_layers(spec)
        self.embedding, self.head = _build_ends(spec)
        self.final_norm = part_class("norm", spec.final_norm["kind"])(spec.final_norm, spec.final_norm_prefix)
        self.runs = spec.runs()
        # Who owns which cache: a run without ``cache_of`` owns pages (and state) of its own, so a layer
        # that runs twice keeps two caches; a run with ``cache_of`` reads the pages of the first owning
        # run of that layer, which must come earlier in the schedule (its keys of this step are written).
        self.run_owner: List[int] = []
        first_owner: Dict[int, int] = {}
        for i, r in enumerate(self.runs):
            if not (0 <= r.layer < len(self.blocks)):
                raise ValueError(f"schedule names layer {r.layer}, the model has {len(self.blocks)}")
            if r.cache_of is None:
                first_owner.setdefault(r.layer, i)
                self.run_owner.append(i)
                continue
            if r.cache_of not in first_owner:
                raise ValueError(f"schedule lets layer {r.layer} read the cache of layer {r.cache_of}, "
                                 f"which has not run (with a cache of its own) before it")
            a, b = self.blocks[r.layer].mixer.cache_need(), self.blocks[r.cache_of].mixer.cache_need()
            if a != b:
                raise ValueError(f"layer {r.layer} cannot read the cache of layer {r.cache_of}: {a} != {b}")
            self.run_owner.append(first_owner[r.cache_of])
        # Cache groups: owning runs put together by what they need.
        self.groups: List[CacheGroup] = []
        self.run_group: Dict[int, Tuple[int, int]] = {}  # owning run -> (group, index within the group)
        for i in sorted(set(self.run_owner)):
            need = self.blocks[self.runs[i].layer].mixer.cache_need()
            if need is None:
                continue
            for gi, g in enumerate(self.groups):
                if g.need == need:
                    break
            else:
                self.groups.append(CacheGroup(need))
                gi = len(self.groups) - 1
            self.run_group[i] = (gi, len(self.groups[gi].layers))
            self.groups[gi].layers.append(i)
        # fixed-size state per request, for every run of a mixer that has some
        self.state_bytes = [self.blocks[r.layer].mixer.state_bytes() for r in self.runs]
        # a step of this model can be captured in a CUDA graph if no part reads the host-side entry list
        self.graph_safe = all(getattr(p, "graph_safe", False)
                              for p in [self.embedding, self.head] + [blk.mixer for blk in self.blocks])

    def declare(self) -> List[TensorDecl]:
        decls = self.embedding.declare()
        for blk in self.blocks:
            decls += blk.declare()
        return decls + self.final_norm.declare() + self.head.declare()

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.embedding.bind(tensors, rt)
        for blk in self.blocks:
            blk.bind(tensors, rt)
        self.final_norm.bind(tensors, rt)
        self.head.bind(tensors, rt, self.embedding)
        if hasattr(rt.ops, "set_weight_order"):  # the step's weight stream, in order of use
            order = [w for r in self.runs for w in self.blocks[r.layer].streamed_weights()]
            rt.ops.set_weight_order(order + self.head.streamed_weights())
        # stretches of the schedule that a decode step of few rows runs as one launch
        self.stacks = plan_stacks(self.blocks, self.runs, self.run_owner, self.run_group, rt)

    # ------------------------------------------------------------------ the forward pass of one step
    def forward(self, ctx: StepContext, cache, rows: torch.Tensor, num_rows: int) -> torch.Tensor:
        """Runs the step's tokens through the model; returns float32 logits [num_rows, vocab]
        at the flat-batch rows listed in ``rows`` (a device int32 array)."""
        resid = self.embedding.forward(ctx)
        delta = None
        view_of = lambda k: cache.layer_view(self.run_owner[k], writes=self.runs[k].cache_of is None, state_run=k)  # noqa: E731
        # decode steps of few rows: stretches of layers as one launch (off by default), or as a chain of streamed linears
        # with the norms folded into them
        stacks = self.stacks if (self.stacks and ctx.decode_only and ctx.T == ctx.S and ctx.T <= STACK_MAX_ROWS) else {}
        one_launch = getattr(self.rt.ops, "fused_layers", False)
        i = 0
        while i < len(self.runs):
            stack = stacks.get(i)
            if stack is not None and one_launch and stack.supports(ctx.T):
                stack.forward(resid, delta, ctx, [view_of(k) for k in range(stack.first, stack.end)])
                delta, i = None, stack.end
                continue
            if stack is not None and stack.chain_supports(ctx.T):
                stack.forward_chain(resid, delta, ctx, [view_of(k) for k in range(stack.first, stack.end)])
                delta, i = None, stack.end
                continue
            delta = self.blocks[self.runs[i].layer].forward(resid, delta, ctx, view_of(i))
            i += 1
        if num_rows == 0:
            join = getattr(self.rt.ops, "join_side_work", None)
            if join is not None:
                join()
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.rt.device)
        h = self.final_norm.forward(resid, delta, ctx, rows=rows, num_rows=num_rows)
        logits = self.head.forward(h, ctx)
        join = getattr(self.rt.ops, "join_side_work", None)
        if join is not None:
            join()
        return logits
