"""Interfaces of the parts a model is put together from.

A model is a list of layers; a layer is a block that arranges a mixer (attention
here), a feed-forward and norms around the residual stream.  Each part takes its
sizes and constants as parameters (a plain dict in the model spec) and does not
know which model it is in.  The reference hard-wires one arrangement
(models/src/llama.rs:203-430: CausalSelfAttention, Mlp, Block); the split below is
this engine's, so that another mixer or feed-forward can stand in any layer.

Life of a part: ``__init__(params, prefix)`` from the spec; ``declare()`` lists the
checkpoint tensors it needs; ``bind(tensors, rt)`` receives them on the device;
``forward`` runs inside a step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..cache.spec import CacheNeed, LayerCache
from ..weights.loader import TensorDecl


@dataclass
class Runtime:
    """What a bound part may use: the device, the compute dtype and the kernels."""

    device: torch.device
    dtype: torch.dtype
    ops: Any


@dataclass
class EntryInfo:
    """One request's share of a step, as the host sees it."""

    req: int
    start: int        # first row of the request's tokens in the step's flat batch
    num_tokens: int
    context_len: int  # tokens of the request already in the cache
    state_slot: int
    is_new: bool      # first step of the request: fixed-size state starts from zero


@dataclass
class StepContext:
    """Everything a part may read about the step under way.

    Device arrays are int32 views into one metadata buffer that the step function
    uploads in a single copy; sizes in capitals are the launch sizes (what buffers
    are padded to), the true ones stand in the metadata header for the kernels.
    """

    rt: Runtime
    T: int                       # rows of the flat batch
    S: int                       # entries (requests) in the batch
    meta: torch.Tensor           # header + arrays (csrc/kernels/common.cuh)
    tokens: torch.Tensor         # [T]
    positions: torch.Tensor      # [T] absolute position of each token in its request
    token_entry: torch.Tensor    # [T] index of the entry a token belongs to
    cu_tokens: torch.Tensor      # [S + 1] first row of each entry
    context_lens: torch.Tensor   # [S]
    state_slots: torch.Tensor    # [S]
    entries: List[EntryInfo] = field(default_factory=list)
    max_tokens_per_entry: int = 0
    max_context: int = 0         # longest context_len + num_tokens in the batch
    decode_only: bool = False    # every entry brings exactly one token
    page_size: int = 0
    table_offsets: Sequence[int] = ()   # per cache group: where its block tables start in ``meta`` ...
    table_strides: Sequence[int] = ()   # ... and how long a request's row is

    def block_table(self, group: int) -> torch.Tensor:
        """The block tables of a cache group as a device view [S, pages per request]: entry k's row lists its
        page ids by absolute page index (-1: no page).  For parts written with tensor operations; the
        kernels read the same memory through ``meta``."""
        off, stride = self.table_offsets[group], self.table_strides[group]
        return self.meta[off:off + self.S * stride].view(self.S, stride)


class Part:
    """Base of all parts: parameters from the spec, tensors by checkpoint name."""

    def __init__(self, params: Dict[str, Any], prefix: str):
        self.params = dict(params)
        self.prefix = prefix

    def declare(self) -> List[TensorDecl]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt

    def streamed_weights(self) -> List[torch.Tensor]:
        """The weight matrices of the part's linears in the order ``forward`` uses them (after ``bind``).  The model
        hands the whole step's list to the kernels, which may fetch a weight ahead of its use."""
        return []

    def activation_width(self) -> int:
        """Elements per token of the widest intermediate result the part makes (0: nothing wider than the
        model's width); the engine sizes its working memory from it when it sizes the cache."""
        return 0

    def fused(self) -> Optional[Dict[str, Any]]:
        """What a kernel that runs several parts at once needs to know of this part (after ``bind``): a dict with
        ``kind``, the part's tensors and constants.  None (the default): the part only runs through ``forward``."""
        return None


class Embedding(Part):
    """The first stage: the step's token ids (and whatever else of the step's metadata it wants, positions
    for instance) become the float32 residual stream.  ``graph_safe = True`` on a subclass says that its
    ``forward`` reads the step's metadata on the device only, so a decode step may be captured in a graph."""

    graph_safe = False

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """Returns the residual stream, float32 [ctx.T, hidden]."""
        raise NotImplementedError

    def table(self) -> Optional[torch.Tensor]:
        """The [vocab, hidden] matrix, for a head that is tied to it (None: there is no such matrix)."""
        return None


class Head(Part):
    """The last stage: normed rows become float32 logits over the vocabulary (``graph_safe`` as for the
    embedding)."""

    graph_safe = False

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime, embedding: Optional["Embedding"] = None) -> None:
        """``embedding``: the model's first stage, for a head that shares its matrix."""
        self.rt = rt

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """``h`` [rows, hidden] in the compute dtype; returns float32 [rows, vocab]."""
        raise NotImplementedError


class Norm(Part):
    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext,
                rows: Optional[torch.Tensor] = None, num_rows: int = 0) -> torch.Tensor:
        """Adds ``delta`` into the float32 residual stream (if given) and returns the normed
        rows in the compute dtype.  With ``rows``: only those rows, residual left untouched."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions enter a mixer.  For attention: ``encode_and_store`` turns the fused
    q|k|v rows of a step into position-encoded queries (in place) and writes keys and
    values to the layer's pages."""

    def encode_and_store(self, qkv: torch.Tensor, ctx: StepContext, cache: LayerCache, *, num_heads: int,
                         num_kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError

    def rotary(self):
        """(inv_freq on the device, rotary_dim) if the encoding is a rotation by position times
        frequency, which the decode attention kernel can apply itself; None otherwise."""
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request."""

    def cache_need(self) -> Optional[CacheNeed]:
        """Keys/values per cached token, or None if the mixer keeps no pages."""
        return None

    def state_bytes(self) -> int:
        """Bytes of fixed-size state per request (0: none)."""
        return 0

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arranges norms, mixer and feed-forward around the residual stream.

    ``forward(resid, delta, ctx, cache)``: ``resid`` is the float32 residual stream
    [T, H], ``delta`` what the previous block left to be added (None at the first);
    returns this block's own pending addition.  Keeping the last addition pending lets
    the next norm do it, in float32, in the same pass."""

    mixer: Mixer

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError

    def decode_fusion(self) -> Optional[Dict[str, Any]]:
        """For a kernel that runs a run of whole layers of a decode step: this block's arrangement and what its
        parts say of themselves (``Part.fused``), or None if the block, or one of its parts, cannot take part."""
        return None
