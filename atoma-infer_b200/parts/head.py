"""Output head: logits = h * W^T in the compute dtype, returned as float32 (models/src/llama.rs:476-477);
W is the embedding matrix when the model ties them (:482-486).  No bias.

Parameters: ``vocab``, ``hidden``, ``tensor`` (checkpoint name of the [vocab, hidden] matrix; None: the
embedding's matrix).
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import Head


class LinearHead(Head):
    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.tensor = params.get("tensor")

    def declare(self):
        return [TensorDecl(self.tensor, (self.vocab, self.hidden))] if self.tensor else []

    def bind(self, tensors, rt, embedding=None):
        super().bind(tensors, rt, embedding)
        if self.tensor:
            self.weight = tensors[self.tensor]
        else:
            self.weight = embedding.table() if embedding is not None else None
            if self.weight is None or tuple(self.weight.shape) != (self.vocab, self.hidden):
                raise ValueError("a head without a matrix of its own needs an embedding with a [vocab, hidden] table")

    def streamed_weights(self):
        return [self.weight]

    def forward(self, h, ctx):
        return self.rt.ops.linear(h, self.weight, out_dtype=torch.float32, meta=ctx.meta, use_rows=True)


register_part("head", "linear", LinearHead)
