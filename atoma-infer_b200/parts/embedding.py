"""Token embedding: resid[t] = scale * E[token[t]], widened to float32 (models/src/llama.rs:470, 481; the
reference has no scale, which is the default 1.0 here).

Parameters: ``vocab``, ``hidden``, ``tensor`` (checkpoint name of the [vocab, hidden] matrix), ``scale``.
A token id -1 - s stands for the token the sampler last left on the device for state slot s.
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import Embedding


class TokenEmbedding(Embedding):
    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.tensor = str(params.get("tensor") or "model.embed_tokens.weight")
        self.scale = float(params.get("scale", 1.0))

    def declare(self):
        return [TensorDecl(self.tensor, (self.vocab, self.hidden))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.tensor]

    def table(self):
        return self.weight

    def forward(self, ctx):
        resid = torch.empty((ctx.T, self.hidden), dtype=torch.float32, device=self.rt.device)
        self.rt.ops.embed(ctx.tokens, self.weight, resid, ctx.meta, ctx.T, scale=self.scale)
        return resid


register_part("embedding", "token", TokenEmbedding)
