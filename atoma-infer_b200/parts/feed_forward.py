"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(models/src/llama.rs:362-366, 370-374).  Gate and up are one stacked matrix here.

Parameters: ``hidden``, ``intermediate``.  Checkpoint tensors:
``<prefix>.{gate,up,down}_proj.weight``.
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import FeedForward


class SwiGLU(FeedForward):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])

    def activation_width(self):
        return 2 * self.intermediate

    def declare(self):
        pre = self.prefix
        return [
            TensorDecl(pre + ".gate_proj.weight", (self.intermediate, self.hidden)),
            TensorDecl(pre + ".up_proj.weight", (self.intermediate, self.hidden)),
            TensorDecl(pre + ".down_proj.weight", (self.hidden, self.intermediate)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre = self.prefix
        self.w_gate_up = torch.cat([tensors[pre + ".gate_proj.weight"], tensors[pre + ".up_proj.weight"]], 0).contiguous()
        self.w_down = tensors[pre + ".down_proj.weight"].contiguous()

    def streamed_weights(self):
        return [self.w_gate_up, self.w_down]

    def fused(self):
        return {"kind": "swiglu", "w_gate_up": self.w_gate_up, "w_down": self.w_down, "hidden": self.hidden,
                "intermediate": self.intermediate}

    def forward(self, x, ctx):
        ops = self.rt.ops
        act = ops.linear(x, self.w_gate_up, silu_mul=True, meta=ctx.meta)
        return ops.linear(act, self.w_down, meta=ctx.meta)


register_part("feed_forward", "swiglu", SwiGLU)
