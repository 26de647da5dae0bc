"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in float32, rounded once.

The reference uses candle's RmsNorm for input_layernorm, post_attention_layernorm
and model.norm (models/src/llama.rs:402, 408, 416-421, 474, 487).  Parameters:
``size`` and ``eps`` (config.json's rms_norm_eps).  Checkpoint tensor: ``<prefix>.weight``.
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import Norm


class RMSNorm(Norm):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])

    def declare(self):
        return [TensorDecl(self.prefix + ".weight", (self.size,), init="ones")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.prefix + ".weight"].to(torch.float32).contiguous()  # exact widening

    def forward(self, resid, delta, ctx, rows=None, num_rows=0):
        n = num_rows if rows is not None else ctx.T
        out = torch.empty((n, self.size), dtype=self.rt.dtype, device=resid.device)
        self.rt.ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, ctx.meta, n, rows=rows)
        return out

    def fused(self):
        return {"kind": "rmsnorm", "weight": self.weight, "eps": self.eps, "size": self.size}


register_part("norm", "rmsnorm", RMSNorm)
