"""Pre-norm residual block: h = x + mixer(norm1(x)); out = h + ff(norm2(h))
(models/src/llama.rs:393-410).  The residual stream is float32 and each addition
happens inside the norm that follows it.

Parameters: ``norm`` (spec of both norms), ``mixer``, ``feed_forward`` (specs), and
the names of the four parts inside the layer's prefix (``names``).
"""
from __future__ import annotations

from ..config.registry import part_class, register_part
from .base import Block

_DEFAULT_NAMES = {"norm1": "input_layernorm", "mixer": "self_attn", "norm2": "post_attention_layernorm",
                  "feed_forward": "mlp"}


class PreNormBlock(Block):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        names = {**_DEFAULT_NAMES, **(params.get("names") or {})}
        mk = lambda fam, spec, name: part_class(fam, spec["kind"])(spec, f"{prefix}.{name}")  # noqa: E731
        self.norm1 = mk("norm", params["norm"], names["norm1"])
        self.mixer = mk("mixer", params["mixer"], names["mixer"])
        self.norm2 = mk("norm", params["norm"], names["norm2"])
        self.feed_forward = mk("feed_forward", params["feed_forward"], names["feed_forward"])

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def streamed_weights(self):
        return self.mixer.streamed_weights() + self.feed_forward.streamed_weights()

    def activation_width(self):
        return max(p.activation_width() for p in self.parts())

    def declare(self):
        return [d for p in self.parts() for d in p.declare()]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        for p in self.parts():
            p.bind(tensors, rt)

    def decode_fusion(self):
        parts = {"norm1": self.norm1.fused(), "mixer": self.mixer.fused(), "norm2": self.norm2.fused(),
                 "feed_forward": self.feed_forward.fused()}
        if any(v is None for v in parts.values()):
            return None
        return {"kind": "prenorm", **parts}

    def forward(self, resid, delta, ctx, cache):
        h = self.norm1.forward(resid, delta, ctx)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norm2.forward(resid, a, ctx)
        return self.feed_forward.forward(h, ctx)


register_part("block", "prenorm", PreNormBlock)
