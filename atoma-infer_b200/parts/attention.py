"""Grouped-query attention over the paged cache.

q, k, v projections without bias (one fused matrix here, three in the reference,
models/src/llama.rs:269-271), position encoding of q and k, keys and values written
to the request's pages, then for the query at position p of a request: scores
scale * q.k_j for j <= p (and p - j < window if the layer has one) over everything
the request has cached, softmax in float32, weighted sum of values; query head h
reads key/value head h // (heads / kv_heads) (csrc/kernels/flash_fwd_kernel.h:153,
159).  Output projection (models/src/llama.rs:310-311).  A portion of a prompt
attends to the portions before it through the block table; the reference's glue
misses that case (models/src/flash_attention.rs:384-410).

Parameters: ``hidden``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``,
``window`` (None: all keys), ``position`` (spec of the position encoding).
Checkpoint tensors: ``<prefix>.{q,k,v,o}_proj.weight``.
"""
from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..config.registry import part_class, register_part
from ..weights.loader import TensorDecl
from .base import Mixer


class Attention(Mixer):
    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.hidden = int(p["hidden"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        pos = dict(p.get("position") or {"kind": "none"})
        pos.setdefault("head_dim", self.head_dim)
        self.position = part_class("position", pos["kind"])(pos, prefix)

    @property
    def q_size(self):
        return self.num_heads * self.head_dim

    @property
    def kv_size(self):
        return self.num_kv_heads * self.head_dim

    def activation_width(self):
        return self.q_size + 2 * self.kv_size

    def streamed_weights(self):
        return [self.w_qkv, self.w_o]

    def cache_need(self):
        return CacheNeed.kv(self.num_kv_heads, self.head_dim, self.window)

    def declare(self):
        pre = self.prefix
        return [
            TensorDecl(pre + ".q_proj.weight", (self.q_size, self.hidden)),
            TensorDecl(pre + ".k_proj.weight", (self.kv_size, self.hidden)),
            TensorDecl(pre + ".v_proj.weight", (self.kv_size, self.hidden)),
            TensorDecl(pre + ".o_proj.weight", (self.hidden, self.q_size)),
        ] + self.position.declare()

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre = self.prefix
        # One matrix [q; k; v]: each output element is the same dot product as before.
        self.w_qkv = torch.cat([tensors[pre + ".q_proj.weight"], tensors[pre + ".k_proj.weight"],
                                tensors[pre + ".v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors[pre + ".o_proj.weight"].contiguous()
        self.position.bind(tensors, rt)

    def fused(self):
        rotary = self.position.rotary()
        if rotary is None:
            return None
        return {"kind": "attention", "w_qkv": self.w_qkv, "w_o": self.w_o, "hidden": self.hidden,
                "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim,
                "scale": self.scale, "window": int(self.window or 0), "inv_freq": rotary[0], "rotary_dim": rotary[1]}

    def forward(self, x, ctx, cache):
        ops = self.rt.ops
        qkv = ops.linear(x, self.w_qkv, meta=ctx.meta)
        # In a decode step the attention kernel can rotate q and write the new key and value itself.
        rope = None
        fast = getattr(ops, "fast_attention", None)
        if ctx.decode_only and getattr(ops, "fused_rope", True) and fast and fast(qkv.dtype, self.head_dim, self.num_heads, self.num_kv_heads, qkv.shape[1]):
            rotary = self.position.rotary()
            if rotary is not None:
                rope = (rotary[0], rotary[1], cache.writes and cache.pages is not None)
        if rope is None:
            self.position.encode_and_store(qkv, ctx, cache, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                                           head_dim=self.head_dim)
        out = torch.empty((ctx.T, self.q_size), dtype=x.dtype, device=x.device)
        ops.attention(qkv, qkv.shape[1], cache.pages, ctx, cache.group, out, self.num_heads, self.num_kv_heads,
                      self.head_dim, cache.page_size, cache.num_pages, int(self.window or 0), self.scale, rope=rope)
        return ops.linear(out, self.w_o, meta=ctx.meta)


register_part("mixer", "attention", Attention)
