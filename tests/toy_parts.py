"""Toy parts for the tests of the parts layer's generality.  They live under tests/ only and are written
with tensor operations (they show that the interfaces suffice, not how fast kernels look): nothing here
is a model of anyone's, and the package never imports it.

* ``RunningMeanMixer``: a mixer with fixed-size state of its own per request and no pages.
* ``LatentMixer``: a mixer that caches ONE latent vector per token (a one-tensor cache need), makes keys
  and values from the cached latents when it attends, and finds its pages through the block table.
* ``ScaledPositionalEmbedding``: an embedding stage that scales the token rows and adds a learned vector
  per absolute position.
* ``CappedBiasHead``: a head with a bias and a soft cap on the logits.
"""
from __future__ import annotations

import torch

from atoma_infer_b200.cache import CachedTensor, CacheNeed
from atoma_infer_b200.parts import Embedding, Head, Mixer
from atoma_infer_b200.weights import TensorDecl


class RunningMeanMixer(Mixer):
    """out[t] = W * mean(x[0..t]) over the request's tokens so far.  Its state (running sum and
    count) is fixed-size per request and lives in the engine's state slots; it keeps no pages."""

    graph_safe = False  # walks the host-side entry list

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden"])

    def state_bytes(self):
        return 4 * (self.hidden + 1)

    def declare(self):
        return [TensorDecl(self.prefix + ".mix.weight", (self.hidden, self.hidden))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w = tensors[self.prefix + ".mix.weight"].float()

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        state = cache.state.view(torch.float32)  # [slots, hidden + 1]
        for e in ctx.entries:
            rows = slice(e.start, e.start + e.num_tokens)
            s = state[e.state_slot]
            sums = s[:self.hidden] + torch.cumsum(x[rows].float(), 0)
            counts = s[self.hidden] + torch.arange(1, e.num_tokens + 1, device=x.device, dtype=torch.float32)
            out[rows] = ((sums / counts[:, None]) @ self.w.T).to(x.dtype)
            s[:self.hidden] = sums[-1]
            s[self.hidden] = counts[-1]
        return out


class LatentMixer(Mixer):
    """Caches c[t] = Wc x[t] (one head of ``latent`` elements) and attends with q = Wq x, k = Wk c, v = Wv c
    over all cached tokens of the request, causally; out = Wo o.  One head, scale 1/sqrt(dim)."""

    graph_safe = False

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden, self.latent, self.dim = int(params["hidden"]), int(params["latent"]), int(params["dim"])

    def cache_need(self):
        return CacheNeed((CachedTensor("latent", 1, self.latent),))

    def declare(self):
        p, h, c, d = self.prefix, self.hidden, self.latent, self.dim
        return [TensorDecl(p + ".c.weight", (c, h)), TensorDecl(p + ".q.weight", (d, h)), TensorDecl(p + ".k.weight", (d, c)),
                TensorDecl(p + ".v.weight", (d, c)), TensorDecl(p + ".o.weight", (h, d))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w = {n: tensors[f"{self.prefix}.{n}.weight"].float() for n in "cqkvo"}

    def forward(self, x, ctx, cache):
        out = torch.zeros_like(x)
        pages = cache.tensors["latent"]            # [num_pages, 1, page_size, latent]
        table = ctx.block_table(cache.group)       # [S, pages per request]
        ps = cache.page_size
        for k, e in enumerate(ctx.entries):
            rows = slice(e.start, e.start + e.num_tokens)
            xf = x[rows].float()
            total = e.context_len + e.num_tokens
            where = torch.arange(total, device=x.device)
            page, slot = table[k][(where // ps).long()].long(), (where % ps).long()
            new = slice(e.context_len, total)
            pages[page[new], 0, slot[new]] = (xf @ self.w["c"].T).to(pages.dtype)
            c = pages[page, 0, slot].float()       # every cached latent of the request, this step's included
            q, kk, vv = xf @ self.w["q"].T, c @ self.w["k"].T, c @ self.w["v"].T
            s = (q @ kk.T) / self.dim ** 0.5
            s = s.masked_fill(where[None, :] > where[new][:, None], float("-inf"))
            out[rows] = ((torch.softmax(s, -1) @ vv) @ self.w["o"].T).to(x.dtype)
        return out


class ScaledPositionalEmbedding(Embedding):
    """resid[t] = scale * E[token[t]] + P[position[t]]."""

    graph_safe = True  # tokens and positions are read on the device

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab, self.hidden, self.max_position = int(params["vocab"]), int(params["hidden"]), int(params["max_position"])
        self.scale = float(params["scale"])

    def declare(self):
        return [TensorDecl("embed.tokens", (self.vocab, self.hidden)), TensorDecl("embed.positions", (self.max_position, self.hidden))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.tokens, self.positions = tensors["embed.tokens"], tensors["embed.positions"].float()

    def table(self):
        return self.tokens

    def forward(self, ctx):
        resid = torch.empty((ctx.T, self.hidden), dtype=torch.float32, device=self.rt.device)
        self.rt.ops.embed(ctx.tokens, self.tokens, resid, ctx.meta, ctx.T, scale=self.scale)
        resid += self.positions[ctx.positions.long()]
        return resid


class CappedBiasHead(Head):
    """logits = cap * tanh((h W^T + b) / cap), W the embedding's token table."""

    graph_safe = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab, self.cap = int(params["vocab"]), float(params["cap"])

    def declare(self):
        return [TensorDecl("head.bias", (self.vocab,))]

    def bind(self, tensors, rt, embedding=None):
        super().bind(tensors, rt, embedding)
        self.weight, self.bias = embedding.table(), tensors["head.bias"].float()

    def forward(self, h, ctx):
        logits = self.rt.ops.linear(h, self.weight, out_dtype=torch.float32, meta=ctx.meta, use_rows=True)
        return self.cap * torch.tanh((logits + self.bias) / self.cap)
