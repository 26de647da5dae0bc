"""A stand-in for the kernel table, for tests of the host side only (engine loop, scheduler, sampler
plumbing, error handling) where no GPU is: the same calls as ``csrc/ops.py`` answered with slow torch
code on the CPU.  It is test material: nothing of the package imports it, and the package has no CPU
path of its own.  The math follows the plain implementation (plain_llama.py), read from the same step
metadata and pages that the kernels read.
"""
from __future__ import annotations

import torch

import plain_llama as P
from atoma_infer_b200.csrc.ops import (META_BT_OFFSET, META_BT_STRIDE, META_NUM_ROWS, META_NUM_TOKENS, STATUS_WORDS,
                                       CudaOps)


class HostOps:
    describe_status = staticmethod(CudaOps.describe_status)

    def __init__(self):
        self.device = torch.device("cpu")
        self.launches = 0
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32)
        self.last_tokens = torch.zeros(1 << 10, dtype=torch.int32)
        self.fused_rope = False
        self.fail_at_launch = None  # (launch number, status word, value): raise a status word there, as a kernel would

    def _count(self):
        self.launches += 1
        if self.fail_at_launch and self.launches >= self.fail_at_launch[0]:
            _, word, value = self.fail_at_launch
            self.status[word] = value
            self.fail_at_launch = None

    def clear_status(self):
        self.status.zero_()

    def check_status(self):
        what = self.describe_status(self.status.tolist())
        if what:
            self.clear_status()
            raise RuntimeError("device status: " + what)

    def fast_attention(self, *a):
        return False

    def embed(self, tokens, table, resid, meta, T, scale=1.0):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        tok = tokens[:n].long()
        neg = tok < 0
        tok = torch.where(neg, self.last_tokens[(-tok - 1).clamp(min=0)].long(), tok)
        resid[:n] = scale * table[tok].float()

    def add_rmsnorm(self, resid, delta, w, eps, out, meta, n, rows=None):
        self._count()
        if rows is None:
            n = int(meta[META_NUM_TOKENS])
            if delta is not None:
                resid[:n] += delta[:n].float()
            x = resid[:n]
        else:
            n = int(meta[META_NUM_ROWS])
            r = rows[:n].long()
            x = resid[r] + (delta[r].float() if delta is not None else 0)
        out[:n] = P.rms_norm(x, w, eps).to(out.dtype)

    def linear(self, x, w, *, out_dtype=None, silu_mul=False, meta=None, use_rows=False):
        self._count()
        y = x.float() @ w.float().T
        if silu_mul:
            inter = w.shape[0] // 2
            g, u = y[:, :inter], y[:, inter:]
            y = g * torch.sigmoid(g) * u
        return y.to(out_dtype or x.dtype)

    def rope_kv_store(self, qkv, positions, token_entry, meta, group, inv_freq, cache, num_pages, T, nq, nkv, d, rot,
                      page_size, store_kv):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        off, stride = int(meta[META_BT_OFFSET + group]), int(meta[META_BT_STRIDE + group])
        rows = qkv[:n].view(n, nq + 2 * nkv, d).float()
        pos = positions[:n]
        qk = rows[:, :nq + nkv].clone()
        qk[..., :rot] = P.rope(qk[..., :rot], pos, inv_freq)
        qkv[:n].view(n, nq + 2 * nkv, d)[:, :nq] = qk[:, :nq].to(qkv.dtype)
        if store_kv:
            for t in range(n):
                p = int(pos[t])
                page = int(meta[off + int(token_entry[t]) * stride + p // page_size])
                if not 0 < page < num_pages:
                    self.status[1] = t + 1
                    continue
                cache[page, 0, :, p % page_size] = qk[t, nq:].to(cache.dtype)
                cache[page, 1, :, p % page_size] = rows[t, nq + nkv:].to(cache.dtype)

    def attention(self, q, q_stride, cache, ctx, group, out, nq, nkv, d, page_size, num_pages, window, scale, rope=None):
        self._count()
        meta = ctx.meta
        n = int(meta[META_NUM_TOKENS])
        off, stride = int(meta[META_BT_OFFSET + group]), int(meta[META_BT_STRIDE + group])
        for t in range(n):
            pos, e = int(ctx.positions[t]), int(ctx.token_entry[t])
            first = max(0, pos - window + 1) if window else 0
            idx = range(first, pos + 1)
            pages = [int(meta[off + e * stride + j // page_size]) for j in idx]
            k = torch.stack([cache[p, 0, :, j % page_size] for p, j in zip(pages, idx)]).float()  # [keys, nkv, d]
            v = torch.stack([cache[p, 1, :, j % page_size] for p, j in zip(pages, idx)]).float()
            qq = q[t].view(-1, d)[:nq].float()
            g = nq // nkv
            for h in range(nq):
                w = torch.softmax((k[:, h // g] @ qq[h]) * scale, 0)
                out[t, h * d:(h + 1) * d] = (w @ v[:, h // g]).to(out.dtype)

    def sample(self, logits, temperature, top_k, top_p, seed, step, out, num_rows=None, slots=None):
        self._count()
        import numpy as np

        seeds = seed.numpy().view(np.uint64)
        steps = step.numpy().view(np.uint64)
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t == 0.0:
                tok = P.greedy(logits[r])
            else:
                tok = P.sample(logits[r], temperature=t, seed=int(seeds[r]), step=int(steps[r]), top_k=int(top_k[r]),
                               top_p=float(top_p[r]))
            out[r] = tok
            if slots is not None:
                self.last_tokens[int(slots[r])] = tok

    def repeat_penalty(self, row, penalty, context):
        self._count()
        row.copy_(P.apply_repeat_penalty(row, penalty, context.tolist()))
