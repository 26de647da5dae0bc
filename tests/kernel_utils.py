"""Hand-made step metadata and paged caches for testing kernels and parts one at a time."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from atoma_infer_b200.csrc import ops as O
from atoma_infer_b200.engine.step import MetaLayout
from atoma_infer_b200.parts.base import EntryInfo, Runtime, StepContext


def make_context(rt: Runtime, entries: Sequence[Tuple[int, int]], page_size: int, tables: Sequence[Sequence[int]],
                 tokens: Sequence[int] = (), rows: Sequence[int] = ()) -> Tuple[StepContext, torch.Tensor]:
    """``entries``: (context_len, num_tokens) per request; ``tables``: its block table (page ids by
    absolute page index).  Returns the context and the device array of wanted rows."""
    S, T, R = len(entries), sum(n for _, n in entries), len(rows)
    stride = max(len(t) for t in tables)
    lay = MetaLayout(T, S, R, (stride,))  # the engine's own layout: a change of it reaches these tests too
    off = {"tokens": lay.tokens, "positions": lay.positions, "token_entry": lay.token_entry, "cu": lay.cu,
           "ctx": lay.ctx, "slots": lay.slots, "rows": lay.rows, "tables": lay.tables[0]}
    h = np.zeros(lay.size, dtype=np.int32)
    h[O.META_NUM_TOKENS], h[O.META_NUM_ENTRIES], h[O.META_NUM_ROWS] = T, S, R
    h[O.META_BT_STRIDE], h[O.META_BT_OFFSET] = stride, off["tables"]
    infos, start = [], 0
    for k, (c, n) in enumerate(entries):
        h[off["positions"] + start:off["positions"] + start + n] = np.arange(c, c + n)
        h[off["token_entry"] + start:off["token_entry"] + start + n] = k
        h[off["cu"] + k], h[off["ctx"] + k], h[off["slots"] + k] = start, c, k
        row = np.full(stride, -1, dtype=np.int32)
        row[:len(tables[k])] = tables[k]
        h[off["tables"] + k * stride:off["tables"] + (k + 1) * stride] = row
        infos.append(EntryInfo(k, start, n, c, k, c == 0))
        start += n
    h[off["cu"] + S] = T
    if len(tokens):
        h[off["tokens"]:off["tokens"] + T] = np.asarray(tokens)
    if R:
        h[off["rows"]:off["rows"] + R] = np.asarray(rows)
    dev = torch.from_numpy(h).to(rt.device)
    v = lambda name, n: dev[off[name]:off[name] + n]  # noqa: E731
    ctx = StepContext(rt=rt, T=T, S=S, meta=dev, tokens=v("tokens", T), positions=v("positions", T),
                      token_entry=v("token_entry", T), cu_tokens=v("cu", S + 1), context_lens=v("ctx", S),
                      state_slots=v("slots", S), entries=infos,
                      max_tokens_per_entry=max(n for _, n in entries), max_context=max(c + n for c, n in entries),
                      decode_only=all(n == 1 for _, n in entries), page_size=page_size,
                      table_offsets=tuple(lay.tables), table_strides=(stride,))
    return ctx, v("rows", max(R, 1))


def scrambled_tables(lengths: Sequence[int], page_size: int, seed: int = 0) -> Tuple[List[List[int]], int]:
    """Block tables for requests of the given total lengths with pages dealt in a random physical
    order (the reference tests this too, models/src/llama.rs:920-1152).  Returns (tables, num_pages)."""
    need = [-(-n // page_size) for n in lengths]
    total = sum(need) + 3
    rng = np.random.RandomState(seed)
    ids = (rng.permutation(total - 1) + 1).tolist()  # page 0 is never handed out
    tables, at = [], 0
    for n in need:
        tables.append(ids[at:at + n])
        at += n
    return tables, total


def fill_cache(cache: torch.Tensor, tables, keys: Sequence[torch.Tensor], values: Sequence[torch.Tensor], page_size: int):
    """cache [pages, 2, kv_heads, page_size, d]; keys/values per request [len, kv_heads, d]."""
    for t, k, v in zip(tables, keys, values):
        for pos in range(k.shape[0]):
            page, slot = t[pos // page_size], pos % page_size
            cache[page, 0, :, slot] = k[pos].to(cache.dtype)
            cache[page, 1, :, slot] = v[pos].to(cache.dtype)
