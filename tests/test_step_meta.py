"""The step's metadata buffer, built natively, against a plain restatement of its layout (no GPU):
random mixes of prompt portions and decode tokens over two cache groups (all keys; a window), with
and without padding to a captured graph's sizes; and what a refused entry leaves behind."""
import random
from types import SimpleNamespace

import numpy as np
import pytest

from atoma_infer_b200.cache import CacheGroup, CacheManager, CacheNeed, OutOfPages
from atoma_infer_b200.csrc.ops import (META_BT_OFFSET, META_BT_STRIDE, META_HEADER_INTS, META_NUM_ENTRIES, META_NUM_ROWS,
                                       META_NUM_TOKENS)
from atoma_infer_b200.engine.step import StepEntry, StepFunction

VOCAB = 97


def make(pages=40, page_size=4, max_seqs=6, window=6):
    groups = [CacheGroup(CacheNeed.kv(2, 16, None), [0], pages + 1), CacheGroup(CacheNeed.kv(1, 32, window), [1], pages + 1)]
    m = CacheManager(page_size, groups, max_seqs)
    step = StepFunction(SimpleNamespace(spec=SimpleNamespace(vocab_size=VOCAB)), None, m, None)
    return m, step


def plain_buffer(m, entries, before, pad_to):
    """The layout in words: header; tokens, positions, entry of each token (T each); starts of the entries' tokens
    (S + 1); tokens cached before the step, state slots (S each); wanted rows (at least one place); one block table per
    group, a row an entry, -1 where no page is held."""
    T, S, R = (max(x, pad_to) for x in (sum(len(e.tokens) for e in entries), len(entries), sum(len(e.want) for e in entries)))
    tokens, positions, owner, cu, ctx, slots, rows = [], [], [], [], [], [], []
    for k, e in enumerate(entries):
        cu.append(len(tokens))
        rows += [len(tokens) + w for w in e.want]
        tokens += list(e.tokens)
        positions += [before[e.req] + i for i in range(len(e.tokens))]
        owner += [k] * len(e.tokens)
        ctx.append(before[e.req])
        slots.append(m.state_slot(e.req))
    true = (len(tokens), len(entries), len(rows))
    pad = lambda a, n, v=0: a + [v] * (n - len(a))  # noqa: E731
    body = pad(tokens, T) + pad(positions, T) + pad(owner, T) + pad(cu, S + 1, true[0]) + pad(ctx, S) + pad(slots, S) + pad(rows, max(R, 1))
    head = [0] * META_HEADER_INTS
    head[META_NUM_TOKENS], head[META_NUM_ENTRIES], head[META_NUM_ROWS] = true
    off = META_HEADER_INTS + len(body)
    tables = []
    for g in range(len(m.groups)):
        stride = max(len(m.table(e.req, g)) for e in entries)
        head[META_BT_STRIDE + g], head[META_BT_OFFSET + g] = stride, off + len(tables)
        for k in range(S):
            tables += pad(m.table(entries[k].req, g), stride, -1) if k < len(entries) else [-1] * stride
    return np.asarray(head + body + tables, dtype=np.int32)


@pytest.mark.parametrize("seed", range(6))
def test_native_metadata_equals_the_plain_layout(seed):
    rng = random.Random(seed)
    m, step = make()
    live, next_id = {}, 1
    for _ in range(40):
        entries = []
        for req in rng.sample(sorted(live), k=min(len(live), rng.randint(0, 3))):
            n = rng.choice([1, 1, 2, 5])
            entries.append(StepEntry(req, [rng.randrange(VOCAB) for _ in range(n)], sorted(rng.sample(range(n), rng.randint(0, min(n, 2))))))
        while len(live) + sum(e.req not in live for e in entries) < 4 and rng.random() < 0.5:
            n = rng.randint(1, 9)
            entries.append(StepEntry(next_id, [rng.randrange(VOCAB) for _ in range(n)], [n - 1] if rng.random() < 0.5 else []))
            next_id += 1
        if not entries:
            continue
        rng.shuffle(entries)
        before = {e.req: (m.num_tokens(e.req) if m.has_request(e.req) else 0) for e in entries}
        pad_to = rng.choice([0, 0, 16]) if sum(len(e.tokens) for e in entries) <= 16 else 0
        host, lay, infos, R = step.prepare(entries, pad_to=pad_to)
        assert np.array_equal(host.numpy(), plain_buffer(m, entries, before, pad_to))
        assert [(i.req, i.start, i.num_tokens, i.context_len, i.is_new) for i in infos] == \
               [(e.req, int(host[lay.cu + k]), len(e.tokens), before[e.req], before[e.req] == 0) for k, e in enumerate(entries)]
        assert R == sum(len(e.want) for e in entries)
        for e in entries:
            m.advance(e.req, len(e.tokens))
            live[e.req] = True
        for req in [r for r in live if m.num_tokens(r) > 30 or rng.random() < 0.1]:
            m.free_request(req)
            del live[req]
        assert m.audit() == ""
    for req in live:
        m.free_request(req)
    assert m.audit() == "" and all(m.num_free_pages(g) == m.num_usable_pages(g) for g in range(2))


def test_a_refused_entry_leaves_nothing_behind():
    m, step = make(pages=3)
    free = [m.num_free_pages(g) for g in range(2)]
    for entries, what in (([StepEntry(1, [], [])], "no tokens"), ([StepEntry(1, [1, 2], [2])], "wanted place"),
                          ([StepEntry(1, [1, 2], [-1])], "wanted place"), ([StepEntry(1, [VOCAB], [0])], "token ids"),
                          ([StepEntry(1, [-1], [0])], "token ids")):
        with pytest.raises(ValueError, match=what):
            step.prepare(entries)
        assert m.num_requests() == 0 and [m.num_free_pages(g) for g in range(2)] == free and m.audit() == ""
    with pytest.raises(ValueError, match="twice"):
        step.prepare([StepEntry(1, [1], [0]), StepEntry(1, [2], [0])])
    assert m.num_requests() == 1  # the first of the two stays, as after a step that ran
    m.free_request(1)
    with pytest.raises(OutOfPages):  # 13 tokens need 4 pages of 4 in the group that keeps all keys
        step.prepare([StepEntry(2, list(range(13)), [])])
    assert m.num_requests() == 0 and [m.num_free_pages(g) for g in range(2)] == free and m.audit() == ""
    step.prepare([StepEntry(3, list(range(12)), [11])])
    m.advance(3, 12)
    with pytest.raises(OutOfPages):
        step.prepare([StepEntry(3, [5], [0])])
    assert m.num_tokens(3) == 12 and m.audit() == ""  # a request that was live keeps what it held
