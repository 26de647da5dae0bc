"""The attention kernels alone against the plain attention, at sizes other than the engine tests use:
head sizes 16..256, several group sizes and page sizes, contexts already in the cache, windows,
split key ranges, pages in scrambled physical order, a never-written (NaN) rest of the cache."""
import math

import pytest
import torch

import kernel_utils as K
import plain_llama as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rts():
    from atoma_infer_b200.engine.runtime import make_runtime

    return {"bfloat16": make_runtime("bfloat16", "cuda:0"), "float32": make_runtime("float32", "cuda:0")}


def run_attention(rt, entries, nq, nkv, d, page_size, window=None, seed=0, scale=None, splits=None, stand_out=None):
    """entries: (context_len, num_tokens).  Returns (engine output, plain output) lists per request,
    each [num_tokens, nq, d]."""
    g = torch.Generator().manual_seed(seed)
    lengths = [c + n for c, n in entries]
    tables, num_pages = K.scrambled_tables(lengths, page_size, seed)
    dt = rt.dtype
    qs = [torch.randn(L, nq, d, generator=g) for L in lengths]
    ks = [torch.randn(L, nkv, d, generator=g) for L in lengths]
    vs = [torch.randn(L, nkv, d, generator=g) for L in lengths]
    if isinstance(stand_out, tuple):  # ("plateau", far): see test_prefill_where_a_late_key_outgrows_the_base
        far = stand_out[1]
        for q, k in zip(qs, ks):
            u = torch.randn(nkv, d, generator=g)
            u = u / u.norm(dim=-1, keepdim=True) * math.sqrt(d)
            k[:far] = u + 0.1 * k[:far]
            k[far] = 1.75 * u
            q[-1] = u.repeat_interleave(nq // nkv, dim=0)
    elif stand_out is not None:  # one far key that the last query must find among all the others
        for q, k in zip(qs, ks):
            k[stand_out] *= 4.0
            q[-1] = k[stand_out].repeat_interleave(nq // nkv, dim=0) * 1.5
    qs, ks, vs = ([t.to(dt).float() for t in x] for x in (qs, ks, vs))  # the values the kernels will see
    cache = torch.full((num_pages, 2, nkv, page_size, d), float("nan"), dtype=dt, device=rt.device)
    K.fill_cache(cache, tables, ks, vs, page_size)
    ctx, _ = K.make_context(rt, entries, page_size, tables)
    T = ctx.T
    qkv = torch.zeros(T, (nq + 2 * nkv) * d, dtype=dt, device=rt.device)
    row = 0
    for (c, n), q in zip(entries, qs):
        qkv[row:row + n, :nq * d] = q[c:c + n].reshape(n, nq * d).to(dt)
        row += n
    out = torch.full((T, nq * d), float("nan"), dtype=dt, device=rt.device)
    scale = scale or 1.0 / math.sqrt(d)
    ops = rt.ops
    if splits is not None:
        ops.decode_splits = lambda *a: splits
    try:
        ops.attention(qkv, qkv.shape[1], cache, ctx, 0, out, nq, nkv, d, page_size, num_pages, int(window or 0), scale)
    finally:
        if splits is not None:
            del ops.decode_splits
    ops.check_status()
    got, want, row = [], [], 0
    for (c, n), q, k, v in zip(entries, qs, ks, vs):
        got.append(out[row:row + n].float().cpu().reshape(n, nq, d))
        if n == 1 and c >= 2048:  # a long context and one query: the plain function on the last row alone (the whole
            # score matrix of all rows would take gigabytes); rows before the last see nothing of it
            first = max(0, c - window + 1) if window else 0
            kk = k[first:c + 1].double().repeat_interleave(nq // nkv, dim=1)
            vv = v[first:c + 1].double().repeat_interleave(nq // nkv, dim=1)
            w = torch.softmax(torch.einsum("hd,shd->hs", q[c].double(), kk) * scale, dim=-1)
            want.append(torch.einsum("hs,shd->hd", w, vv)[None].float())
        else:
            want.append(P.causal_attention(q.double(), k.double(), v.double(), scale, window)[c:c + n].float())
        row += n
    return got, want


def worst(got, want):
    return max(float((a - b).abs().max()) for a, b in zip(got, want))


@pytest.mark.parametrize("d,nq,nkv,page", [(16, 4, 2, 4), (64, 3, 1, 8), (64, 32, 8, 16), (128, 8, 8, 16),
                                           (32, 6, 2, 64), (48, 5, 5, 16), (80, 16, 2, 16), (256, 2, 1, 16)])
def test_prefill_with_cached_context_bf16(rts, d, nq, nkv, page):
    entries = [(0, 70), (37, 29), (130, 2), (64, 1), (5, 131)]
    got, want = run_attention(rts["bfloat16"], entries, nq, nkv, d, page, seed=d)
    assert worst(got, want) < 2e-2  # values are O(1); bfloat16 P and outputs


@pytest.mark.parametrize("d,nq,nkv,page", [(64, 8, 2, 16), (128, 6, 2, 16), (64, 3, 1, 8)])
def test_prefill_where_a_late_key_outgrows_the_base(rts, d, nq, nkv, page):
    """The tcgen05 kernel keeps the output in tensor memory and moves the base of its exponentials only when a
    row's maximum has grown by more than 2^8; then it scales the output there.  Here the last query of each request
    meets, in its third and later key tiles, a key whose score towers over everything before it (and, in the
    second request, a second such key further on), so the scaling runs, more than once, at a page's and a tile's edge."""
    rt = rts["bfloat16"]
    for entries, far in (([(0, 450)], 300), ([(130, 390)], 383), ([(0, 1100)], 1023)):
        got, want = run_attention(rt, entries, nq, nkv, d, page, seed=far, stand_out=far, scale=1.0)
        assert worst(got, want) < 3e-2, (entries, far)
        # a plateau of equal scores and then one key 2^8.7 (head size 64) above it: the hundreds of keys before it
        # still carry as much weight together as the one, so a wrong scaling of what was summed before would show
        got, want = run_attention(rt, entries, nq, nkv, d, page, seed=far, stand_out=("plateau", far))
        assert worst(got, want) < 3e-2, (entries, far, "plateau")
        assert float(want[-1][-1].abs().max()) > 0.05


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("d,nq,nkv,page,splits", [(64, 32, 8, 16, 1), (64, 32, 8, 16, 5), (128, 8, 2, 16, 3),
                                                  (16, 4, 2, 4, 2), (64, 3, 1, 8, 4), (256, 4, 1, 16, 2),
                                                  (96, 12, 4, 32, 7), (64, 32, 8, 16, 8), (64, 8, 2, 16, 11)])
def test_decode_with_splits_bf16(rts, d, nq, nkv, page, splits, cluster):
    """Splits of the key range merged inside a thread-block cluster (up to eight) or through scratch memory
    (any number; also what runs when the cluster merge is switched off).  Some requests are shorter than
    the number of splits, so some blocks have no key at all."""
    entries = [(0, 1), (1, 1), (31, 1), (32, 1), (300, 1), (777, 1), (63, 1)]
    ops = rts["bfloat16"].ops
    ops.decode_cluster = cluster
    try:
        got, want = run_attention(rts["bfloat16"], entries, nq, nkv, d, page, seed=splits, splits=splits)
    finally:
        ops.decode_cluster = True
    assert worst(got, want) < 2e-2


@pytest.mark.parametrize("d,nq,nkv", [(64, 32, 8), (128, 8, 2)])
def test_decode_of_one_long_request_takes_many_splits(rts, d, nq, nkv):
    """A long context of one or two requests is cut into more than eight splits (the engine's own choice, merged
    through scratch memory by the last block to arrive); one key far back stands out, so a lost split would show."""
    rt = rts["bfloat16"]
    lib = rt.ops._attention_library(d)
    for entries in ([(9000, 1)], [(9000, 1), (4100, 1)]):
        splits = rt.ops.decode_splits(len(entries), nkv, 9001, lib.attn_decode_blocks_per_sm())
        assert splits > 8, splits
        got, want = run_attention(rt, entries, nq, nkv, d, 16, seed=7, stand_out=1234, scale=1.0)
        assert worst(got, want) < 3e-2


@pytest.mark.parametrize("blocks", [1, 2, 5, 37, 444])
@pytest.mark.parametrize("d,nq,nkv,page", [(64, 32, 8, 16), (128, 8, 2, 16), (16, 4, 2, 4), (96, 12, 4, 32), (256, 2, 1, 16)])
def test_decode_flat_bf16(rts, d, nq, nkv, page, blocks):
    """The large-batch decode kernel: a fixed number of blocks share all key tiles evenly, a block's run of tiles
    may span several requests and head groups, a pair may be spread over many blocks (or lie inside one)."""
    entries = [(0, 1), (1, 1), (31, 1), (32, 1), (300, 1), (777, 1), (63, 1), (64, 1), (500, 1)]
    ops = rts["bfloat16"].ops
    ops._decode_flat_blocks = lambda *a: blocks
    try:
        got, want = run_attention(rts["bfloat16"], entries, nq, nkv, d, page, seed=blocks)
        assert worst(got, want) < 2e-2
        got, want = run_attention(rts["bfloat16"], entries, nq, nkv, d, page, seed=blocks, window=100)
        assert worst(got, want) < 2e-2
        got, want = run_attention(rts["bfloat16"], [(599, 1), (700, 1)], nq, nkv, d, page, seed=255, stand_out=255, scale=1.0)
        assert worst(got, want) < 3e-2
    finally:
        del ops._decode_flat_blocks


def test_cluster_and_scratch_merges_agree_bitwise(rts):
    """Both merges add the splits in split order with the same arithmetic: the same bits."""
    ops = rts["bfloat16"].ops
    entries = [(5, 1), (300, 1), (1029, 1)]
    outs = []
    for cluster in (True, False):
        ops.decode_cluster = cluster
        try:
            got, _ = run_attention(rts["bfloat16"], entries, 32, 8, 64, 16, seed=3, splits=6)
        finally:
            ops.decode_cluster = True
        outs.append(torch.cat(got))
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("d", list(range(16, 257, 16)))
def test_every_head_size_bf16(rts, d):
    """Head sizes in steps of 16 up to 256: portions of prompts, decode steps with fixed splits and with the
    large-batch kernel."""
    rt = rts["bfloat16"]
    got, want = run_attention(rt, [(0, 70), (37, 29), (130, 2)], 4, 2, d, 16, seed=d)
    assert worst(got, want) < 2e-2
    decode = [(0, 1), (31, 1), (300, 1), (63, 1)]
    got, want = run_attention(rt, decode, 4, 2, d, 16, seed=d, splits=3)
    assert worst(got, want) < 2e-2
    rt.ops._decode_flat_blocks = lambda *a: 5
    try:
        got, want = run_attention(rt, decode, 4, 2, d, 16, seed=d)
    finally:
        del rt.ops._decode_flat_blocks
    assert worst(got, want) < 2e-2


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_window_bf16_and_float32(rts, window):
    for dtype, tol in (("bfloat16", 2e-2), ("float32", 2e-5)):
        got, want = run_attention(rts[dtype], [(0, 150), (90, 40), (200, 3)], 4, 2, 64, 16, window=window, seed=window)
        assert worst(got, want) < tol, dtype
        got, want = run_attention(rts[dtype], [(0, 1), (99, 1), (100, 1), (340, 1)], 4, 2, 64, 16, window=window,
                                  seed=window, splits=3 if dtype == "bfloat16" else None)
        assert worst(got, want) < tol, dtype


@pytest.mark.parametrize("d,nq,nkv,page", [(16, 4, 2, 4), (64, 3, 1, 8), (40, 2, 2, 16), (200, 2, 1, 16), (256, 2, 2, 4)])
def test_plain_kernel_float32_any_head_size(rts, d, nq, nkv, page):
    entries = [(0, 70), (37, 29), (130, 2), (64, 1)]
    got, want = run_attention(rts["float32"], entries, nq, nkv, d, page, seed=d)
    assert worst(got, want) < 2e-5


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_a_far_key_among_hundreds_is_found(rts, dtype):
    """The last query matches one key far back; if any page or tile were skipped or misplaced the
    output would be an average of values instead of (almost) that key's value."""
    for far in (3, 64, 255, 256, 511):
        got, want = run_attention(rts[dtype], [(0, 600)], 4, 2, 64, 16, seed=far, stand_out=far, scale=1.0)
        assert worst(got, want) < (3e-2 if dtype == "bfloat16" else 1e-4)
        got, want = run_attention(rts[dtype], [(599, 1)], 4, 2, 64, 16, seed=far, stand_out=far, scale=1.0,
                                  splits=4 if dtype == "bfloat16" else None)
        assert worst(got, want) < (3e-2 if dtype == "bfloat16" else 1e-4)


def test_float32_attention_is_bitwise_independent_of_cutting(rts):
    """The same query gives the same bits whether it comes alone, in a portion, or beside others."""
    rt = rts["float32"]
    whole, _ = run_attention(rt, [(0, 90)], 4, 2, 64, 8, seed=7)
    tail, _ = run_attention(rt, [(60, 30)], 4, 2, 64, 8, seed=7)
    single, _ = run_attention(rt, [(89, 1)], 4, 2, 64, 8, seed=7)
    assert torch.equal(whole[0][60:], tail[0]) and torch.equal(whole[0][89:], single[0])


def test_head_sizes_beyond_the_kernels_are_refused(rts):
    from atoma_infer_b200.csrc.ops import KernelError

    with pytest.raises(KernelError):
        run_attention(rts["bfloat16"], [(0, 4)], 1, 1, 272, 16)


@pytest.mark.parametrize("flat", [0, 3, 100])  # 0: fixed splits; else the large-batch kernel with that many blocks
@pytest.mark.parametrize("d,rot,nq,nkv,page,splits", [(64, 64, 32, 8, 16, 3), (64, 64, 3, 1, 8, 1), (128, 64, 8, 2, 16, 2),
                                                       (16, 16, 4, 2, 4, 4)])
def test_decode_with_fused_rotation_and_cache_write(rts, d, rot, nq, nkv, page, splits, flat):
    """The decode kernel given unrotated q, k, v of the new token: it must rotate q, write the rotated
    key and the value to the right page and slot, and attend over old keys and the new one."""
    rt = rts["bfloat16"]
    contexts = [0, 1, 15, 16, 31, 32, 200, 513]
    g = torch.Generator().manual_seed(d + splits)
    lengths = [c + 1 for c in contexts]
    tables, num_pages = K.scrambled_tables(lengths, page, d)
    inv = torch.tensor([1.0 / 10000.0 ** (i / rot) for i in range(0, rot, 2)], dtype=torch.float32)
    bf = lambda t: t.bfloat16().float()  # noqa: E731
    qs = [bf(torch.randn(L, nq, d, generator=g)) for L in lengths]
    ks = [bf(torch.randn(L, nkv, d, generator=g)) for L in lengths]
    vs = [bf(torch.randn(L, nkv, d, generator=g)) for L in lengths]

    def rotate(x):  # [L, heads, d] -> rotated in the first `rot` dims, rounded as the kernels round
        y = x.clone().double()
        y[..., :rot] = P.rope(x[..., :rot].double(), torch.arange(x.shape[0]), inv)
        return bf(y.float())

    rks, rqs = [rotate(k) for k in ks], [rotate(q) for q in qs]
    cache = torch.full((num_pages, 2, nkv, page, d), float("nan"), dtype=torch.bfloat16, device=rt.device)
    K.fill_cache(cache, tables, [rk[:-1] for rk in rks], [v[:-1] for v in vs], page)  # everything but the new token
    ctx, _ = K.make_context(rt, [(c, 1) for c in contexts], page, tables)
    S = len(contexts)
    qkv = torch.zeros(S, (nq + 2 * nkv) * d, dtype=torch.bfloat16, device=rt.device)
    for i in range(S):
        qkv[i] = torch.cat([qs[i][-1].reshape(-1), ks[i][-1].reshape(-1), vs[i][-1].reshape(-1)]).bfloat16()
    out = torch.full((S, nq * d), float("nan"), dtype=torch.bfloat16, device=rt.device)
    rt.ops.decode_splits = lambda *a: splits
    rt.ops._decode_flat_blocks = lambda *a: flat
    try:
        rt.ops.attention(qkv, qkv.shape[1], cache, ctx, 0, out, nq, nkv, d, page, num_pages, 0, 1 / math.sqrt(d),
                         rope=(inv.to(rt.device), rot, True))
    finally:
        del rt.ops.decode_splits
        del rt.ops._decode_flat_blocks
    rt.ops.check_status()
    for i, c in enumerate(contexts):
        want = P.causal_attention(rqs[i].double(), rks[i].double(), vs[i].double(), 1 / math.sqrt(d))[-1]
        assert (out[i].float().cpu().reshape(nq, d) - want.float()).abs().max() < 2e-2, c
        pg, slot = tables[i][c // page], c % page
        assert (cache[pg, 0, :, slot].float().cpu() - rks[i][-1]).abs().max() < 2e-2
        assert torch.equal(cache[pg, 1, :, slot].float().cpu(), vs[i][-1])


def test_decode_page_loads_by_tma(rts):
    """The decode kernel's TMA page loads (opt-in) give the same result as its cp.async loads."""
    lib = rts["bfloat16"].ops._attention_library(64)
    entries = [(0, 1), (15, 1), (16, 1), (31, 1), (300, 1), (777, 1), (1023, 1)]
    try:
        lib.attn_set_decode_tma(1)
        for page, splits in ((16, 1), (16, 5), (8, 3), (32, 2)):
            got, want = run_attention(rts["bfloat16"], entries, 32, 8, 64, page, seed=splits, splits=splits)
            assert worst(got, want) < 2e-2, (page, splits)
        got, want = run_attention(rts["bfloat16"], [(599, 1)], 4, 2, 64, 16, seed=255, stand_out=255, scale=1.0, splits=4)
        assert worst(got, want) < 3e-2
    finally:
        lib.attn_set_decode_tma(0)
