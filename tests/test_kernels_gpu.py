"""Each kernel alone against a plain float64 reference of the same operation, at sizes other
than the engine tests use (widths and vocabularies that are no power of two, odd row counts)."""
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


def ctx_for(rt, T, rows=()):
    tables, _ = K.scrambled_tables([T], 16)
    return K.make_context(rt, [(0, T)], 16, tables, tokens=list(range(T)), rows=rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_bad_token_flag(rts, dtype):
    from atoma_infer_b200.csrc.ops import KernelError

    rt = rts[dtype]
    V, H = 301, 200
    table = torch.randn(V, H).to(rt.dtype).to(rt.device)
    toks = [0, 300, 17, 17, 5]
    tables, _ = K.scrambled_tables([5], 16)
    ctx, _ = K.make_context(rt, [(0, 5)], 16, tables, tokens=toks)
    resid = torch.full((5, H), float("nan"), device=rt.device)
    rt.ops.embed(ctx.tokens, table, resid, ctx.meta, 5)
    rt.ops.check_status()
    assert torch.equal(resid.cpu(), table.float().cpu()[toks])
    ctx, _ = K.make_context(rt, [(0, 2)], 16, tables, tokens=[3, V])
    rt.ops.embed(ctx.tokens, table, resid, ctx.meta, 2)
    with pytest.raises(KernelError, match="token id out of range"):
        rt.ops.check_status()


@pytest.mark.parametrize("H", [1024, 2048, 3072, 4096, 1152, 8192])
def test_add_rmsnorm_many_rows(rts, H):
    """A thousand rows and more of bfloat16 activations take the warp-per-row kernel (widths 1024..4096 in
    steps of 1024); 1152 and 8192 do not fit it and take the block-per-row kernel."""
    rt = rts["bfloat16"]
    T, eps = 1100, 1e-6
    g = torch.Generator().manual_seed(H)
    resid0 = torch.randn(T, H, generator=g) * 3
    delta = torch.randn(T, H, generator=g).bfloat16()
    w = 1 + 0.1 * torch.randn(H, generator=g)
    ctx, _ = ctx_for(rt, T)
    resid = resid0.clone().to(rt.device)
    out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=rt.device)
    rt.ops.add_rmsnorm(resid, None, w.to(rt.device), eps, out, ctx.meta, T)
    want = P.rms_norm(resid0.double(), w.double(), eps)
    assert (out.double().cpu() - want).abs().max() < 2e-2 * want.abs().max()
    assert torch.equal(resid.cpu(), resid0)
    rt.ops.add_rmsnorm(resid, delta.to(rt.device), w.to(rt.device), eps, out, ctx.meta, T)
    summed = resid0 + delta.float()
    assert torch.equal(resid.cpu(), summed)
    want = P.rms_norm(summed.double(), w.double(), eps)
    assert (out.double().cpu() - want).abs().max() < 2e-2 * want.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [200, 2048, 3000])
def test_add_rmsnorm(rts, dtype, H):
    rt = rts[dtype]
    T, eps = 7, 1e-5
    g = torch.Generator().manual_seed(H)
    resid0 = torch.randn(T, H, generator=g) * 3
    delta = (torch.randn(T, H, generator=g)).to(rt.dtype)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    ctx, rows = ctx_for(rt, T, rows=[5, 0, 6])
    tol = 1e-5 if dtype == "float32" else 2e-2
    # plain norm of the first layer: no addition
    resid = resid0.clone().to(rt.device)
    out = torch.empty(T, H, dtype=rt.dtype, device=rt.device)
    rt.ops.add_rmsnorm(resid, None, w.to(rt.device), eps, out, ctx.meta, T)
    want = P.rms_norm(resid0.double(), w.double(), eps)
    assert (out.double().cpu() - want).abs().max() < tol * want.abs().max()
    assert torch.equal(resid.cpu(), resid0)
    # addition in float32, then the norm
    rt.ops.add_rmsnorm(resid, delta.to(rt.device), w.to(rt.device), eps, out, ctx.meta, T)
    summed = resid0 + delta.float()
    assert torch.equal(resid.cpu(), summed)
    want = P.rms_norm(summed.double(), w.double(), eps)
    assert (out.double().cpu() - want).abs().max() < tol * want.abs().max()
    # at chosen rows only, residual untouched
    out3 = torch.empty(3, H, dtype=rt.dtype, device=rt.device)
    rt.ops.add_rmsnorm(resid, delta.to(rt.device), w.to(rt.device), eps, out3, ctx.meta, 3, rows=rows)
    want = P.rms_norm((summed + delta.float())[[5, 0, 6]].double(), w.double(), eps)
    assert (out3.double().cpu() - want).abs().max() < tol * want.abs().max()
    assert torch.equal(resid.cpu(), summed)


def test_float32_gemm_is_true_float32_and_row_independent(rts):
    rt = rts["float32"]
    M, N, Kd = 37, 131, 77
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(M, Kd, generator=g), torch.randn(N, Kd, generator=g)
    y = rt.ops.linear(x.to(rt.device), w.to(rt.device))
    want = x.double() @ w.double().T
    assert (y.double().cpu() - want).abs().max() < 2e-5  # TF32 would be off by 1e-2 here
    one = rt.ops.linear(x[11:12].to(rt.device), w.to(rt.device))
    assert torch.equal(one[0], y[11])  # a row's bits do not depend on its neighbours


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 40])
@pytest.mark.parametrize("N,Kd", [(48, 64), (3000, 2048), (1001, 200)])
def test_bfloat16_linear_all_row_counts(rts, M, N, Kd):
    rt = rts["bfloat16"]
    g = torch.Generator().manual_seed(M * N)
    x = torch.randn(M, Kd, generator=g).bfloat16()
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).bfloat16()
    want = x.double() @ w.double().T
    y = rt.ops.linear(x.to(rt.device), w.to(rt.device))
    assert y.dtype == torch.bfloat16 and (y.double().cpu() - want).abs().max() < 2e-2
    y32 = rt.ops.linear(x.to(rt.device), w.to(rt.device), out_dtype=torch.float32)
    assert y32.dtype == torch.float32 and (y32.double().cpu() - want).abs().max() < 2e-3  # float32 accumulation kept


@pytest.mark.parametrize("M,N,Kd", [(5, 272, 2048), (16, 64, 8192), (1, 1000, 4096)])
def test_few_row_linear_with_every_split_of_k(rts, M, N, Kd):
    """The blocks of a cluster split K when a matrix has few 16-row tiles (the engine picks the count from the
    number of tiles); here every count is forced in turn, the leader adding the others' partial sums from their
    shared memory.  All give the product, and a given count the same bits twice."""
    rt = rts["bfloat16"]
    g = torch.Generator().manual_seed(N)
    x = torch.randn(M, Kd, generator=g).bfloat16()
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).bfloat16()
    want = x.double() @ w.double().T
    xd, wd = x.to(rt.device), w.to(rt.device)
    try:
        for splits in range(1, 9):
            rt.ops.lib.linear_skinny_set_ksplit(splits)
            y = rt.ops.linear(xd, wd, out_dtype=torch.float32)
            assert (y.double().cpu() - want).abs().max() < 2e-3, splits
            assert torch.equal(y, rt.ops.linear(xd, wd, out_dtype=torch.float32)), splits
    finally:
        rt.ops.lib.linear_skinny_set_ksplit(0)


@pytest.mark.parametrize("M,N,Kd,silu,out", [
    (1, 4100, 4096, False, "bfloat16"),    # one row
    (2, 272, 2048, False, "bfloat16"),     # few tiles: most blocks stay out
    (7, 1000, 192, False, "float32"),      # K no multiple of 512 (a stage that is part zeros), N no multiple of 16
    (8, 3072, 2048, False, "bfloat16"),
    (9, 40, 64, False, "float32"),         # two n-tiles, one group of k
    (16, 2048, 8192, False, "bfloat16"),   # x too large to stay in shared memory: in chunks through its own ring
    (13, 2 * 520, 1088, True, "bfloat16"), # silu(gate) * up, columns no multiple of 8, x in chunks (13 rows of 1,088 stay; 17 chunks)
    (16, 2 * 8192, 2048, True, "bfloat16"),
    (5, 2 * 176, 4160, True, "bfloat16"),
])
def test_streamed_few_row_linear(rts, M, N, Kd, silu, out):
    """The TMA-fed persistent linear (kernels/linear_stream.cu) against the product in float64, for shapes that meet
    every branch: rows of x resident or in chunks, one and two n-tiles, partial last stage, partial last tile, both
    epilogues and both output types; the same call twice gives the same bits; the direct kernel gives the same
    product within rounding."""
    rt = rts["bfloat16"]
    ops = rt.ops
    g = torch.Generator().manual_seed(N + M)
    x = torch.randn(M, Kd, generator=g).bfloat16()
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).bfloat16()
    full = x.double() @ w.double().T
    want = full[:, :N // 2] * torch.sigmoid(full[:, :N // 2]) * full[:, N // 2:] if silu else full
    xd, wd = x.to(rt.device), w.to(rt.device)
    odt = torch.float32 if out == "float32" else torch.bfloat16
    was = ops.stream_linear
    try:
        ops.stream_linear = True
        assert ops._stream_linear(M, N, Kd), "the shape was meant to take the streamed kernel"
        before = ops.launches
        y = ops.linear(xd, wd, out_dtype=odt, silu_mul=silu)
        assert ops.launches == before + 1
        ops.check_status()
        tol = (2e-3 if out == "float32" else 2e-2) * want.abs().max()
        assert y.shape == want.shape and y.dtype == odt
        assert (y.double().cpu() - want).abs().max() < tol
        assert torch.equal(y, ops.linear(xd, wd, out_dtype=odt, silu_mul=silu))
        ops.stream_linear = False
        z = ops.linear(xd, wd, out_dtype=odt, silu_mul=silu)
        assert (z.double().cpu() - want).abs().max() < tol
    finally:
        ops.stream_linear = was


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M", [2, 8, 13, 33])
def test_swiglu_gate_epilogue(rts, dtype, M):
    rt = rts[dtype]
    inter, Kd = 176, 64
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, Kd, generator=g).to(rt.dtype)
    w = (torch.randn(2 * inter, Kd, generator=g) / 4).to(rt.dtype)
    ctx, _ = ctx_for(rt, M)
    y = rt.ops.linear(x.to(rt.device), w.to(rt.device), silu_mul=True, meta=ctx.meta)
    gu = x.double() @ w.double().T
    want = gu[:, :inter] * torch.sigmoid(gu[:, :inter]) * gu[:, inter:]
    assert y.shape == (M, inter)
    assert (y.double().cpu() - want).abs().max() < (1e-5 if dtype == "float32" else 4e-2) * want.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("many", [False, True])  # few tokens: a block per head; 256 and more: a block per token, 16-byte accesses
@pytest.mark.parametrize("nq,nkv,d,rot,page", [(4, 2, 16, 16, 4), (3, 1, 64, 64, 8), (5, 5, 48, 32, 16)])
def test_rotation_and_cache_write(rts, dtype, nq, nkv, d, rot, page, many):
    rt = rts[dtype]
    entries = [(0, 60), (21, 50), (1000, 1), (3, 63), (100, 61), (7, 40)] if many else [(0, 9), (21, 5), (1000, 1)]  # a long position checks the float32 angle
    lengths = [c + n for c, n in entries]
    tables, num_pages = K.scrambled_tables(lengths, page)
    ctx, _ = K.make_context(rt, entries, page, tables)
    T = ctx.T
    g = torch.Generator().manual_seed(d)
    qkv0 = torch.randn(T, (nq + 2 * nkv) * d, generator=g).to(rt.dtype)
    qkv = qkv0.clone().to(rt.device)
    cache = torch.full((num_pages, 2, nkv, page, d), float("nan"), dtype=rt.dtype, device=rt.device)
    inv = torch.tensor([1.0 / 500000.0 ** (i / rot) for i in range(0, rot, 2)], dtype=torch.float32)
    rt.ops.rope_kv_store(qkv, ctx.positions, ctx.token_entry, ctx.meta, 0, inv.to(rt.device), cache, num_pages, T, nq,
                         nkv, d, rot, page, True)
    rt.ops.check_status()
    tol = 1e-5 if dtype == "float32" else 2e-2
    row = 0
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for (c, n), table in zip(entries, tables):
        for i in range(n):
            pos = c + i
            x = qkv0[row].double().reshape(nq + 2 * nkv, d)
            rotated = x.clone()
            rotated[:nq + nkv, :rot] = P.rope(x[None, :nq + nkv, :rot], torch.tensor([pos]), inv)[0]
            got_q = qkv[row].double().cpu().reshape(nq + 2 * nkv, d)[:nq]
            assert (got_q - rotated[:nq]).abs().max() < tol * 4
            page_id, slot = table[pos // page], pos % page
            written[page_id, slot] = True
            assert (cache[page_id, 0, :, slot].double().cpu() - rotated[nq:nq + nkv]).abs().max() < tol * 4
            assert torch.equal(cache[page_id, 1, :, slot].cpu(), qkv0[row].reshape(nq + 2 * nkv, d)[nq + nkv:])
            row += 1
    untouched = torch.isnan(cache[:, 0, 0, :, 0].float().cpu())
    assert torch.equal(untouched, ~written)  # nothing else was written
    if many and dtype == "float32":
        # the same tokens, one request at a time (fewer than 256 tokens a call: the other kernel): the same bits
        row = 0
        for (c, n), table in zip(entries, tables):
            ctx1, _ = K.make_context(rt, [(c, n)], page, [table])
            part = qkv0[row:row + n].clone().to(rt.device)
            cache1 = torch.zeros_like(cache)
            rt.ops.rope_kv_store(part, ctx1.positions, ctx1.token_entry, ctx1.meta, 0, inv.to(rt.device), cache1, num_pages,
                                 n, nq, nkv, d, rot, page, True)
            assert torch.equal(part[:, :nq * d], qkv[row:row + n, :nq * d])
            for i in range(n):
                pg, slot = table[(c + i) // page], (c + i) % page
                assert torch.equal(cache1[pg, :, :, slot], cache[pg, :, :, slot])
            row += n


def test_sampling_kernel_against_the_plain_sampler(rts):
    rt = rts["float32"]
    V, R = 1000, 64
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(R, V, generator=g) * 2.5
    logits[5, 17] = logits[5, 400] = logits[5].max() + 1  # equal maxima: the lower index wins
    dev = logits.to(rt.device)
    out = torch.empty(R, dtype=torch.int32, device=rt.device)

    def run(temp, top_k, top_p, seeds, steps):
        t = lambda v, dt: torch.tensor(v, dtype=dt, device=rt.device)  # noqa: E731
        rt.ops.sample(dev, t(temp, torch.float32), t(top_k, torch.int32), t(top_p, torch.float32),
                      t(seeds, torch.int64), t(steps, torch.int64), out)
        return out.tolist()

    zeros = [0] * R
    greedy = run([0.0] * R, zeros, [1.0] * R, zeros, zeros)
    assert greedy == [P.greedy(l) for l in logits] and greedy[5] == 17
    seeds, steps = [1000 + i for i in range(R)], [i * 3 for i in range(R)]
    for temp, k, p in ((0.8, 0, 1.0), (1.3, 0, 1.0), (0.7, 5, 1.0), (0.9, 0, 0.6), (1.1, 40, 0.8), (0.5, 1, 1.0)):
        got = run([temp] * R, [k] * R, [p] * R, seeds, steps)
        want = [P.sample(logits[i], temperature=temp, seed=seeds[i], step=steps[i], top_k=k, top_p=p) for i in range(R)]
        assert got == want, (temp, k, p)
    # the same row, seed and step give the same token whatever else is in the batch
    alone = torch.empty(1, dtype=torch.int32, device=rt.device)
    rt.ops.sample(dev[9:10], torch.tensor([0.8], device=rt.device), None, None,
                  torch.tensor([1009], dtype=torch.int64, device=rt.device),
                  torch.tensor([27], dtype=torch.int64, device=rt.device), alone)
    assert alone.item() == run([0.8] * R, zeros, [1.0] * R, seeds, steps)[9]


def test_sampling_at_llama_vocabulary_size(rts):
    rt = rts["float32"]
    V = 128256
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(3, V, generator=g) * 3
    out = torch.empty(3, dtype=torch.int32, device=rt.device)
    t = lambda v, dt: torch.tensor(v, dtype=dt, device=rt.device)  # noqa: E731
    rt.ops.sample(logits.to(rt.device), t([0.0, 0.9, 0.9], torch.float32), t([0, 0, 50], torch.int32),
                  t([1.0, 1.0, 0.9], torch.float32), t([1, 2, 3], torch.int64), t([0, 5, 9], torch.int64), out)
    assert out.tolist() == [P.greedy(logits[0]), P.sample(logits[1], temperature=0.9, seed=2, step=5),
                            P.sample(logits[2], temperature=0.9, seed=3, step=9, top_k=50, top_p=0.9)]


def test_repetition_penalty_kernel(rts):
    rt = rts["float32"]
    row = torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5, 0.0], device=rt.device)
    rt.ops.repeat_penalty(row, 2.0, torch.tensor([1, 1, 3, 5, 1], dtype=torch.int32, device=rt.device))
    assert row.tolist() == P.apply_repeat_penalty(torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5, 0.0]), 2.0, [1, 1, 3, 5, 1]).tolist()


@pytest.mark.parametrize("ra,rb,K,kw", [
    (128, 256, 64, dict(bn=256)),
    (300, 1000, 200, dict(bn=128)),                       # ragged rows, columns and K (zero-filled by TMA)
    (515, 777, 2048, dict(bn=256)),
    (260, 320, 192, dict(bn=256, silu_mul=True)),         # SwiGLU epilogue on a stacked [gate; up] weight
    (200, 1000, 264, dict(bn=256, out_dtype=torch.float32)),
    (3072, 40, 2048, dict(bn=64, transpose=True)),        # weights fill the 128-row side, few activation rows
    (1000, 17, 8192, dict(bn=32, transpose=True)),
    (1000, 100, 264, dict(bn=128, transpose=True, out_dtype=torch.float32)),
    # one block a multiprocessor walking several tiles each (the default); the one-tile-a-block form
    (2500, 3000, 328, dict(bn=256)),
    (2500, 3000, 328, dict(bn=128, silu_mul=True)),
    (2100, 2900, 136, dict(bn=256, silu_mul=True)),
    (515, 777, 2048, dict(bn=256, persistent=False)),
    (260, 320, 192, dict(bn=256, silu_mul=True, persistent=False)),
    (300, 1000, 200, dict(bn=128, ksplit=3)),             # K split over a cluster, partial tiles added through shared memory
])
def test_tcgen05_gemm(rts, ra, rb, K, kw):
    """The TMA + tcgen05 + TMEM GEMM against a float64 product."""
    rt = rts["bfloat16"]
    g = torch.Generator().manual_seed(ra + rb)
    a = torch.randn(ra, K, generator=g).bfloat16()
    b = (torch.randn(rb * (2 if kw.get("silu_mul") else 1), K, generator=g) / math.sqrt(K)).bfloat16()
    c = rt.ops.gemm_tc(a.to(rt.device), b.to(rt.device), **kw)
    rt.ops.check_status()
    ref = a.double() @ b.double().T
    if kw.get("silu_mul"):
        ref = ref[:, :rb] * torch.sigmoid(ref[:, :rb]) * ref[:, rb:]
    if kw.get("transpose"):
        ref = ref.T
    assert c.shape == ref.shape
    tol = 2e-5 if c.dtype == torch.float32 else 1e-2
    assert (c.double().cpu() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))


def test_linear_swiglu_of_a_long_prompt_runs_on_tcgen05(rts):
    """ops.linear picks the persistent tcgen05 kernel with the SwiGLU epilogue when the tiles fill whole
    rounds of the multiprocessors; the result matches the float64 formula either way."""
    rt = rts["bfloat16"]
    ops = rt.ops
    M, n_out, K = 2368, 3968, 136
    rounds = -(-(19 * 31) // ops.num_sms)
    chosen = 19 * 31 >= 0.97 * rounds * ops.num_sms
    assert ops._swiglu_on_tcgen05(M, n_out, K) == chosen  # true on a B200 (148 multiprocessors)
    assert not ops._swiglu_on_tcgen05(512, n_out, K)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(2 * n_out, K, generator=g) / math.sqrt(K)).bfloat16()
    meta = torch.zeros(64, dtype=torch.int32, device=rt.device)
    meta[0] = M
    y = ops.linear(x.to(rt.device), w.to(rt.device), silu_mul=True, meta=meta)
    ops.check_status()
    ref = x.double() @ w.double().T
    ref = ref[:, :n_out] * torch.sigmoid(ref[:, :n_out]) * ref[:, n_out:]
    assert y.shape == ref.shape
    assert (y.double().cpu() - ref).abs().max() < 2e-2 * max(1.0, float(ref.abs().max()))
