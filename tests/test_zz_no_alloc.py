"""The decode-attention entry point that allocates nothing (attention_noalloc.h), called the way
its users call it: through the exported C symbol, with plain pointers.

Its users are hosts that cannot hand a kernel library an allocator when requests flow: an engine
that gave all free device memory to its page pool at start-up, a loop that must never reach
cudaMalloc (which stalls the device), a binding from another language.  The test checks, on two
calls in a row that share the built-in scratch array, that the output equals the ordinary entry
point's (which takes its scratch from the caller), and that a call too large for the array is
refused with a message instead of run.  This file sorts last, so a run that stops at the first
failure has already run every other test."""
import ctypes
import math

import pytest
import torch

import kernel_utils as K

pytestmark = pytest.mark.gpu

NOALLOC_SOURCES = ["kernels/attention_noalloc.cu"]


def _library(d):
    from atoma_infer_b200.csrc import build

    lib = build.load_library(f"attention_noalloc_d{d}", NOALLOC_SOURCES, cuda=True, defines={"HEAD_DIM": d})
    c = ctypes
    lib.attn_decode_noalloc.restype = c.c_int
    lib.attn_decode_noalloc.argtypes = (
        [c.c_void_p, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_void_p, c.c_void_p]
        + [c.c_int] * 6 + [c.c_float, c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_char_p, c.c_int])
    return lib


def _case(rt, contexts, nq, nkv, d, page, seed):
    g = torch.Generator().manual_seed(seed)
    entries = [(c, 1) for c in contexts]
    tables, num_pages = K.scrambled_tables([c + 1 for c in contexts], page, seed)
    cache = torch.full((num_pages, 2, nkv, page, d), float("nan"), dtype=torch.bfloat16, device=rt.device)
    ks = [torch.randn(c + 1, nkv, d, generator=g) for c in contexts]
    vs = [torch.randn(c + 1, nkv, d, generator=g) for c in contexts]
    K.fill_cache(cache, tables, ks, vs, page)
    ctx, _ = K.make_context(rt, entries, page, tables)
    qkv = torch.randn(len(contexts), (nq + 2 * nkv) * d, generator=g).bfloat16().to(rt.device)
    return ctx, cache, qkv, num_pages


@pytest.mark.parametrize("nq,nkv,d,page,splits", [(8, 2, 64, 16, 4), (6, 2, 128, 8, 3)])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(nq, nkv, d, page, splits):
    from atoma_infer_b200.engine.runtime import make_runtime

    rt = make_runtime("bfloat16", "cuda:0")
    lib = _library(d)
    err = ctypes.create_string_buffer(512)
    stream = ctypes.c_void_p(torch.cuda.current_stream(rt.device).cuda_stream)
    scale = 1.0 / math.sqrt(d)
    for call, contexts in enumerate([(700, 33, 0, 257), (90, 1200)]):  # the second call reuses the array as it was left
        ctx, cache, qkv, num_pages = _case(rt, contexts, nq, nkv, d, page, seed=call)
        S = len(contexts)
        want = torch.full((S, nq * d), float("nan"), dtype=torch.bfloat16, device=rt.device)
        rt.ops.decode_splits = lambda *a: splits
        try:
            rt.ops.attention(qkv, qkv.shape[1], cache, ctx, 0, want, nq, nkv, d, page, num_pages, 0, scale)
        finally:
            del rt.ops.decode_splits
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated(rt.device)
        rc = lib.attn_decode_noalloc(qkv.data_ptr(), qkv.shape[1], cache.data_ptr(), ctx.meta.data_ptr(), 0,
                                     ctx.cu_tokens.data_ptr(), ctx.positions.data_ptr(), got.data_ptr(), S, nq, nkv, page,
                                     num_pages, 0, scale, splits, ctx.max_context, rt.ops.status.data_ptr(), stream, err, 512)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        rt.ops.check_status()
        assert torch.cuda.memory_allocated(rt.device) == before
        assert torch.isfinite(got.float()).all()
        assert (got.float() - want.float()).abs().max() < 2e-2  # the tolerance of the attention tests; same kernels
        assert torch.equal(got, want)                            # and in fact the same bits
    # too large for the built-in array: refused, nothing launched, the message names the sizes
    rc = lib.attn_decode_noalloc(qkv.data_ptr(), qkv.shape[1], cache.data_ptr(), ctx.meta.data_ptr(), 0,
                                 ctx.cu_tokens.data_ptr(), ctx.positions.data_ptr(), got.data_ptr(), 2048, nq, nkv, page,
                                 num_pages, 0, scale, 32, ctx.max_context, rt.ops.status.data_ptr(), stream, err, 512)
    assert rc == -1 and b"floats of scratch" in err.value and b"1048576" in err.value
    # more splits than the merging block can stage in its shared memory (the scratch array would hold them):
    # refused as well, the message names the limit
    most = lib.attn_decode_max_splits(16, 1)
    rc = lib.attn_decode_noalloc(qkv.data_ptr(), qkv.shape[1], cache.data_ptr(), ctx.meta.data_ptr(), 0,
                                 ctx.cu_tokens.data_ptr(), ctx.positions.data_ptr(), got.data_ptr(), 1, 16, 1, page,
                                 num_pages, 0, scale, most + 1, ctx.max_context, rt.ops.status.data_ptr(), stream, err, 512)
    assert rc == -1
    if (most + 1) * 16 * (d + 2) <= (1 << 20):  # the case fits the array, so only the split limit refuses it
        assert b"splits" in err.value and str(most).encode() in err.value
    torch.cuda.synchronize()
    rt.ops.check_status()
