"""Each part of a layer alone, built from its parameters and bound to random tensors, against the
plain function of the same name; sizes differ from the tiny configurations of the engine tests."""
import math

import pytest
import torch

import kernel_utils as K
import plain_llama as P
from atoma_infer_b200.cache import LayerCache
from atoma_infer_b200.config import part_class

pytestmark = pytest.mark.gpu

CFG = {"hidden_size": 120, "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 200,
       "rms_norm_eps": 3e-6, "rope_theta": 20000.0,
       "rope_scaling": {"factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 2.0,
                        "original_max_position_embeddings": 32, "rope_type": "llama3"}}
NORM = {"kind": "rmsnorm", "size": 120, "eps": 3e-6}
MIXER = {"kind": "attention", "hidden": 120, "num_heads": 5, "num_kv_heads": 1, "head_dim": 32,
         "scale": 1 / math.sqrt(32), "window": None,
         "position": {"kind": "rope", "head_dim": 32, "theta": 20000.0, "scaling": CFG["rope_scaling"]}}
FF = {"kind": "swiglu", "hidden": 120, "intermediate": 200}


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def rt(request):
    from atoma_infer_b200.engine.runtime import make_runtime

    return make_runtime(request.param, "cuda:0")


def tol(rt):
    return 2e-5 if rt.dtype == torch.float32 else 3e-2


def bound(part, rt, seed=0):
    """Random tensors for the part's declarations (in the runtime's dtype), bound; returns float64 copies."""
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for d in part.declare():
        t = torch.randn(d.shape, generator=g) * (0.1 if d.init == "normal" else 0.1)
        if d.init == "ones":
            t = t + 1
        tensors[d.name] = t.to(rt.dtype)
    part.bind({k: v.to(rt.device) for k, v in tensors.items()}, rt)
    return {k: v.double() for k, v in tensors.items()}


def close(got, want, rt):
    want = want.double()
    assert (got.double().cpu() - want).abs().max() <= tol(rt) * max(1.0, float(want.abs().max()))


def test_norm_part(rt):
    part = part_class("norm", "rmsnorm")(NORM, "n")
    w = bound(part, rt)
    ctx, _ = K.make_context(rt, [(0, 6)], 8, [[1]])
    x = torch.randn(6, 120)
    resid = x.clone().to(rt.device)
    close(part.forward(resid, None, ctx), P.rms_norm(x.double(), w["n.weight"], 3e-6), rt)


def test_feed_forward_part(rt):
    part = part_class("feed_forward", "swiglu")(FF, "ff")
    w = bound(part, rt)
    for T in (3, 20):  # the few-row and the many-row kernels
        ctx, _ = K.make_context(rt, [(0, T)], 8, [[1, 2, 3]])
        x = torch.randn(T, 120).to(rt.dtype)
        close(part.forward(x.to(rt.device), ctx), P.swiglu(x.double(), w, "ff."), rt)


def attention_case(rt, entries, page=8, seed=0):
    """Runs the attention part over hand-made entries whose earlier tokens are run first (to fill the
    cache), and returns (outputs of the last step, plain outputs at the same places)."""
    part = part_class("mixer", "attention")(MIXER, "a")
    w = bound(part, rt, seed)
    lengths = [c + n for c, n in entries]
    tables, num_pages = K.scrambled_tables(lengths, page, seed)
    pages = torch.full((num_pages, 2, 1, page, 32), float("nan"), dtype=rt.dtype, device=rt.device)
    cache = LayerCache(group=0, pages=pages, num_pages=num_pages, page_size=page, writes=True)
    g = torch.Generator().manual_seed(seed + 1)
    xs = [torch.randn(L, 120, generator=g).to(rt.dtype) for L in lengths]
    first = [(0, c) for c, _ in entries if c > 0]
    if first:  # the contexts, as one earlier step of whole prompts
        idx = [i for i, (c, _) in enumerate(entries) if c > 0]
        ctx, _ = K.make_context(rt, first, page, [tables[i] for i in idx])
        part.forward(torch.cat([xs[i][:entries[i][0]] for i in idx]).to(rt.device), ctx, cache)
    ctx, _ = K.make_context(rt, entries, page, tables)
    out = part.forward(torch.cat([x[c:c + n] for x, (c, n) in zip(xs, entries)]).to(rt.device), ctx, cache)
    rt.ops.check_status()
    want = []
    for x, (c, n) in zip(xs, entries):
        full = P.attention_block(x.double(), torch.arange(x.shape[0]), w, "a.", CFG)
        want.append(full[c:c + n])
    return out, torch.cat(want)


def test_attention_part_whole_portion_and_decode(rt):
    out, want = attention_case(rt, [(0, 40)])
    close(out, want, rt)
    out, want = attention_case(rt, [(17, 23), (0, 9), (33, 1)], seed=1)  # portions over cached contexts, mixed
    close(out, want, rt)
    out, want = attention_case(rt, [(39, 1), (5, 1), (64, 1)], seed=2)   # a decode step
    close(out, want, rt)


def test_position_part_rotates_like_the_plain_rope(rt):
    part = part_class("position", "rope")(MIXER["position"], "p")
    bound(part, rt)
    inv = P.rope_inv_freq(CFG)
    assert torch.equal(part.inv_freq.cpu(), inv)  # the same float32 frequencies, bit for bit
    none = part_class("position", "none")({"kind": "none", "head_dim": 32}, "p")
    none.bind({}, rt)
    assert torch.count_nonzero(none.inv_freq) == 0


def test_block_part(rt):
    spec = {"kind": "prenorm", "norm": NORM, "mixer": MIXER, "feed_forward": FF}
    part = part_class("block", "prenorm")(spec, "model.layers.0")
    w = bound(part, rt, seed=5)
    T, page = 21, 8
    tables, num_pages = K.scrambled_tables([T], page)
    pages = torch.full((num_pages, 2, 1, page, 32), float("nan"), dtype=rt.dtype, device=rt.device)
    cache = LayerCache(group=0, pages=pages, num_pages=num_pages, page_size=page, writes=True)
    ctx, _ = K.make_context(rt, [(0, T)], page, tables)
    x = torch.randn(T, 120)
    prev = (torch.randn(T, 120) * 0.3).to(rt.dtype)  # what the block before left to be added
    resid = x.clone().to(rt.device)
    delta = part.forward(resid, prev.to(rt.device), ctx, cache)
    cfg = dict(CFG, num_hidden_layers=1)
    h0 = x.double() + prev.double()
    want = P.decoder_block(h0, torch.arange(T), w, 0, cfg)
    # the block leaves its last addition pending: residual + pending = the plain block's output
    close(resid.double().cpu() + delta.double().cpu(), want, rt)
