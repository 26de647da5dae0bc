"""Trace replay on the GPU against the plain implementation: every way of cutting the work."""
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (1, 7, 16, 33, 70, 131), "B": (5, 29, 64, 97, 150)}


@pytest.fixture(scope="module")
def references(tiny_models):
    out = {}
    for name, (d, cfg, page) in tiny_models.items():
        seqs = helpers.random_tokens(cfg["vocab_size"], LENGTHS[name], seed=3)
        w = helpers.read_weights(d)
        out[name] = (seqs, {k: P.forward(w, cfg, v) for k, v in seqs.items()})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_every_cutting_matches_plain(name, dtype, tiny_models, references, tmp_path):
    d, cfg, page = tiny_models[name]
    seqs, ref = references[name]
    families = {
        "w": helpers.trace_whole(seqs, tag="w"),
        "t": helpers.trace_tail(seqs, tag="t"),
        "c": helpers.trace_chunks(seqs, tag="c"),
        "m": helpers.trace_mixed(seqs, tag="m"),
    }
    steps = [s for f in families.values() for s in f]
    # four live requests of the longest lengths, rounded up to 64 each: pages are used again
    longest = sorted((len(v) for v in seqs.values()), reverse=True)[:4]
    max_tokens = sum(-(-n // 64) * 64 for n in longest)
    steps, out = helpers.run_trace(d, dtype, steps, str(tmp_path), max_tokens, page)
    tol = helpers.FP32_TOL if dtype == "float32" else helpers.BF16_TOL
    for tag in families:
        sub = [s for s in steps if s["entries"][0]["id"].startswith(tag)]
        worst, where, agree = helpers.compare_trace(sub, out, cfg["vocab_size"], ref)
        assert worst <= tol, f"family {tag!r}: error {worst:.3g} of the logit scale at (step, request, position) {where}"
        if dtype == "float32":
            assert agree == 1.0, f"family {tag!r}: greedy tokens differ from the plain implementation"
