"""Trace replay on the GPU against the plain implementation: every way of cutting the work."""
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

# bfloat16 families: share of places whose top-1 token must equal the plain implementation's (random tiny models
# have many near-ties, which is why it is not 1), and all of them where the plain lead is clear
BF16_TOP1 = 0.9

LENGTHS = {"A": (1, 7, 16, 33, 70, 131), "B": (5, 29, 64, 97, 150), "C": (3, 40, 129, 300)}


@pytest.fixture(scope="module")
def references(tiny_models):
    out = {}
    for name, (d, cfg, page) in tiny_models.items():
        seqs = helpers.random_tokens(cfg["vocab_size"], LENGTHS[name], seed=3)
        w = helpers.read_weights(d)
        out[name] = (seqs, {k: P.forward(w, cfg, v) for k, v in seqs.items()})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
        worst, where, agree, clear = helpers.compare_trace(sub, out, cfg["vocab_size"], ref)
        assert worst <= tol, f"family {tag!r}: error {worst:.3g} of the logit scale at (step, request, position) {where}"
        if dtype == "float32":
            assert agree == 1.0, f"family {tag!r}: greedy tokens differ from the plain implementation"
        else:
            assert agree >= BF16_TOP1 and clear == 1.0, f"family {tag!r}: top-1 agreement {agree:.3f} ({clear:.3f} where clear)"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_one_token_at_a_time(dtype, tiny_models, tmp_path):
    """A short prompt and hundreds of single-token steps (the captured decode graph, many page edges)."""
    d, cfg, page = tiny_models["B"]
    seq = helpers.random_tokens(cfg["vocab_size"], (420,), seed=11)
    ref = {k: P.forward(helpers.read_weights(d), cfg, v) for k, v in seq.items()}
    steps = helpers.trace_tail(seq, tail=412)
    steps, out = helpers.run_trace(d, dtype, steps, str(tmp_path), 448, page)
    worst, where, agree, clear = helpers.compare_trace(steps, out, cfg["vocab_size"], ref)
    assert worst <= (helpers.FP32_TOL if dtype == "float32" else helpers.BF16_TOL), (worst, where)
    assert agree == 1.0 if dtype == "float32" else agree > 0.97


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_sequences(name, dtype, tiny_models, tmp_path):
    """Requests of one, two and three tokens: alone, together in one step, and token by token."""
    d, cfg, page = tiny_models[name]
    seqs = helpers.random_tokens(cfg["vocab_size"], (1, 2, 3, 1), seed=12)
    ref = {k: P.forward(helpers.read_weights(d), cfg, v) for k, v in seqs.items()}
    together = [{"entries": [{"id": f"g{k}", "tokens": v, "want": list(range(len(v)))} for k, v in seqs.items()],
                 "end": [f"g{k}" for k in seqs]}]
    steps = helpers.trace_whole(seqs, tag="w") + together + helpers.trace_tail(seqs, tail=3, tag="t")
    steps, out = helpers.run_trace(d, dtype, steps, str(tmp_path), 256, page)
    worst, where, agree, clear = helpers.compare_trace(steps, out, cfg["vocab_size"], ref)
    assert worst <= (helpers.FP32_TOL if dtype == "float32" else helpers.BF16_TOL), (worst, where)
    # twenty-one places only, some of them near-ties: in bfloat16 the floor holds where the plain lead is clear
    assert (agree == 1.0 if dtype == "float32" else True) and clear == 1.0, (agree, clear)


@pytest.mark.parametrize("name", sorted(helpers.MORE))
def test_other_geometries(name, tmp_path):
    """One replay (whole, tail decoded one by one, mixed) per further geometry, in both precisions."""
    cfg, page = helpers.MORE[name]
    d = helpers.make_model(str(tmp_path / "model"), cfg, seed=len(name))
    seqs = helpers.random_tokens(cfg["vocab_size"], (2, 37, 90, 150), seed=5)
    w = helpers.read_weights(d)
    ref = {k: P.forward(w, cfg, v) for k, v in seqs.items()}
    families = {"w": helpers.trace_whole(seqs, tag="w"), "t": helpers.trace_tail(seqs, tag="t"),
                "m": helpers.trace_mixed(seqs, tag="m")}
    steps = [s for f in families.values() for s in f]
    max_tokens = sum(-(-len(v) // max(64, page)) * max(64, page) for v in seqs.values())
    for dtype, tol in (("float32", helpers.FP32_TOL), ("bfloat16", helpers.BF16_TOL)):
        numbered, out = helpers.run_trace(d, dtype, steps, str(tmp_path / dtype), max_tokens, page)
        for tag in families:
            sub = [s for s in numbered if s["entries"][0]["id"].startswith(tag)]
            worst, where, agree, clear = helpers.compare_trace(sub, out, cfg["vocab_size"], ref)
            assert worst <= tol, f"{dtype}, family {tag!r}: error {worst:.3g} of the logit scale at {where}"
            assert agree >= (1.0 if dtype == "float32" else BF16_TOP1) and clear == 1.0, (dtype, tag, agree, clear)


@pytest.mark.parametrize("name,blocks", [("B", 3), ("C", 10)])
def test_decode_steps_on_the_large_batch_kernel(name, blocks, tiny_models, references, tmp_path):
    """The decode attention of large batches (key tiles dealt out over a fixed number of blocks), forced on
    for these small ones: tails decoded one by one and mixed steps, captured graphs included."""
    d, cfg, page = tiny_models[name]
    seqs, ref = references[name]
    families = {"t": helpers.trace_tail(seqs, tag="t"), "m": helpers.trace_mixed(seqs, tag="m")}
    # four requests decoding together: one token each per step, for 40 steps after their prompts
    together = []
    keys = list(seqs)[-4:]
    heads = {k: max(len(seqs[k]) - 40, 1) for k in keys}
    together.append({"entries": [{"id": f"g{k}", "tokens": seqs[k][:heads[k]], "want": []} for k in keys], "end": []})
    longest = max(len(seqs[k]) - heads[k] for k in keys)
    for i in range(longest):
        ent = [{"id": f"g{k}", "tokens": [seqs[k][heads[k] + i]], "want": [0]} for k in keys if heads[k] + i < len(seqs[k])]
        end = [f"g{k}" for k in keys if heads[k] + i == len(seqs[k]) - 1]
        together.append({"entries": ent, "end": end})
    families["g"] = together
    steps = [s for f in families.values() for s in f]
    longest4 = sorted((len(v) for v in seqs.values()), reverse=True)[:4]
    max_tokens = sum(-(-n // 64) * 64 for n in longest4)
    steps, out = helpers.run_trace(d, "bfloat16", steps, str(tmp_path), max_tokens, page,
                                   env={"ATOMA_INFER_DECODE_FLAT": str(blocks)})
    for tag in families:
        sub = [s for s in steps if s["entries"][0]["id"].startswith(tag)]
        worst, where, agree, clear = helpers.compare_trace(sub, out, cfg["vocab_size"], ref)
        assert worst <= helpers.BF16_TOL, f"family {tag!r}: error {worst:.3g} of the logit scale at {where}"
        assert agree >= BF16_TOP1 and clear == 1.0, (tag, agree, clear)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt(dtype, tiny_models, tmp_path):
    """2,040 tokens: whole (16 key tiles of 128 for the last query tile, the many-token rotation and norm
    kernels), in three portions (each attending to what the earlier ones cached), then decoded tokens up to
    the model's 2,048 positions."""
    d, cfg, page = tiny_models["C"]
    seq = helpers.random_tokens(cfg["vocab_size"], (2048,), seed=31)
    (k, v), = seq.items()
    ref = {k: P.forward(helpers.read_weights(d), cfg, v, compute=torch.float32)}
    want = [0, 127, 128, 1000, 2039]
    steps = [{"entries": [{"id": f"w{k}", "tokens": v[:2040], "want": want}], "end": [f"w{k}"]}]
    cuts = [0, 700, 1500, 2040]
    for a, b in zip(cuts, cuts[1:]):
        steps.append({"entries": [{"id": f"c{k}", "tokens": v[a:b], "want": [0, b - a - 1]}], "end": []})
    for i in range(2040, 2048):
        steps.append({"entries": [{"id": f"c{k}", "tokens": [v[i]], "want": [0]}], "end": [f"c{k}"] if i == 2047 else []})
    steps, out = helpers.run_trace(d, dtype, steps, str(tmp_path), 2048, page)
    worst, where, agree, clear = helpers.compare_trace(steps, out, cfg["vocab_size"], ref)
    assert worst <= (5e-5 if dtype == "float32" else helpers.BF16_TOL), (worst, where)


def test_replay_beyond_the_configured_positions(tmp_path):
    """A request longer than max_position_embeddings replays (positions are not table rows here) and still
    equals the plain implementation."""
    cfg = dict(helpers.CONFIG_A, max_position_embeddings=32)
    d = helpers.make_model(str(tmp_path / "model"), cfg, seed=3)
    seqs = helpers.random_tokens(cfg["vocab_size"], (90,), seed=2)
    ref = {k: P.forward(helpers.read_weights(d), cfg, v) for k, v in seqs.items()}
    steps = helpers.trace_tail(seqs, tail=40)
    steps, out = helpers.run_trace(d, "float32", steps, str(tmp_path / "out"), 128, 4)
    worst, where, agree, clear = helpers.compare_trace(steps, out, cfg["vocab_size"], ref)
    assert worst <= helpers.FP32_TOL and agree == 1.0, (worst, where)
