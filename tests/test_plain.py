"""The plain implementation itself (no GPU): literal vectors that the reference's own tests
carry, closed formulas, and properties every causal decoder has."""
import math

import pytest
import torch

import helpers
import plain_llama as P


def test_attention_reproduces_the_reference_test_vector():
    # csrc/tests/flash_attn_tests.rs:33-71: q, k, v = arange(48)/30, /40, /50 in half precision, laid
    # out (3 heads, 2 tokens, 8), scale 0.5, no mask.  The second token's row of a causal
    # attention sees both keys, so it equals the unmasked row; the first row equals v[0]
    # (as the reference's causal test says, models/src/flash_attention.rs:633-705).
    base = torch.arange(48, dtype=torch.float32).reshape(3, 2, 8)
    q = (base.half() / 30.0).double().permute(1, 0, 2)  # [tokens, heads, d]
    k = (base.half() / 40.0).double().permute(1, 0, 2)
    v = (base.half() / 50.0).double().permute(1, 0, 2)
    out = P.causal_attention(q, k, v, 0.5)
    expected_second_rows = torch.tensor([
        [0.0922, 0.1122, 0.1322, 0.1522, 0.1721, 0.1921, 0.2122, 0.2322],
        [0.428, 0.448, 0.468, 0.488, 0.5083, 0.5283, 0.5483, 0.5684],
        [0.7622, 0.7822, 0.8022, 0.8223, 0.8423, 0.8623, 0.8823, 0.9023],
    ], dtype=torch.float64)
    # The literals are half precision printed to 4 digits, from inputs that candle scales by a
    # reciprocal rounded to half precision: two half-precision roundings near 0.9, about 5e-4 each.
    assert (out[1] - expected_second_rows).abs().max() < 1e-3
    assert torch.equal(out[0], v[0])


def test_grouped_heads_read_the_right_key_head():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 6, 8, dtype=torch.float64), torch.randn(5, 2, 8, dtype=torch.float64), torch.randn(5, 2, 8, dtype=torch.float64)
    out = P.causal_attention(q, k, v, 0.3)
    for h in range(6):
        one = P.causal_attention(q[:, h:h + 1], k[:, h // 3:h // 3 + 1], v[:, h // 3:h // 3 + 1], 0.3)
        assert torch.allclose(out[:, h], one[:, 0])


def test_window_keeps_the_last_keys_only():
    torch.manual_seed(1)
    q, k, v = (torch.randn(9, 1, 4, dtype=torch.float64) for _ in range(3))
    out = P.causal_attention(q, k, v, 0.5, window=3)
    for t in range(9):
        lo = max(0, t - 2)
        s = torch.softmax((k[lo:t + 1, 0] @ q[t, 0]) * 0.5, 0)
        assert torch.allclose(out[t, 0], s @ v[lo:t + 1, 0])


def test_default_rotary_frequencies():
    f = P.rope_inv_freq(helpers.CONFIG_A)
    d = 16
    want = [1.0 / 10000.0 ** (i / d) for i in range(0, d, 2)]
    assert f.dtype == torch.float32 and torch.allclose(f.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6)


def test_llama3_scaling_has_all_three_bands():
    cfg = helpers.CONFIG_B
    sc = cfg["rope_scaling"]
    f = P.rope_inv_freq(cfg).double()
    base = P.rope_inv_freq({k: v for k, v in cfg.items() if k != "rope_scaling"}).double()
    orig, lo, hi, factor = sc["original_max_position_embeddings"], sc["low_freq_factor"], sc["high_freq_factor"], sc["factor"]
    kinds = set()
    for fi, bi in zip(f.tolist(), base.tolist()):
        wl = 2 * math.pi / bi
        if wl < orig / hi:
            kinds.add("kept")
            assert fi == pytest.approx(bi, rel=1e-6)
        elif wl > orig / lo:
            kinds.add("divided")
            assert fi == pytest.approx(bi / factor, rel=1e-6)
        else:
            kinds.add("between")
            s = (orig / wl - lo) / (hi - lo)
            assert fi == pytest.approx((1 - s) * bi / factor + s * bi, rel=1e-5)
            assert bi / factor < fi < bi
    assert kinds == {"kept", "divided", "between"}


def test_rotation_is_half_split_and_norm_preserving():
    x = torch.arange(8, dtype=torch.float64).reshape(1, 1, 8) + 1
    inv = torch.tensor([1.0, 0.5, 0.25, 0.125])
    y = P.rope(x, torch.tensor([3]), inv)
    for i in range(4):
        a = 3 * float(inv[i])
        assert y[0, 0, i] == pytest.approx(float(x[0, 0, i]) * math.cos(a) - float(x[0, 0, i + 4]) * math.sin(a), abs=1e-6)
        assert y[0, 0, i + 4] == pytest.approx(float(x[0, 0, i]) * math.sin(a) + float(x[0, 0, i + 4]) * math.cos(a), abs=1e-6)
    assert torch.equal(P.rope(x, torch.tensor([0]), inv), x)


def test_rms_norm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = P.rms_norm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]], dtype=torch.float64))
    wd = {"p.gate_proj.weight": torch.tensor([[1.0, 0.0]]), "p.up_proj.weight": torch.tensor([[0.0, 2.0]]),
          "p.down_proj.weight": torch.tensor([[1.0], [-1.0]])}
    wd = {k: v.double() for k, v in wd.items()}
    z = 3.0 / (1 + math.exp(-3.0)) * 8.0
    assert torch.allclose(P.swiglu(x, wd, "p."), torch.tensor([[z, -z]], dtype=torch.float64))


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_model_is_causal_and_tied_head_is_the_embedding(name, tiny_models):
    d, cfg, _ = tiny_models[name]
    w = helpers.read_weights(d)
    toks = helpers.random_tokens(cfg["vocab_size"], (24,), seed=9)["r0"]
    full = P.forward(w, cfg, toks)
    assert full.shape == (24, cfg["vocab_size"]) and torch.isfinite(full).all()
    assert torch.allclose(P.forward(w, cfg, toks[:10]), full[:10], atol=1e-12)  # later tokens change nothing before them
    other = list(toks)
    other[0] = (other[0] + 1) % cfg["vocab_size"]
    assert not torch.allclose(P.forward(w, cfg, other)[-1], full[-1], atol=1e-6)  # the first token reaches the last
    assert ("lm_head.weight" in w) == (not cfg["tie_word_embeddings"])


def test_philox_known_answers():
    # Random123's published vectors for Philox4x32-10
    assert P.philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert P.philox4x32([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert P.philox4x32([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    us = [P.uniform(7, i) for i in range(2000)]
    assert all(0.0 <= u < 1.0 for u in us) and 0.45 < sum(us) / len(us) < 0.55


def test_samplers():
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5])
    assert P.greedy(logits) == 1  # the lowest index among equals
    picks = [P.sample(logits, temperature=0.7, seed=3, step=i) for i in range(400)]
    assert set(picks) <= {0, 1, 2, 3, 4} and picks.count(1) > 100 and picks.count(2) > 100
    assert set(P.sample(logits, temperature=0.7, seed=3, step=i, top_k=2) for i in range(200)) == {1, 2}
    assert set(P.sample(logits, temperature=0.7, seed=3, step=i, top_k=3) for i in range(300)) == {0, 1, 2}
    p = torch.softmax(logits / 0.7, 0)
    assert float(p[1] + p[2]) > 0.8  # so a nucleus of 0.8 is the two equal tokens
    assert set(P.sample(logits, temperature=0.7, seed=3, step=i, top_p=0.8) for i in range(200)) == {1, 2}
    pen = P.apply_repeat_penalty(logits, 2.0, [1, 1, 3])
    assert pen.tolist() == [1.0, 1.5, 3.0, -4.0, 0.5]
