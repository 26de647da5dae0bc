"""Generality of the parts layer, shown with toy parts that live in this test only: a mixer with
per-request state of its own (no pages), an architecture whose layers differ (attention, toy
mixer, attention that reads another layer's cache, a layer that runs twice), a feed-forward that
routes tokens to experts, a position encoding that is a learned table: registered, written as
random model folders, loaded and stepped without any change to the framework's files."""
import json
import math

import pytest
import torch

import helpers
import plain_llama as P
from toy_parts import RunningMeanMixer
from atoma_infer_b200.config import register_architecture, register_part
from atoma_infer_b200.parts import FeedForward, LayerRun, LayerSpec, Mixer, ModelSpec, PositionEncoding
from atoma_infer_b200.weights import TensorDecl

pytestmark = pytest.mark.gpu

H, V = 48, 97


def toy_config(raw):
    return dict(raw)


def toy_spec(cfg):
    norm = {"kind": "rmsnorm", "size": H, "eps": cfg["eps"]}
    attn = {"kind": "attention", "hidden": H, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
            "scale": 0.25, "window": None, "position": {"kind": "rope", "head_dim": 16, "theta": 100.0}}
    windowed = dict(attn, window=cfg["window"], num_kv_heads=3)
    ff = {"kind": "swiglu", "hidden": H, "intermediate": 80}
    mean = {"kind": "toy_running_mean", "hidden": H}
    blocks = [attn, mean, attn, windowed]
    names = [None, {"mixer": "mean"}, None, None]
    layers = [LayerSpec(f"model.layers.{i}", {"kind": "prenorm", "norm": norm, "mixer": m, "feed_forward": ff,
                                               **({"names": n} if n else {})})
              for i, (m, n) in enumerate(zip(blocks, names))]
    # layer 2 keeps no keys of its own: it reads layer 0's; layer 1 (the toy mixer) runs twice
    schedule = [LayerRun(0), LayerRun(1), LayerRun(2, cache_of=0), LayerRun(3), LayerRun(1)]
    return ModelSpec(hidden_size=H, vocab_size=V, layers=layers, final_norm=norm, head_tensor="lm_head.weight",
                     schedule=schedule, max_position=512)


@pytest.fixture(scope="module")
def toy_model(tmp_path_factory):
    register_part("mixer", "toy_running_mean", RunningMeanMixer, replace=True)
    register_architecture("ToyForCausalLM", toy_config, toy_spec, replace=True)
    d = str(tmp_path_factory.mktemp("toy"))
    cfg = {"architectures": ["ToyForCausalLM"], "eps": 1e-5, "window": 7}
    helpers.make_model(d, cfg, seed=4, std=0.2)
    return d, cfg


def plain_toy(w, cfg, tokens):
    """The same model, whole sequence, float64, no cache, no state."""
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    pos = torch.arange(T)
    x = w["model.embed_tokens.weight"][torch.as_tensor(tokens)]
    inv = 1.0 / torch.pow(torch.tensor(100.0), torch.arange(0, 16, 2, dtype=torch.float32) / 16)

    def attention(h, p, nkv, window, kv_from=None):
        q = (h @ w[p + "q_proj.weight"].T).reshape(T, 3, 16)
        src = kv_from if kv_from is not None else h
        sp = kv_from_prefix if kv_from is not None else p
        k = (src @ w[sp + "k_proj.weight"].T).reshape(T, nkv, 16)
        v = (src @ w[sp + "v_proj.weight"].T).reshape(T, nkv, 16)
        o = P.causal_attention(P.rope(q, pos, inv), P.rope(k, pos, inv), v, 0.25, window)
        return o.reshape(T, 48) @ w[p + "o_proj.weight"].T

    def mean_mixer(h, p):
        return (torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]) @ w[p + "mix.weight"].T

    def block(x, i, mix):
        p = f"model.layers.{i}."
        h = x + mix(P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"]))
        return h + P.swiglu(P.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")

    normed0 = P.rms_norm(x, w["model.layers.0.input_layernorm.weight"], cfg["eps"])  # what layer 0's keys are made from
    kv_from_prefix = "model.layers.0.self_attn."
    x = block(x, 0, lambda h: attention(h, "model.layers.0.self_attn.", 1, None))
    x = block(x, 1, lambda h: mean_mixer(h, "model.layers.1.mean."))
    x = block(x, 2, lambda h: attention(h, "model.layers.2.self_attn.", 1, None, kv_from=normed0))
    x = block(x, 3, lambda h: attention(h, "model.layers.3.self_attn.", 3, cfg["window"]))
    x = block(x, 1, lambda h: mean_mixer(h, "model.layers.1.mean."))
    return P.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T


def test_toy_architecture_is_built_and_stepped_without_touching_the_framework(toy_model):
    from atoma_infer_b200.engine import StepEntry, load_model

    d, cfg = toy_model
    lm = load_model(d, dtype="float32", device="cuda:0", page_size=4, num_pages=40, max_seqs=3, poison_cache=True)
    model = lm.model
    # the cache plan follows the spec: layers 0 and 3 own pages (two groups: all keys / a window),
    # layer 2 owns none, layer 1 has state and no pages
    assert [g.layers for g in model.groups] == [[0], [3]] and model.groups[1].need.window == 7
    assert model.state_bytes == [0, 4 * (H + 1), 0, 0, 4 * (H + 1)] and not model.graph_safe  # per run
    w = helpers.read_weights(d)
    seqs = helpers.random_tokens(V, (23, 9, 31), seed=8)
    ref = {k: plain_toy(w, cfg, v) for k, v in seqs.items()}
    # mixed steps: portions of changing size, requests beside one another, one request after another in a slot
    pos = {k: 0 for k in seqs}
    live, pending, sizes, si = ["r0", "r1"], ["r2"], (5, 1, 3, 2, 7), 0
    ids = {k: i for i, k in enumerate(seqs)}
    worst = 0.0
    while live:
        entries, meta = [], []
        for k in list(live):
            n = min(sizes[si % len(sizes)], len(seqs[k]) - pos[k])
            si += 1
            entries.append(StepEntry(ids[k], seqs[k][pos[k]:pos[k] + n], list(range(n))))
            meta.append((k, pos[k], n))
            pos[k] += n
        logits = lm.step.run(entries).double().cpu()
        lm.rt.ops.check_status()
        row = 0
        for k, start, n in meta:
            scale = float(ref[k].abs().max())
            worst = max(worst, float((logits[row:row + n] - ref[k][start:start + n]).abs().max()) / scale)
            row += n
            if pos[k] == len(seqs[k]):
                lm.step.finish(ids[k])
                live.remove(k)
                if pending:
                    live.append(pending.pop())  # takes the freed state slot and pages
        assert lm.manager.audit() == ""
    assert worst < 5e-5, worst
    # the windowed group gave pages back while requests ran; in the end nothing is held
    assert lm.manager.num_requests() == 0
    assert all(lm.manager.num_free_pages(g) == 40 for g in range(2)) and lm.manager.num_free_slots() == 3


# ----------------------------------------------------------------------------- a routed feed-forward and another position encoding
class LearnedPositions(PositionEncoding):
    """A table of learned vectors, one per position, added to every query and key head; the keys go to the
    pages with their position already in them.  Not a rotation: ``rotary()`` stays None, so attention never
    asks its decode kernel to encode positions itself."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.head_dim = int(params["head_dim"])
        self.max_position = int(params["max_position"])

    def declare(self):
        return [TensorDecl(self.prefix + ".position_table", (self.max_position, self.head_dim))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.table = tensors[self.prefix + ".position_table"]
        self.zero_freq = torch.zeros(self.head_dim // 2, dtype=torch.float32, device=rt.device)

    def encode_and_store(self, qkv, ctx, cache, *, num_heads, num_kv_heads, head_dim):
        T = ctx.T
        rows = self.table[ctx.positions[:T].long()].to(qkv.dtype)  # [T, d]
        qk = qkv[:T, :(num_heads + num_kv_heads) * head_dim].view(T, num_heads + num_kv_heads, head_dim)
        qk += rows[:, None, :]
        # a rotation by angle zero: the framework's kernel that writes keys and values to their pages
        self.rt.ops.rope_kv_store(qkv, ctx.positions, ctx.token_entry, ctx.meta, max(cache.group, 0), self.zero_freq,
                                  cache.pages, cache.num_pages, T, num_heads, num_kv_heads, head_dim, head_dim,
                                  cache.page_size, cache.writes and cache.pages is not None)


class Top1Experts(FeedForward):
    """Router logits in float32, the best expert per token, its gate probability as the weight:
    out = p_e * W2_e relu(W1_e x)."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden, self.inner, self.experts = int(params["hidden"]), int(params["inner"]), int(params["experts"])

    def declare(self):
        pre = self.prefix
        return [TensorDecl(pre + ".router.weight", (self.experts, self.hidden))] + [
            TensorDecl(f"{pre}.experts.{e}.{n}.weight", shape) for e in range(self.experts)
            for n, shape in (("w1", (self.inner, self.hidden)), ("w2", (self.hidden, self.inner)))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre = self.prefix
        self.router = tensors[pre + ".router.weight"].float()
        self.w1 = [tensors[f"{pre}.experts.{e}.w1.weight"] for e in range(self.experts)]
        self.w2 = [tensors[f"{pre}.experts.{e}.w2.weight"] for e in range(self.experts)]

    def forward(self, x, ctx):
        T = ctx.T
        probs = torch.softmax(x[:T].float() @ self.router.T, dim=-1)
        weight, choice = probs.max(dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                h = torch.relu(x[rows] @ self.w1[e].T)
                out[rows] = ((h @ self.w2[e].T).float() * weight[rows, None]).to(x.dtype)
        return out


def routed_spec(cfg):
    norm = {"kind": "rmsnorm", "size": H, "eps": cfg["eps"]}
    attn = {"kind": "attention", "hidden": H, "num_heads": 3, "num_kv_heads": 3, "head_dim": 16, "scale": 0.25,
            "window": None, "position": {"kind": "toy_learned", "head_dim": 16, "max_position": 64}}
    dense = {"kind": "swiglu", "hidden": H, "intermediate": 80}
    routed = {"kind": "toy_top1", "hidden": H, "inner": 40, "experts": 3}
    layers = [LayerSpec(f"model.layers.{i}", {"kind": "prenorm", "norm": norm, "mixer": attn, "feed_forward": ff})
              for i, ff in enumerate([routed, dense, routed])]
    return ModelSpec(hidden_size=H, vocab_size=V, layers=layers, final_norm=norm, head_tensor="lm_head.weight",
                     schedule=[LayerRun(i) for i in range(3)], max_position=64)


def plain_routed(w, cfg, tokens):
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    x = w["model.embed_tokens.weight"][torch.as_tensor(tokens)]
    for i in range(3):
        p = f"model.layers.{i}."
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        table = w[p + "self_attn.position_table"][:T]
        q = (h @ w[p + "self_attn.q_proj.weight"].T).reshape(T, 3, 16) + table[:, None, :]
        k = (h @ w[p + "self_attn.k_proj.weight"].T).reshape(T, 3, 16) + table[:, None, :]
        v = (h @ w[p + "self_attn.v_proj.weight"].T).reshape(T, 3, 16)
        x = x + P.causal_attention(q, k, v, 0.25, None).reshape(T, 48) @ w[p + "self_attn.o_proj.weight"].T
        h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        if i == 1:
            x = x + P.swiglu(h, w, p + "mlp.")
        else:
            probs = torch.softmax(h @ w[p + "mlp.router.weight"].T, dim=-1)
            weight, choice = probs.max(dim=-1)
            out = torch.zeros_like(h)
            for e in range(3):
                rows = (choice == e).nonzero().flatten()
                hh = torch.relu(h[rows] @ w[f"{p}mlp.experts.{e}.w1.weight"].T)
                out[rows] = (hh @ w[f"{p}mlp.experts.{e}.w2.weight"].T) * weight[rows, None]
            x = x + out
    return P.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["lm_head.weight"].T


def test_routed_feed_forward_and_learned_positions_without_touching_the_framework(tmp_path):
    """A feed-forward that routes each token to one of three experts (beside a dense one in another layer) and
    a position encoding that is a learned table, both defined here, registered, built from a model folder and
    stepped in portions and single tokens."""
    from atoma_infer_b200.engine import StepEntry, load_model

    register_part("position", "toy_learned", LearnedPositions, replace=True)
    register_part("feed_forward", "toy_top1", Top1Experts, replace=True)
    register_architecture("RoutedToyForCausalLM", toy_config, routed_spec, replace=True)
    cfg = {"architectures": ["RoutedToyForCausalLM"], "eps": 1e-5}
    d = helpers.make_model(str(tmp_path / "routed"), cfg, seed=6, std=0.2)
    lm = load_model(d, dtype="float32", device="cuda:0", page_size=4, num_pages=40, max_seqs=2, poison_cache=True)
    w = helpers.read_weights(d)
    assert "model.layers.0.self_attn.position_table" in w and "model.layers.2.mlp.experts.2.w2.weight" in w
    seqs = helpers.random_tokens(V, (29, 17), seed=3)
    ref = {k: plain_routed(w, cfg, v) for k, v in seqs.items()}
    # every expert of the first layer is chosen by some token (else the routing would show little)
    h0 = torch.cat([P.rms_norm(w["model.embed_tokens.weight"].double()[torch.as_tensor(v)],
                               w["model.layers.0.input_layernorm.weight"].double(), cfg["eps"]) for v in seqs.values()])
    assert set((h0 @ w["model.layers.0.mlp.router.weight"].double().T).argmax(-1).tolist()) == {0, 1, 2}
    pos = {k: 0 for k in seqs}
    ids = {k: i for i, k in enumerate(seqs)}
    sizes, si, worst = (6, 1, 1, 4, 2, 9), 0, 0.0
    live = list(seqs)
    while live:
        entries, meta = [], []
        for k in list(live):
            n = min(sizes[si % len(sizes)], len(seqs[k]) - pos[k])
            si += 1
            entries.append(StepEntry(ids[k], seqs[k][pos[k]:pos[k] + n], list(range(n))))
            meta.append((k, pos[k], n))
            pos[k] += n
        logits = lm.step.run(entries).double().cpu()
        lm.rt.ops.check_status()
        row = 0
        for k, start, n in meta:
            scale = float(ref[k].abs().max())
            worst = max(worst, float((logits[row:row + n] - ref[k][start:start + n]).abs().max()) / scale)
            row += n
            if pos[k] == len(seqs[k]):
                lm.step.finish(ids[k])
                live.remove(k)
    assert worst < 5e-5, worst
    assert lm.manager.num_requests() == 0 and lm.manager.audit() == ""
