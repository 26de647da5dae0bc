"""The model's two ends and the cache need as parts too, and a stateful model through the whole engine.

A toy architecture defined here (parts in toy_parts.py) has an embedding stage that scales the token rows
and adds learned absolute positions, a head with a bias and a soft cap, a mixer that caches one latent
vector per token (a cache need of one named tensor, not keys and values), a mixer with fixed-size state of
its own, and one ordinary attention layer.  It is registered, written as a random model folder, loaded,
stepped and generated from through ``Engine`` (scheduler, preemption by recompute, re-admission) without
a change to the framework's files.  The tests run on the CPU with the torch stand-in for the kernels and on
the GPU with the kernels (``-m gpu``)."""
import pytest
import torch

import helpers
import plain_llama as P
import toy_parts
from atoma_infer_b200.config import register_architecture, register_part
from atoma_infer_b200.parts import LayerSpec, ModelSpec

H, V, MAXPOS = 40, 61, 96
CFG = {"architectures": ["ToyEndsForCausalLM"], "eps": 1e-5, "scale": 3.0, "cap": 4.0}


def spec(cfg):
    norm = {"kind": "rmsnorm", "size": H, "eps": cfg["eps"]}
    ff = {"kind": "swiglu", "hidden": H, "intermediate": 56}
    attn = {"kind": "attention", "hidden": H, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "scale": 0.25,
            "window": None, "position": {"kind": "rope", "head_dim": 16, "theta": 50.0}}
    latent = {"kind": "toy_latent", "hidden": H, "latent": 24, "dim": 20}
    mean = {"kind": "toy_running_mean", "hidden": H}
    mixers = [(attn, None), (latent, {"mixer": "latent"}), (mean, {"mixer": "mean"})]
    layers = [LayerSpec(f"model.layers.{i}", {"kind": "prenorm", "norm": norm, "mixer": m, "feed_forward": ff,
                                               **({"names": n} if n else {})}) for i, (m, n) in enumerate(mixers)]
    return ModelSpec(hidden_size=H, vocab_size=V, layers=layers, final_norm=norm, max_position=MAXPOS,
                     embedding={"kind": "toy_scaled_positional", "vocab": V, "hidden": H, "max_position": MAXPOS,
                                "scale": cfg["scale"]},
                     head={"kind": "toy_capped_bias", "vocab": V, "cap": cfg["cap"]})


def plain(w, cfg, tokens):
    """The same model: whole sequence, float64, no cache, no state."""
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    pos = torch.arange(T)
    x = cfg["scale"] * w["embed.tokens"][torch.as_tensor(tokens)] + w["embed.positions"][:T]
    inv = 1.0 / torch.pow(torch.tensor(50.0), torch.arange(0, 16, 2, dtype=torch.float32) / 16)

    def attention(h, p):
        q = (h @ w[p + "q_proj.weight"].T).reshape(T, 2, 16)
        k = (h @ w[p + "k_proj.weight"].T).reshape(T, 1, 16)
        v = (h @ w[p + "v_proj.weight"].T).reshape(T, 1, 16)
        return P.causal_attention(P.rope(q, pos, inv), P.rope(k, pos, inv), v, 0.25).reshape(T, 32) @ w[p + "o_proj.weight"].T

    def latent(h, p):
        c = h @ w[p + "c.weight"].T
        q, k, v = h @ w[p + "q.weight"].T, c @ w[p + "k.weight"].T, c @ w[p + "v.weight"].T
        return P.causal_attention(q[:, None], k[:, None], v[:, None], 20 ** -0.5)[:, 0] @ w[p + "o.weight"].T

    def mean(h, p):
        return (torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]) @ w[p + "mix.weight"].T

    for i, (mix, name) in enumerate(((attention, "self_attn"), (latent, "latent"), (mean, "mean"))):
        p = f"model.layers.{i}."
        x = x + mix(P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"]), f"{p}{name}.")
        x = x + P.swiglu(P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")
    logits = P.rms_norm(x, w["model.norm.weight"], cfg["eps"]) @ w["embed.tokens"].T + w["head.bias"]
    return cfg["cap"] * torch.tanh(logits / cfg["cap"])


def plain_greedy(w, cfg, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(plain(w, cfg, toks)[-1].float())))
    return toks[len(prompt):]


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    register_part("mixer", "toy_running_mean", toy_parts.RunningMeanMixer, replace=True)
    register_part("mixer", "toy_latent", toy_parts.LatentMixer, replace=True)
    register_part("embedding", "toy_scaled_positional", toy_parts.ScaledPositionalEmbedding, replace=True)
    register_part("head", "toy_capped_bias", toy_parts.CappedBiasHead, replace=True)
    register_architecture("ToyEndsForCausalLM", dict, spec, replace=True)
    d = str(tmp_path_factory.mktemp("toy_ends"))
    helpers.make_model(d, CFG, seed=12, std=0.2)
    return d, helpers.read_weights(d)


def _ops(device):
    if device == "cpu":
        from host_ops import HostOps

        return HostOps()
    return None


DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


@pytest.mark.parametrize("device", DEVICES)
def test_ends_and_a_one_tensor_cache_need_in_every_cutting(device, toy):
    from atoma_infer_b200.engine import StepEntry, load_model

    d, w = toy
    lm = load_model(d, dtype="float32", device="cuda:0" if device == "cuda" else "cpu", ops=_ops(device), page_size=4,
                    num_pages=30, max_seqs=3, poison_cache=True)
    model = lm.model
    # two cache groups: keys and values of the attention layer, one latent of 24 elements per token for the other
    needs = [g.need for g in model.groups]
    assert [n.is_kv for n in needs] == [True, False] and needs[1].elements_per_token == 24
    assert [tuple(t.shape[1:]) for t in lm.cache.pages] == [(31, 2 * 16 * 4), (31, 24 * 4)]
    assert model.state_bytes == [0, 0, 4 * (H + 1)] and not model.graph_safe
    assert "embed.positions" in w and "head.bias" in w and "lm_head.weight" not in w
    seqs = helpers.random_tokens(V, (27, 8, 33), seed=5)
    ref = {k: plain(w, CFG, v) for k, v in seqs.items()}
    assert max(float(r.abs().max()) for r in ref.values()) > 0.5 * CFG["cap"], "the cap should matter"
    pos = {k: 0 for k in seqs}
    live, pending, sizes, si = ["r0", "r1"], ["r2"], (5, 1, 3, 2, 7, 1, 1), 0
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
            worst = max(worst, float((logits[row:row + n] - ref[k][start:start + n]).abs().max()) / float(ref[k].abs().max()))
            row += n
            if pos[k] == len(seqs[k]):
                lm.step.finish(ids[k])
                live.remove(k)
                if pending:
                    live.append(pending.pop())
        assert lm.manager.audit() == ""
    assert worst < 5e-5, worst
    assert lm.manager.num_requests() == 0 and all(lm.manager.num_free_pages(g) == 30 for g in range(2))


@pytest.mark.parametrize("device", DEVICES)
def test_a_model_with_state_is_scheduled_preempted_and_readmitted(device, toy):
    """Through ``Engine``: so few pages that running requests are preempted and recomputed.  A re-admitted
    request gets a state slot that another request has used meanwhile; its state must start from zero again
    (the running-mean mixer would otherwise average over a stranger's tokens)."""
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    d, w = toy
    prompts = list(helpers.random_tokens(V, (13, 15, 12, 3), seed=9).values())
    want = [plain_greedy(w, CFG, p, 16) for p in prompts]
    sp = SamplingParams(do_sample=False, max_new_tokens=16, ignore_eos_token=True)
    kw = dict(dtype="float32", block_size=4, max_num_sequences=3, max_num_batched_tokens=16, ops=_ops(device))
    roomy = Engine(d, num_gpu_blocks_override=64, **kw)
    assert [o.token_ids for o in roomy.generate(prompts, sp)] == want
    tight = Engine(d, num_gpu_blocks_override=17, **kw)  # 68 tokens of cache for three requests of about 30 each
    outs = tight.generate(prompts, sp)
    assert tight.scheduler.num_preemptions > 0
    assert [o.token_ids for o in outs] == want
    assert tight.lm.manager.audit() == "" and tight.lm.manager.num_requests() == 0
    assert all(tight.lm.manager.num_free_pages(g) == 17 for g in range(2)) and tight.lm.manager.num_free_slots() == 3
