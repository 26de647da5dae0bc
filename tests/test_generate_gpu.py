"""Generation through the Python entry point on the GPU, against the plain implementation."""
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu


def _engine(d, page, dtype, **kw):
    from atoma_infer_b200.engine import Engine

    kw.setdefault("num_gpu_blocks_override", 64)
    kw.setdefault("max_num_sequences", 4)
    kw.setdefault("max_num_batched_tokens", 16)
    return Engine(d, dtype=dtype, block_size=page, **kw)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_equals_plain_in_float32(name, tiny_models):
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models[name]
    w = helpers.read_weights(d)
    lengths = (1, 7, 16, 33) if name == "A" else (5, 29, 64)
    prompts = list(helpers.random_tokens(cfg["vocab_size"], lengths, seed=int(name == "B")).values())
    n = 8 if name == "A" else 16
    want = [P.generate_greedy(w, cfg, p, n) for p in prompts]
    eng = _engine(d, page, "float32")
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=n, ignore_eos_token=True))
    assert [o.token_ids for o in outs] == want
    assert all(o.finish_reason == "length" for o in outs)
    assert eng.lm.manager.num_requests() == 0 and eng.lm.manager.audit() == ""
    assert eng.lm.manager.num_free_pages(0) == eng.lm.manager.num_usable_pages(0)


def test_seeded_temperature_sampling_equals_plain_and_ignores_batch(tiny_models):
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["B"]
    w = helpers.read_weights(d)
    prompts = list(helpers.random_tokens(cfg["vocab_size"], (5, 29, 64), seed=1).values())
    sp = [SamplingParams(temperature=0.8, random_seed=100 + i, max_new_tokens=16, ignore_eos_token=True)
          for i in range(3)]
    # the plain loop: whole sequence each time, float64 softmax, same random numbers
    want = []
    for p, s in zip(prompts, sp):
        toks, out = list(p), []
        for step in range(16):
            t = P.sample(P.forward(w, cfg, toks)[-1], temperature=0.8, seed=s.random_seed, step=step)
            out.append(t)
            toks.append(t)
        want.append(out)
    eng = _engine(d, page, "float32", max_num_batched_tokens=8)
    together = [o.token_ids for o in eng.generate(prompts, sp)]
    alone = [eng.generate([p], s)[0].token_ids for p, s in zip(prompts, sp)]
    assert together == alone, "a request's sampled tokens depend on who shares its batch"
    assert together == want


def test_stop_rules_and_eos(tiny_models):
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["A"]
    eng = _engine(d, page, "float32")
    base = eng.generate([[1, 2, 3]], SamplingParams(do_sample=False, max_new_tokens=12, ignore_eos_token=True))[0]
    stop_at = base.token_ids[4]
    first = base.token_ids.index(stop_at)
    out = eng.generate([[1, 2, 3]], SamplingParams(do_sample=False, max_new_tokens=12, stop_token_ids=(stop_at,)))[0]
    assert out.finish_reason == "stop" and out.token_ids == base.token_ids[:first + 1]


def test_preemption_by_recompute_keeps_tokens(tiny_models):
    """So few pages that running requests must be preempted; tokens equal the roomy run."""
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["A"]
    prompts = list(helpers.random_tokens(cfg["vocab_size"], (14, 15, 13), seed=5).values())
    sp = SamplingParams(do_sample=False, max_new_tokens=20, ignore_eos_token=True)
    roomy = [o.token_ids for o in _engine(d, page, "float32").generate(prompts, sp)]
    tight = _engine(d, page, "float32", num_gpu_blocks_override=16)  # 64 tokens of cache for 3 x ~34
    outs = tight.generate(prompts, sp)
    assert [o.token_ids for o in outs] == roomy
    assert tight.scheduler.num_preemptions > 0
    assert tight.lm.manager.audit() == "" and tight.lm.manager.num_requests() == 0


@pytest.mark.parametrize("name", ["A", "B"])
def test_many_requests_few_pages_small_budget(name, tiny_models):
    """Twenty requests of mixed lengths through eight sequence slots, a token budget that cuts prompts into
    portions beside decoding requests, and a page pool that forces preemptions: every request's greedy
    tokens still equal the plain implementation's, and every page comes back."""
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models[name]
    w = helpers.read_weights(d)
    g = torch.Generator().manual_seed(17)
    lengths = torch.randint(1, 60, (20,), generator=g).tolist()
    news = torch.randint(1, 18, (20,), generator=g).tolist()
    prompts = list(helpers.random_tokens(cfg["vocab_size"], lengths, seed=9).values())
    want = [P.generate_greedy(w, cfg, p, n) for p, n in zip(prompts, news)]
    eng = _engine(d, page, "float32", num_gpu_blocks_override=(128 // page) + 1, max_num_sequences=8,
                  max_num_batched_tokens=24)  # 128 tokens of cache for up to 8 x 77
    params = [SamplingParams(do_sample=False, max_new_tokens=n, ignore_eos_token=True) for n in news]
    outs = eng.generate(prompts, params)
    assert [o.token_ids for o in outs] == want
    assert eng.scheduler.num_preemptions > 0
    assert eng.lm.manager.audit() == "" and eng.lm.manager.num_requests() == 0
    assert eng.lm.manager.num_free_pages(0) == eng.lm.manager.num_usable_pages(0)


def test_smoke_entry():
    import __graft_entry__ as g

    g.smoke()
