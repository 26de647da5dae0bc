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


def test_greedy_generation_in_bfloat16(tiny_models):
    """The serving precision through scheduler, decode graphs and tokens kept on the device.  Policy: see
    helpers.greedy_agreement (every token is the plain top-1 on the engine's own history, or within the error
    bound of it); nine in ten must be the top-1 itself."""
    from atoma_infer_b200.sampling import SamplingParams

    for name, lengths, n in (("A", (1, 7, 16, 33), 24), ("B", (5, 29, 64), 24), ("C", (3, 40, 129), 24)):
        d, cfg, page = tiny_models[name]
        w = helpers.read_weights(d)
        prompts = list(helpers.random_tokens(cfg["vocab_size"], lengths, seed=21).values())
        eng = _engine(d, page, "bfloat16", max_num_batched_tokens=48)
        outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=n, ignore_eos_token=True))
        eng.lm.rt.ops.check_status()
        assert eng.lm.step.graph_replays > 0, "decode steps did not run as captured graphs"
        same = total = 0
        for p, o in zip(prompts, outs):
            assert len(o.token_ids) == n and o.finish_reason == "length"
            a, b = helpers.greedy_agreement(w, cfg, p, o.token_ids)
            same, total = same + a, total + b
        assert same >= 0.9 * total, f"config {name}: only {same} of {total} tokens are the plain top-1"
        assert eng.lm.manager.num_requests() == 0 and eng.lm.manager.audit() == ""


@pytest.mark.parametrize("name", ["A", "B"])
def test_many_requests_few_pages_small_budget_in_bfloat16(name, tiny_models):
    """The twenty-request run above in the serving precision: preemptions, portions beside decode tokens, graphs."""
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models[name]
    w = helpers.read_weights(d)
    g = torch.Generator().manual_seed(17)
    lengths = torch.randint(1, 60, (20,), generator=g).tolist()
    news = torch.randint(1, 18, (20,), generator=g).tolist()
    prompts = list(helpers.random_tokens(cfg["vocab_size"], lengths, seed=9).values())
    eng = _engine(d, page, "bfloat16", num_gpu_blocks_override=(128 // page) + 1, max_num_sequences=8,
                  max_num_batched_tokens=24)
    params = [SamplingParams(do_sample=False, max_new_tokens=n, ignore_eos_token=True) for n in news]
    outs = eng.generate(prompts, params)
    eng.lm.rt.ops.check_status()
    same = total = 0
    for p, o, n in zip(prompts, outs, news):
        assert len(o.token_ids) == n
        a, b = helpers.greedy_agreement(w, cfg, p, o.token_ids)
        same, total = same + a, total + b
    assert same >= 0.9 * total, f"only {same} of {total} tokens are the plain top-1"
    assert eng.scheduler.num_preemptions > 0
    assert eng.lm.manager.audit() == "" and eng.lm.manager.num_requests() == 0
    assert eng.lm.manager.num_free_pages(0) == eng.lm.manager.num_usable_pages(0)


def test_sampling_options_through_the_engine(tiny_models):
    """top-k, top-p, both, and a repetition penalty through ``Engine`` on the device kernels, against the plain
    sampler on the plain logits (float32: the same tokens)."""
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["B"]
    w = helpers.read_weights(d)
    prompts = list(helpers.random_tokens(cfg["vocab_size"], (5, 11, 8, 4), seed=6).values())
    common = dict(max_new_tokens=10, ignore_eos_token=True)
    sps = [SamplingParams(temperature=0.9, top_k=5, random_seed=11, **common),
           SamplingParams(temperature=1.3, top_p=0.7, random_seed=12, **common),
           SamplingParams(temperature=0.7, top_k=9, top_p=0.8, random_seed=13, **common),
           SamplingParams(temperature=0.8, repetition_penalty=1.5, repeat_last_n=6, random_seed=14, **common)]
    want = [helpers.plain_sampled(w, cfg, p, 10, sp) for p, sp in zip(prompts, sps)]
    eng = _engine(d, page, "float32")
    assert [o.token_ids for o in eng.generate(prompts, sps)] == want
    alone = [eng.generate([p], sp)[0].token_ids for p, sp in zip(prompts, sps)]
    assert alone == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_only_without_chunked_prefill(dtype, tiny_models):
    """``enable_chunked_prefill=False`` (backends/vllm/src/scheduler.rs:1057-1217) through ``Engine`` on the GPU:
    a step holds whole prompts or decode tokens, never both, and the tokens are the plain ones."""
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["B"]
    w = helpers.read_weights(d)
    prompts = list(helpers.random_tokens(cfg["vocab_size"], (30, 33, 9, 17), seed=8).values())
    eng = _engine(d, page, dtype, enable_chunked_prefill=False, max_num_batched_tokens=64, max_model_len=64)
    sp = SamplingParams(do_sample=False, max_new_tokens=9, ignore_eos_token=True)
    ids = [eng.add_request(p, sp) for p in prompts]
    kinds, done = [], {}
    run = eng.lm.step.run

    def spy(entries):
        kinds.append(sorted({"prompt" if len(e.tokens) > 1 else "decode" for e in entries}))
        return run(entries)

    eng.lm.step.run = spy
    while eng.has_unfinished():
        for o in eng.step():
            done[o.request_id] = o
    assert all(len(k) == 1 for k in kinds), kinds
    assert kinds[:2] == [["prompt"], ["prompt"]]  # 30 + 33 fit the budget of 64, the third prompt does not
    for p, i in zip(prompts, ids):
        if dtype == "float32":
            assert done[i].token_ids == P.generate_greedy(w, cfg, p, 9)
        else:
            helpers.greedy_agreement(w, cfg, p, done[i].token_ids)


def test_page_count_from_free_memory(tiny_models):
    """No page count given: the pools are sized from the memory that is free after the weights are loaded,
    floor(free * gpu_memory_utilization) / bytes of a page over all layers (backends/vllm/src/config.rs:626-641,
    708-718), after the step's working memory (and state slots, none for this model) are taken out."""
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["B"]
    w = helpers.read_weights(d)
    eng = Engine(d, dtype="bfloat16", block_size=page, gpu_memory_utilization=0.002, max_num_sequences=4,
                 max_num_batched_tokens=64)
    m = eng.lm.memory
    assert m is not None and 0 < m["free"] <= m["total"] and m["state_bytes"] == 0 and m["workspace_bytes"] > 0
    head_dim = cfg["hidden_size"] // cfg["num_attention_heads"]
    page_bytes = 2 * page * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * head_dim * 2
    budget = int(m["free"] * 0.002) - m["workspace_bytes"]
    assert m["budget"] == budget
    assert eng.lm.num_pages == budget // page_bytes - 1 > 100  # page 0 of the pool is never handed out
    assert eng.lm.manager.num_usable_pages(0) == eng.lm.num_pages
    assert sum(t.numel() * t.element_size() for t in eng.lm.cache.pages) == (eng.lm.num_pages + 1) * page_bytes <= budget
    prompts = list(helpers.random_tokens(cfg["vocab_size"], (40, 3), seed=2).values())
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=8, ignore_eos_token=True))
    for p, o in zip(prompts, outs):
        helpers.greedy_agreement(w, cfg, p, o.token_ids)


def test_smoke_entry():
    import __graft_entry__ as g

    g.smoke()
