"""The host side of the engine without a GPU: engine loop, scheduler, sampler plumbing, stop rules and the
handling of a kernel's status word, driven through ``Engine`` with the torch stand-in of host_ops.py in
place of the kernels.  What the kernels compute is tested on the GPU; here the questions are which
tokens run when, what is sampled with which parameters, and what comes back."""
import pytest
import torch

import helpers
import plain_llama as P
from host_ops import HostOps


def _engine(d, page, **kw):
    from atoma_infer_b200.engine import Engine

    kw.setdefault("num_gpu_blocks_override", 64)
    kw.setdefault("max_num_sequences", 4)
    kw.setdefault("max_num_batched_tokens", 16)
    return Engine(d, dtype="float32", block_size=page, cuda_graphs=False, ops=HostOps(), **kw)


def test_greedy_through_the_engine_with_few_pages(tiny_models):
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["A"]
    w = helpers.read_weights(d)
    prompts = list(helpers.random_tokens(cfg["vocab_size"], (3, 14, 9, 21, 6), seed=4).values())
    want = [P.generate_greedy(w, cfg, p, 12) for p in prompts]
    eng = _engine(d, page, num_gpu_blocks_override=13, max_num_batched_tokens=10)  # 52 tokens of cache
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=12, ignore_eos_token=True))
    assert [o.token_ids for o in outs] == want
    assert eng.scheduler.num_preemptions > 0
    assert eng.lm.manager.audit() == "" and eng.lm.manager.num_requests() == 0
    assert eng.lm.manager.num_free_pages(0) == eng.lm.manager.num_usable_pages(0)


def test_sampling_options_reach_the_sampler(tiny_models):
    """top-k, top-p, both, and a repetition penalty, each request with its own seed, in one batch."""
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["A"]
    w = helpers.read_weights(d)
    prompts = list(helpers.random_tokens(cfg["vocab_size"], (5, 11, 8, 4), seed=6).values())
    sps = [SamplingParams(temperature=0.9, top_k=5, random_seed=11, max_new_tokens=6, ignore_eos_token=True),
           SamplingParams(temperature=1.3, top_p=0.7, random_seed=12, max_new_tokens=6, ignore_eos_token=True),
           SamplingParams(temperature=0.7, top_k=9, top_p=0.8, random_seed=13, max_new_tokens=6, ignore_eos_token=True),
           SamplingParams(temperature=0.8, repetition_penalty=1.5, repeat_last_n=6, random_seed=14, max_new_tokens=6,
                          ignore_eos_token=True)]
    want = [helpers.plain_sampled(w, cfg, p, 6, sp) for p, sp in zip(prompts, sps)]
    got = [o.token_ids for o in _engine(d, page).generate(prompts, sps)]
    assert got == want


def test_whole_prompts_only_without_chunked_prefill(tiny_models):
    """``enable_chunked_prefill=False``: a step holds whole prompts or decode tokens, never both
    (backends/vllm/src/scheduler.rs:1057-1217); the tokens are the same."""
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["A"]
    w = helpers.read_weights(d)
    prompts = list(helpers.random_tokens(cfg["vocab_size"], (12, 13, 9), seed=8).values())
    want = [P.generate_greedy(w, cfg, p, 5) for p in prompts]
    eng = _engine(d, page, enable_chunked_prefill=False, max_num_batched_tokens=24, max_model_len=24)
    ids = [eng.add_request(p, SamplingParams(do_sample=False, max_new_tokens=5, ignore_eos_token=True)) for p in prompts]
    kinds, done = [], {}
    run = eng.lm.step.run

    def spy(entries):
        kinds.append(sorted({"prompt" if len(e.tokens) > 1 else "decode" for e in entries}))
        return run(entries)

    eng.lm.step.run = spy
    while eng.has_unfinished():
        for o in eng.step():
            done[o.request_id] = o
    assert [done[i].token_ids for i in ids] == want
    assert all(len(k) == 1 for k in kinds), kinds           # never a prompt beside a decode token
    assert kinds[0] == ["prompt"] and kinds[1] == ["prompt"]  # 12 + 13 exceed the budget of 24: two prompt steps


def test_a_status_word_ends_the_steps_requests_with_an_error(tiny_models, capsys):
    """A kernel that gives up a wait, or meets a bad page, raises a status word instead of hanging.  The
    engine reads the words with the step's tokens: the requests of that step end with reason "error", their
    pages come back, the word is cleared and later requests run as if nothing had happened."""
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = tiny_models["A"]
    w = helpers.read_weights(d)
    sp = SamplingParams(do_sample=False, max_new_tokens=6, ignore_eos_token=True)
    eng = _engine(d, page)
    ops = eng.lm.rt.ops
    ops.fail_at_launch = (ops.launches + 40, 3, 5)  # "tensor-core attention block 4 gave up", a few steps in
    outs = eng.generate([[1, 2, 3, 4], [9, 8, 7]], sp)
    assert [o.finish_reason for o in outs] == ["error", "error"]
    assert all("attention block (4)" in o.error for o in outs)
    assert eng.num_device_errors >= 1 and not any(ops.status.tolist())
    assert "device status" in capsys.readouterr().err
    assert eng.lm.manager.num_requests() == 0 and eng.lm.manager.audit() == ""
    assert eng.lm.manager.num_free_pages(0) == eng.lm.manager.num_usable_pages(0)
    again = eng.generate([[1, 2, 3, 4]], sp)[0]
    assert again.finish_reason == "length" and again.token_ids == P.generate_greedy(w, cfg, [1, 2, 3, 4], 6)


def test_step_function_refuses_token_ids_outside_the_vocabulary(tiny_models):
    from atoma_infer_b200.engine import StepEntry

    d, cfg, page = tiny_models["A"]
    eng = _engine(d, page)
    step, mgr = eng.lm.step, eng.lm.manager
    for bad in ([1, cfg["vocab_size"]], [-1], [3, -2], [-70000]):
        with pytest.raises(ValueError, match="token ids"):
            step.run([StepEntry(7, bad, [0])])
        assert mgr.num_requests() == 0 and mgr.num_free_pages(0) == mgr.num_usable_pages(0)
    logits = step.run([StepEntry(7, [1, 2], [1])])
    assert logits.shape == (1, cfg["vocab_size"])
    # the one negative id a decode step may bring: "what the sampler left in my own slot"
    eng.lm.rt.ops.last_tokens[mgr.state_slot(7)] = 5
    a = step.run([StepEntry(7, [-1 - mgr.state_slot(7)], [0])])
    step.finish(7)
    step.run([StepEntry(8, [1, 2], [])])
    b = step.run([StepEntry(8, [5], [0])])
    assert torch.equal(a, b)
    with pytest.raises(ValueError, match="token ids"):
        step.run([StepEntry(8, [-1 - (mgr.state_slot(8) + 1)], [0])])  # another request's slot


def test_trace_lines_and_counters(tiny_models, capsys, monkeypatch):
    """ATOMA_INFER_TRACE=1: one line per step with the batch's composition; ``stats()`` counts what happened."""
    from atoma_infer_b200.sampling import SamplingParams

    monkeypatch.setenv("ATOMA_INFER_TRACE", "1")
    d, cfg, page = tiny_models["A"]
    eng = _engine(d, page, max_num_batched_tokens=8)
    eng.generate([[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], [5, 6, 7, 8, 9, 10, 11, 12, 13]], SamplingParams(do_sample=False, max_new_tokens=3, ignore_eos_token=True))
    lines = [l for l in capsys.readouterr().err.splitlines() if l.startswith("[trace] step")]
    assert len(lines) == eng.num_steps and "8 prompt tokens, 0 decode tokens" in lines[0]
    assert any("4 prompt tokens, 1 decode tokens" in l for l in lines)  # a portion of the second prompt beside a decode token
    st = eng.stats()
    assert st["generated_tokens"] == 6 and st["steps"] == eng.num_steps and st["running"] == 0
    assert st["free_pages"] == st["usable_pages"]
