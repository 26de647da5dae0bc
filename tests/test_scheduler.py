"""The scheduler's decisions, on the reference's test geometry (pages of 4 tokens, a few
pages, small budgets; backends/vllm/src/scheduler.rs:2459-2491).  No GPU, no model: the
test plays the step function's part by advancing the cache itself."""
import pytest

from atoma_infer_b200.cache import CacheGroup, CacheManager, CacheNeed
from atoma_infer_b200.engine.scheduler import RUNNING, UNKNOWN, WAITING, Scheduler


def make(pages=8, budget=100, seqs=4, model_len=64, chunked=True, page_size=4):
    cm = CacheManager(page_size, [CacheGroup(CacheNeed.kv(1, 16), [0], pages + 1)], seqs)
    return cm, Scheduler(cm, max_num_batched_tokens=budget, max_num_seqs=seqs, max_model_len=model_len,
                         enable_chunked_prefill=chunked)


def run_step(cm, s, finish=()):
    """schedule -> 'run' -> every sampling entry gets a token (or finishes)."""
    plan = s.schedule()
    for e in plan.entries:
        assert cm.num_tokens(e.req) == e.context_len
        cm.advance(e.req, e.num_tokens)
    s.step_done()
    for e in plan.entries:
        if e.samples:
            s.finish(e.req) if e.req in finish else s.append_token(e.req)
    assert cm.audit() == ""
    return plan


def summary(plan):
    return [(e.req, e.num_tokens, e.samples) for e in plan.entries]


def test_fcfs_admission_under_the_token_budget_with_chunking():
    cm, s = make(pages=16, budget=10)
    for r, n in ((0, 6), (1, 7), (2, 3)):
        s.add_request(r, n)
    p = run_step(cm, s)
    assert summary(p) == [(0, 6, True), (1, 4, False)]  # the second prompt is clipped to what is left
    assert s.status(2) == WAITING
    p = run_step(cm, s)
    # running requests first (a decode, the rest of prompt 1), then the new prompt
    assert summary(p) == [(0, 1, True), (1, 3, True), (2, 3, True)]
    assert [e.is_prompt for e in p.entries] == [False, True, True]
    p = run_step(cm, s)
    assert summary(p) == [(0, 1, True), (1, 1, True), (2, 1, True)]


def test_a_portion_can_be_one_token_and_in_flight_prompts_stay_running():
    cm, s = make(pages=16, budget=4)
    s.add_request(0, 9)
    sizes = []
    for _ in range(3):
        p = run_step(cm, s)
        sizes.append(summary(p))
        assert s.status(0) == RUNNING  # the reference loses prompts in flight here (scheduler.rs:1313-1338)
    assert sizes == [[(0, 4, False)], [(0, 4, False)], [(0, 1, True)]]
    assert s.num_computed(0) == 9 and s.length(0) == 10


def test_without_chunking_prompts_go_whole_and_alone():
    cm, s = make(pages=16, budget=12, chunked=False, model_len=12)
    for r, n in ((0, 5), (1, 6), (2, 4)):
        s.add_request(r, n)
    assert summary(run_step(cm, s)) == [(0, 5, True), (1, 6, True)]  # 5 + 6 fit the budget, 4 more do not
    assert summary(run_step(cm, s)) == [(2, 4, True)]                  # a prompt-only step, decodes wait
    assert summary(run_step(cm, s)) == [(0, 1, True), (1, 1, True), (2, 1, True)]
    assert s.prompt_limit == 12


def test_max_num_seqs_bounds_the_running_queue():
    cm, s = make(pages=16, budget=100, seqs=2)
    for r in range(3):
        s.add_request(r, 2)
    assert [e.req for e in run_step(cm, s).entries] == [0, 1]
    assert [e.req for e in run_step(cm, s, finish={0}).entries] == [0, 1]
    assert [e.req for e in run_step(cm, s).entries] == [1, 2]


def test_too_long_prompts_are_ignored_and_do_not_block():
    cm, s = make(pages=4, budget=100, model_len=12)
    s.add_request(0, 13)  # longer than max_model_len
    s.add_request(1, 5)
    p = s.schedule()
    assert p.ignored == [0] and [e.req for e in p.entries] == [1] and s.status(0) == UNKNOWN
    cm2, s2 = make(pages=2, budget=100, model_len=64)
    s2.add_request(0, 9)  # 3 pages, the pool has 2: never fits
    assert s2.schedule().ignored == [0]


def test_a_prompt_that_does_not_fit_now_blocks_the_queue_behind_it():
    cm, s = make(pages=4, budget=100)
    s.add_request(0, 10)  # 3 of 4 pages
    s.add_request(1, 8)   # 2 pages: not now
    s.add_request(2, 2)   # would fit, but waits behind request 1
    assert [e.req for e in run_step(cm, s).entries] == [0]
    assert [e.req for e in run_step(cm, s).entries] == [0]
    assert s.num_waiting == 2
    assert [e.req for e in run_step(cm, s, finish={0}).entries] == [0]
    assert cm.num_free_pages() == 4  # a finished request gives its pages back at once
    assert [e.req for e in run_step(cm, s).entries] == [1, 2]


def test_out_of_pages_preempts_the_last_running_request_by_recompute():
    cm, s = make(pages=4, budget=100)
    s.add_request(0, 7)
    s.add_request(1, 7)
    assert summary(run_step(cm, s)) == [(0, 7, True), (1, 7, True)]  # 2 + 2 pages, both full after one decode
    assert summary(run_step(cm, s)) == [(0, 1, True), (1, 1, True)]
    p = run_step(cm, s)  # both need a third page, none is free: the last one goes
    assert p.preempted == [1] and summary(p) == [(0, 1, True)]
    assert s.status(1) == WAITING and s.num_computed(1) == 0 and s.length(1) == 9
    assert not cm.has_request(1) and s.num_preemptions == 1
    # no new admission in the step that preempted; afterwards request 1 starts over with its 9 tokens
    p = run_step(cm, s, finish={0})
    assert summary(p) == [(0, 1, True)]
    p = run_step(cm, s)
    assert summary(p) == [(1, 9, True)] and p.entries[0].context_len == 0 and p.entries[0].is_prompt


def test_a_lone_request_that_outgrows_the_cache_is_dropped_not_spun():
    cm, s = make(pages=2, budget=100)
    s.add_request(0, 7)
    for _ in range(2):
        assert summary(run_step(cm, s)) == [(0, 7 if _ == 0 else 1, True)]
    p = run_step(cm, s)  # 9 tokens need 3 pages, the pool has 2
    assert p.entries == [] and p.ignored == [0] and not cm.has_request(0)
    assert not s.has_unfinished() and cm.num_free_pages() == 2


def test_abort_from_either_queue_frees_everything():
    cm, s = make(pages=8, budget=6)
    s.add_request(0, 5)
    s.add_request(1, 5)
    run_step(cm, s)  # 0 whole, 1 clipped to one token
    s.finish(1)      # running, mid-prompt
    s.add_request(2, 3)
    s.finish(2)      # still waiting
    assert s.status(1) == UNKNOWN and s.status(2) == UNKNOWN and not cm.has_request(1)
    assert [e.req for e in run_step(cm, s).entries] == [0]
    s.finish(0)
    assert cm.num_free_pages() == 8 and cm.num_requests() == 0 and cm.audit() == ""
    with pytest.raises(Exception):
        s.finish(0)


def test_many_ignored_requests_in_one_step_do_not_lose_the_plan():
    """Forty prompts beyond the model length wait in front of two that fit, with four sequence slots: the
    step that drops the forty (backends/vllm/src/scheduler.rs:957-992 marks them ignored) still returns
    its whole plan, the two prompts run, and the scheduler forgets the dropped ones."""
    cm, s = make(pages=16, budget=32, seqs=4, model_len=12)
    for r in range(40):
        s.add_request(r, 13 + r % 5)
    s.add_request(100, 5)
    s.add_request(101, 12)
    p = run_step(cm, s)
    assert sorted(p.ignored) == list(range(40))
    assert summary(p) == [(100, 5, True), (101, 12, True)]
    assert all(s.status(r) == UNKNOWN for r in range(40))
    assert s.num_waiting == 0 and s.num_running == 2
    p = run_step(cm, s, finish=(100, 101))
    assert summary(p) == [(100, 1, True), (101, 1, True)] and not p.ignored
    assert cm.num_requests() == 0 and cm.num_free_pages(0) == cm.num_usable_pages(0)


def test_prompts_that_no_empty_cache_could_hold_are_ignored_in_any_number():
    cm, s = make(pages=4, budget=64, seqs=2, model_len=64)  # 16 tokens of cache
    for r in range(30):
        s.add_request(r, 17 + r)
    s.add_request(99, 16)
    p = run_step(cm, s)
    assert sorted(p.ignored) == list(range(30)) and summary(p) == [(99, 16, True)]
