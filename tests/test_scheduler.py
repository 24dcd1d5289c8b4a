"""The scheduler's decisions, on the CPU with a host-only cache manager: admission,
the token budget, portions, decoding first, finishing and freeing, and what happens
when pages run out (preemption of the last admitted, recomputation)."""
import pytest

from tuff_b200.cache import CacheManager
from tuff_b200.engine.scheduler import RequestStatus, Scheduler, SchedulerError
from tuff_b200.parts import PagedKVNeed, StateNeed
from tuff_b200.sampling import SamplingParams


def make(max_tokens=64, page_size=4, budget=16, max_running=4, max_requests=4, ctx=None):
    cm = CacheManager([StateNeed((2, 8)), PagedKVNeed(2, 16)], page_size, max_tokens, max_requests)
    return cm, Scheduler(cm, max_batched_tokens=budget, max_running=max_running, max_context=ctx)


def run_step(cm, sch, next_token=lambda req: 1000 + len(req.output)):
    """What the engine does with a plan, without a model."""
    plan = sch.plan()
    assert len({id(e.request) for e in plan.entries}) == len(plan.entries)
    assert plan.n_tokens <= sch.max_batched_tokens
    for e in plan.entries:
        r = e.request                 # an entry continues exactly where the request's cache ends
        assert e.tokens == r.all_tokens()[r.n_cached:r.n_cached + len(e.tokens)] and e.tokens
        assert e.samples == (r.n_cached + len(e.tokens) == len(r.all_tokens()))
        cm.reserve(e.request.cache, len(e.tokens))
    for e in plan.entries:
        cm.commit(e.request.cache, len(e.tokens))
    sampled = [next_token(e.request) for e in plan.entries if e.samples]
    done = sch.update(plan, sampled)
    cm.check()
    return plan, done


def test_prompt_is_cut_under_the_budget_then_decoded():
    cm, sch = make(budget=16)
    r = sch.add("a", list(range(40)), SamplingParams(max_new_tokens=3))
    sizes = []
    while sch.has_work():
        plan, _ = run_step(cm, sch)
        sizes.append([(len(e.tokens), e.samples) for e in plan.entries])
    assert sizes == [[(16, False)], [(16, False)], [(8, True)], [(1, True)], [(1, True)]]
    assert r.output == [1000, 1001, 1002] and r.status is RequestStatus.FINISHED and r.finish_reason == "length"
    assert cm.groups[0].pool.n_free == 16 and cm.slots.n_free == 4       # freed in the same tick


def test_decode_first_then_running_prompts_then_admission():
    cm, sch = make(max_tokens=256, budget=10)
    a = sch.add("a", [1, 2, 3], SamplingParams(max_new_tokens=8))
    run_step(cm, sch)                                   # a: whole prompt, samples
    b = sch.add("b", list(range(14)), SamplingParams(max_new_tokens=2))
    c = sch.add("c", list(range(5)), SamplingParams(max_new_tokens=2))
    plan, _ = run_step(cm, sch)
    assert [(e.request.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 9)]
    assert [r.request_id for r in plan.admitted] == ["b"]
    plan, _ = run_step(cm, sch)                         # a decodes, b's rest, c admitted with what is left
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in plan.entries] == \
        [("a", 1, True), ("b", 5, True), ("c", 4, False)]
    plan, _ = run_step(cm, sch)
    assert [(e.request.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 1), ("c", 1)]
    assert sch.stats["prompt_tokens"] == 3 + 14 + 5


def test_max_running_and_slots_bound_admission():
    cm, sch = make(max_tokens=256, budget=64, max_running=2)
    for i in range(4):
        sch.add(i, [1, 2, 3], SamplingParams(max_new_tokens=2))
    plan, _ = run_step(cm, sch)
    assert len(plan.entries) == 2 and len(sch.waiting) == 2
    plan, done = run_step(cm, sch)                      # both finish (2 tokens each)
    assert len(done) == 2
    plan, _ = run_step(cm, sch)
    assert [e.request.request_id for e in plan.entries] == [2, 3]


def test_pages_run_out_preempts_last_admitted_and_recomputes():
    cm, sch = make(max_tokens=32, page_size=4, budget=64)          # 8 pages
    a = sch.add("a", list(range(14)), SamplingParams(max_new_tokens=8))   # 4 pages, grows to 6
    b = sch.add("b", list(range(100, 114)), SamplingParams(max_new_tokens=8))
    outs = {}
    preempted = []
    steps = 0
    while sch.has_work():
        plan, done = run_step(cm, sch, next_token=lambda req: (req.key + 1) * 1000 + len(req.output))
        preempted += [r.request_id for r in plan.preempted]
        for r in done:
            outs[r.request_id] = r.output
        steps += 1
        assert steps < 200
    assert preempted and set(preempted) == {"b"}        # the one admitted last gives way, never the first
    assert b.preemptions >= 1
    assert outs["a"] == [1000 + i for i in range(8)] and outs["b"] == [2000 + i for i in range(8)]
    assert cm.groups[0].pool.n_free == 8 and cm.slots.n_free == 4


def test_preempted_request_recomputes_prompt_plus_outputs():
    cm, sch = make(max_tokens=24, page_size=4, budget=64)          # 6 pages
    a = sch.add("a", list(range(11)), SamplingParams(max_new_tokens=6))
    b = sch.add("b", list(range(50, 59)), SamplingParams(max_new_tokens=6))
    seen = []
    while sch.has_work():
        plan, _ = run_step(cm, sch)
        for r in plan.preempted:
            seen.append((r.request_id, list(r.output)))
            assert r.n_cached == 0 and r.status is RequestStatus.WAITING and sch.waiting[0] is r
    # b was preempted after it had produced tokens; they were kept and fed again (run_step checks
    # that every entry continues the request's prompt + outputs from its cache's end)
    assert seen and seen[0][0] == "b" and any(out for _, out in seen)
    assert b.output == [1000 + i for i in range(6)] and a.output == [1000 + i for i in range(6)]


def test_preempted_request_returns_to_the_head_of_the_queue():
    """A request that had to give its pages back is admitted again before requests that came after it."""
    cm, sch = make(max_tokens=32, page_size=4, budget=64, max_running=2)   # 8 pages, two may run
    sch.add("a", list(range(14)), SamplingParams(max_new_tokens=8))
    sch.add("b", list(range(100, 114)), SamplingParams(max_new_tokens=8))
    sch.add("c", list(range(200, 206)), SamplingParams(max_new_tokens=2))
    order, hit = [], False
    steps = 0
    while sch.has_work():
        plan, done = run_step(cm, sch)
        order += [r.request_id for r in plan.admitted]
        for r in plan.preempted:
            hit = True
            assert [w.request_id for w in sch.waiting][:2] == [r.request_id, "c"]
        steps += 1
        assert steps < 300
    assert hit and order.index("c") > max(i for i, rid in enumerate(order) if rid == "b")


def test_errors():
    cm, sch = make(max_tokens=16, ctx=32)
    with pytest.raises(SchedulerError):
        sch.add("empty", [], SamplingParams())
    with pytest.raises(SchedulerError):
        sch.add("long", list(range(30)), SamplingParams(max_new_tokens=3))     # beyond the context
    with pytest.raises(SchedulerError):
        sch.add("big", list(range(20)), SamplingParams(max_new_tokens=3))      # beyond the whole cache
    r = sch.add("zero", [1, 2], SamplingParams(max_new_tokens=0))
    assert r.status is RequestStatus.FINISHED and not sch.has_work()


def test_stop_token_and_context_limit():
    cm, sch = make(max_tokens=64, ctx=12)
    a = sch.add("a", [1, 2, 3], SamplingParams(max_new_tokens=9, stop_token_ids=(1002,)))
    while sch.has_work():
        run_step(cm, sch)
    assert a.output == [1000, 1001, 1002] and a.finish_reason == "stop"
    b = sch.add("b", [1, 2, 3, 4], SamplingParams(max_new_tokens=8))
    while sch.has_work():
        run_step(cm, sch)
    assert b.finish_reason == "length" and len(b.output) == 8


def test_same_arrivals_same_plans():
    def trace():
        cm, sch = make(max_tokens=48, page_size=4, budget=12)
        for i, n in enumerate((9, 17, 5, 11)):
            sch.add(i, list(range(n)), SamplingParams(max_new_tokens=5))
        out = []
        while sch.has_work():
            plan, _ = run_step(cm, sch)
            out.append([(e.request.request_id, tuple(e.tokens), e.samples) for e in plan.entries])
        return out
    assert trace() == trace()


def run_ahead_loop(cm, sch, next_token):
    """The engine's loop with steps planned ahead of the sampled tokens where the scheduler
    allows it, without a model: returns how many steps were planned ahead."""
    ahead, n_ahead = None, 0
    while sch.has_work() or ahead is not None:
        if ahead is not None:
            plan, ahead = ahead, None
        else:
            plan = sch.plan()
            for e in plan.entries:
                cm.reserve(e.request.cache, len(e.tokens))
                cm.commit(e.request.cache, len(e.tokens))
        nxt = sch.plan_ahead(plan)
        if nxt is not None:
            n_ahead += 1
            for e in nxt.entries:
                assert e.tokens == [0] and e.samples and e.request.n_pending() == 0
                cm.reserve(e.request.cache, 1)
                cm.commit(e.request.cache, 1)
        sampled = [next_token(e.request) for e in plan.entries if e.samples]
        sch.update(plan, sampled)
        cm.check()
        if nxt is not None and sch.running:
            ahead = nxt
    return n_ahead


def test_steps_planned_ahead_of_their_tokens():
    """While everybody decodes and nothing else can happen, the next step is planned before the
    tokens of the current one are known: not while a prompt is in portions, not while someone
    waits, not when a request reaches its length with the pending token; a request that meets a
    stop token in mid-flight is skipped by the step that was planned ahead; the outputs are those of
    the plain loop."""
    def token(req):
        return 7 if (req.request_id == "b" and len(req.output) == 5) else 1000 + len(req.output)

    def requests(sch):
        return [sch.add("a", list(range(9)), SamplingParams(max_new_tokens=12)),
                sch.add("b", list(range(21)), SamplingParams(max_new_tokens=20, stop_token_ids=(7,))),
                sch.add("c", list(range(3)), SamplingParams(max_new_tokens=4))]

    cm, sch = make(max_tokens=256, budget=8, max_running=4)
    plain = requests(sch)
    while sch.has_work():
        run_step(cm, sch, token)
    cm2, sch2 = make(max_tokens=256, budget=8, max_running=4)
    ahead = requests(sch2)
    n_ahead = run_ahead_loop(cm2, sch2, token)
    assert [r.output for r in ahead] == [r.output for r in plain]
    assert [r.finish_reason for r in ahead] == ["length", "stop", "length"]
    assert n_ahead >= 4 and not cm2.live
    # nothing is planned ahead of a prompt in portions, of a waiting request, or of a last token
    cm3, sch3 = make(max_tokens=256, budget=8, max_running=1)
    r1 = sch3.add("x", list(range(20)), SamplingParams(max_new_tokens=3))
    r2 = sch3.add("y", list(range(4)), SamplingParams(max_new_tokens=2))
    seen = []
    while sch3.has_work():
        plan = sch3.plan()
        for e in plan.entries:
            cm3.reserve(e.request.cache, len(e.tokens)); cm3.commit(e.request.cache, len(e.tokens))
        seen.append(sch3.plan_ahead(plan) is not None)
        sch3.update(plan, [1000 for e in plan.entries if e.samples])
    assert not any(seen)            # "y" waits all the while "x" runs, and then "y" has two tokens to go
    assert r1.finish_reason == r2.finish_reason == "length"
