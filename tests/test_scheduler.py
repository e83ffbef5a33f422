"""The scheduler's decisions: admission, portions under the token budget, decode first, finishing,
and what happens when pages run out (preempt the youngest, recompute later)."""
import pytest

from inferrs_b200.cache.manager import CacheManager, GroupLayout
from inferrs_b200.engine.scheduler import Request, Scheduler, SchedulerError
from inferrs_b200.sampling.params import SamplingParams


def make(n_pages=64, page_size=4, max_batch=4, budget=16, max_positions=1000, eos=(), chunk=None, slots=8):
    m = CacheManager([GroupLayout("full")], page_size, [n_pages], slots)
    return Scheduler(m, max_batch, budget, max_positions, eos, chunk), m


def req(rid, n, max_tokens=4, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams.greedy(max_tokens=max_tokens, **kw), seed=0)


def run_step(s, m, token=7):
    """Plan a step, pretend to run it (reserve and commit as the step function does) and sample ``token``."""
    plan, ended = s.plan()
    if plan:
        m.reserve({e.request.rid: e.n for e in plan})
        for e in plan:
            m.commit(e.request.rid, e.n)
    fin = s.update(plan, [token] * sum(e.samples for e in plan))
    m.check_invariants()
    return plan, ended + fin


def test_prompts_are_cut_under_the_budget_and_decodes_go_first():
    s, m = make(budget=16)
    s.add(req("a", 10)); s.add(req("b", 30))
    plan, _ = run_step(s, m)
    assert [(e.request.rid, e.start, e.n, e.samples) for e in plan] == [("a", 0, 10, True), ("b", 0, 6, False)]
    plan, _ = run_step(s, m)   # a decodes one token first, b gets the rest of the budget
    assert [(e.request.rid, e.start, e.n, e.samples) for e in plan] == [("a", 10, 1, True), ("b", 6, 15, False)]
    plan, _ = run_step(s, m)
    assert [(e.request.rid, e.start, e.n, e.samples) for e in plan] == [("a", 11, 1, True), ("b", 21, 9, True)]
    assert sum(e.n for e in plan) <= 16


def test_prefill_chunk_limits_a_portion():
    s, m = make(budget=64, chunk=8)
    s.add(req("a", 20))
    sizes = []
    while True:
        plan, fin = run_step(s, m)
        sizes.append(plan[0].n)
        if plan[0].samples:
            break
    assert sizes == [8, 8, 4]


def test_admission_is_first_come_first_served_up_to_the_batch_size():
    s, m = make(max_batch=2, budget=100)
    for i in range(4):
        s.add(req(i, 5, max_tokens=2))
    plan, _ = run_step(s, m)
    assert [e.request.rid for e in plan] == [0, 1]
    plan, fin = run_step(s, m)            # both sample their second token and finish
    assert sorted(r.rid for r in fin) == [0, 1] and all(r.finish_reason == "length" for r in fin)
    plan, _ = run_step(s, m)
    assert [e.request.rid for e in plan] == [2, 3]
    assert m.n_live == 2


def test_finish_reasons():
    s, m = make(eos=(7,), max_positions=14)
    s.add(req("stop", 3, max_tokens=9))
    s.add(req("ignores", 3, max_tokens=2, ignore_eos=True))
    s.add(Request("own", [1, 2], SamplingParams.greedy(max_tokens=9, stop_token_ids=(5,)), seed=0))
    plan, fin = run_step(s, m, token=5)
    assert {r.rid: r.finish_reason for r in fin} == {"own": "stop"}
    plan, fin = run_step(s, m, token=7)
    assert {r.rid: r.finish_reason for r in fin} == {"ignores": "length", "stop": "stop"}
    s.add(req("ctx", 12, max_tokens=50))   # 14 positions: two more tokens fit
    reasons = []
    while not s.idle:
        reasons += [r.finish_reason for r in run_step(s, m, token=1)[1]]
    assert reasons == ["length"] and m.n_live == 0


def test_refusals_when_added():
    s, m = make(n_pages=4, page_size=4, max_positions=50)
    with pytest.raises(SchedulerError, match="empty"):
        s.add(Request("e", [], SamplingParams.greedy(), 0))
    with pytest.raises(SchedulerError, match="even alone"):
        s.add(req("big", 16))
    with pytest.raises(SchedulerError, match="positions"):
        s.add(req("long", 50))


def test_out_of_pages_preempts_the_youngest_and_recomputes():
    s, m = make(n_pages=6, page_size=4, budget=64, max_batch=4)
    s.add(req("old", 8, max_tokens=12)); s.add(req("young", 8, max_tokens=12))
    plan, _ = run_step(s, m)              # 2 + 2 pages hold the prompts
    plan, _ = run_step(s, m)              # each takes its third page: the pool is full
    assert m.pools[0].n_free == 0
    for _ in range(3):
        plan, _ = run_step(s, m)          # positions 9..11 fit the third pages
    plan, _ = run_step(s, m)              # position 12 needs a fourth page: the youngest goes
    assert [e.request.rid for e in plan] == ["old"] and s.n_preemptions == 1
    young = s.waiting[0]
    assert young.rid == "young" and young.n_computed == 0 and len(young.output) == 5 and not m.has("young")
    outputs = {}
    while not s.idle:
        for r in run_step(s, m)[1]:
            outputs[r.rid] = r
    assert len(outputs["old"].output) == 12 and len(outputs["young"].output) == 12
    assert outputs["young"].n_preempted >= 1 and m.pools[0].n_free == 6


def test_a_lone_request_that_outgrows_the_cache_ends_with_length():
    s, m = make(n_pages=3, page_size=4, budget=64)
    s.add(req("r", 8, max_tokens=100))
    fin = []
    while not s.idle:
        fin += run_step(s, m)[1]
    assert [r.finish_reason for r in fin] == ["length"] and len(fin[0].output) == 5
    assert m.pools[0].n_free == 3 and m.n_live == 0


def test_abort_frees_everything():
    s, m = make()
    s.add(req("a", 9)); s.add(req("b", 9))
    run_step(s, m)
    assert s.abort("a").finish_reason == "cancelled" and not m.has("a")
    assert s.abort("nobody") is None
    s.add(req("c", 3))
    assert s.abort("c").finish_reason == "cancelled" and len(s.waiting) == 0
    m.check_invariants()


def launch(s, m, may_preempt=True):
    """Plan and launch a step as the engine does when it goes one ahead: the tokens are not known yet."""
    planned = s.plan(may_preempt=may_preempt)
    if planned is None:
        return None
    plan, ended = planned
    assert not ended
    m.reserve({e.request.rid: e.n for e in plan})
    for e in plan:
        m.commit(e.request.rid, e.n)
    s.advance(plan)
    return plan


def shape(plan):
    return [(e.request.rid, e.start, e.n, e.samples) for e in plan]


def test_the_next_step_is_planned_before_the_tokens_of_the_last_are_known():
    """``advance`` at the launch, ``deliver`` when the tokens come: in between the request counts one token that
    nobody knows yet, and the next plan gives it a step of one token at the place after its known tokens."""
    s, m = make(budget=16, eos=(99,))
    s.add(req("a", 10, max_tokens=8)); s.add(req("b", 30, max_tokens=8))
    p1 = launch(s, m)
    assert shape(p1) == [("a", 0, 10, True), ("b", 0, 6, False)]
    a = p1[0].request
    assert (a.n_tokens, a.n_in_flight, a.n_pending) == (10, 1, 1)
    p2 = launch(s, m, may_preempt=False)        # a's first token is still on its way
    assert shape(p2) == [("a", 10, 1, True), ("b", 6, 15, False)]
    assert p2[0].start + p2[0].n > a.n_tokens    # the engine sees from this that the token comes from the device
    assert a.n_in_flight == 2 and a.n_pending == 1
    assert s.deliver(p1, [5]) == []
    assert (a.output, a.n_in_flight, a.n_pending) == ([5], 1, 1)
    p3 = launch(s, m, may_preempt=False)
    assert shape(p3) == [("a", 11, 1, True), ("b", 21, 9, True)]
    # the token of the second step ends a: the third step, already launched, ran a in vain
    fin = s.deliver(p2, [99])
    assert [r.rid for r in fin] == ["a"] and a.finish_reason == "stop" and not m.has("a")
    alive = [e for e in p3 if e.request.finish_reason is None]
    assert s.deliver(alive, [6]) == []
    b = p3[1].request
    assert (b.output, b.n_in_flight, b.n_pending) == ([6], 0, 1)
    m.check_invariants()
    # update is both at once
    plan, _ = s.plan()
    m.reserve({e.request.rid: e.n for e in plan})
    m.commit("b", 1)
    s.update(plan, [7])
    assert (b.output, b.n_in_flight, b.n_computed) == ([6, 7], 0, 31)


def test_a_plan_that_would_preempt_is_not_made_while_a_step_is_on_its_way():
    """Too few pages for the next tokens: asked not to preempt, the scheduler answers None and changes nothing; a
    plan that may preempt is refused while tokens are on their way (the youngest request's last token would be
    lost) and made once they are delivered."""
    s, m = make(n_pages=4, page_size=4, budget=32)
    s.add(req("old", 7, max_tokens=20)); s.add(req("young", 7, max_tokens=20))
    p1 = launch(s, m)
    assert shape(p1) == [("old", 0, 7, True), ("young", 0, 7, True)]     # two pages each: the cache is full
    p2 = launch(s, m, may_preempt=False)
    assert shape(p2) == [("old", 7, 1, True), ("young", 7, 1, True)]     # the eighth places are in the pages held
    s.deliver(p1, [3, 4])
    before = (m.pools[0].n_free, [r.rid for r in s.running], [r.rid for r in s.waiting], s.n_preemptions)
    assert s.plan(may_preempt=False) is None                             # a ninth place needs a third page
    assert before == (m.pools[0].n_free, [r.rid for r in s.running], [r.rid for r in s.waiting], s.n_preemptions)
    with pytest.raises(SchedulerError, match="delivered"):
        s.plan()
    s.deliver(p2, [5, 6])
    plan, ended = s.plan()
    assert not ended and s.n_preemptions == 1
    assert shape(plan) == [("old", 8, 1, True)]
    young = p1[1].request
    assert young in s.waiting and young.n_computed == 0 and young.output == [4, 6] and young.n_in_flight == 0
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_the_native_scheduler_decides_as_the_plain_model_does(seed):
    """Random requests (lengths, token limits, stop tokens), random sampled tokens, a cache so small that requests
    are preempted and some outgrow it, aborts, and steps launched one ahead: the native scheduler over the native
    cache book and the plain Python model over the plain book must make the same plans, end the same requests
    for the same reasons and hand out the same pages."""
    import random
    import plain_cache
    import plain_scheduler
    rng = random.Random(seed)
    page_size, n_pages, slots = rng.choice([(4, 24, 5), (8, 10, 4), (4, 40, 3)])
    budget, chunk, max_batch = rng.choice([(16, None, 4), (24, 8, 5), (9, 5, 3)])
    max_positions, eos = 90, (3,)
    m = CacheManager([GroupLayout("full")], page_size, [n_pages], slots)
    s = Scheduler(m, max_batch, budget, max_positions, eos, chunk)
    pm = plain_cache.CacheManager([plain_cache.GroupLayout("full")], page_size, [n_pages], slots)
    ps = plain_scheduler.Scheduler(pm, max_batch, budget, max_positions, eos, chunk)

    def new_request(i):
        n = rng.choice([1, 2, 5, 9, 17, 30, 60])
        params = SamplingParams(temperature=0.0, max_tokens=rng.choice([1, 3, 8, 40]),
                                stop_token_ids=rng.choice([(), (5,), (5, 6)]), ignore_eos=rng.random() < 0.2)
        prompt = [rng.randrange(10) for _ in range(n)]
        return (Request(i, list(prompt), params, seed=0), plain_scheduler.Request(i, list(prompt), params, seed=0))

    def shape_of(plan):
        return [(e.request.rid, e.start, e.n, e.samples) for e in plan]

    def launch_both(may_preempt):
        a, b = s.plan(may_preempt=may_preempt), ps.plan(may_preempt=may_preempt)
        assert (a is None) == (b is None)
        if a is None:
            return None
        (plan, ended), (pplan, pended) = a, b
        assert shape_of(plan) == shape_of(pplan)
        assert [(r.rid, r.finish_reason) for r in ended] == [(r.rid, r.finish_reason) for r in pended]
        for mgr, pl in ((m, plan), (pm, pplan)):
            if pl:
                mgr.reserve({e.request.rid: e.n for e in pl})
                for e in pl:
                    mgr.commit(e.request.rid, e.n)
        s.advance(plan)
        ps.advance(pplan)
        for e in plan:
            assert list(m.block_table(e.request.rid, 0)) == list(pm.block_table(e.request.rid, 0))
        return plan, pplan

    def deliver_both(step):
        plan, pplan = step
        alive = [e for e in plan if e.request.finish_reason is None]
        palive = [e for e in pplan if e.request.finish_reason is None]
        tokens = [rng.randrange(10) for e in alive if e.samples]
        fin, pfin = s.deliver(alive, tokens), ps.deliver(palive, tokens)
        assert [(r.rid, r.finish_reason, r.output) for r in fin] == [(r.rid, r.finish_reason, r.output) for r in pfin]

    n_added, in_flight, n_ahead = 0, None, 0
    for turn in range(300):
        if n_added < 40 and rng.random() < 0.35:
            a, b = new_request(n_added)
            try:
                s.add(a)
                refused = False
            except SchedulerError:
                refused = True
            if refused:
                with pytest.raises(plain_scheduler.SchedulerError):
                    ps.add(b)
            else:
                ps.add(b)
            n_added += 1
        if rng.random() < 0.04 and (s.running or s.waiting):
            victim = rng.choice([r.rid for r in list(s.running) + list(s.waiting)])
            assert s.abort(victim).finish_reason == ps.abort(victim).finish_reason == "cancelled"
        # as the engine does: the next step is launched before the last one's tokens are delivered where that can
        # be; else the tokens come first
        step = None
        if in_flight is not None and rng.random() < 0.8:
            step = launch_both(may_preempt=False)
            n_ahead += step is not None
        if in_flight is not None:
            deliver_both(in_flight)
            in_flight = None
        if step is None:
            step = launch_both(may_preempt=True)
        in_flight = step if step and step[0] else None
        s.check()
        m.check_invariants()
        pm.check_invariants()
        assert [r.rid for r in s.running] == [r.rid for r in ps.running]
        assert [r.rid for r in s.waiting] == [r.rid for r in ps.waiting]
        assert s.n_preemptions == ps.n_preemptions
        assert m.pools[0].n_free == pm.pools[0].n_free
    assert n_ahead > 20 and n_added == 40
