"""The scheduler's decisions, on the host: admission order, token budget, portions,
decode-before-prefill, what happens when pages run out, stop conditions."""
import pytest

from neurogrid_b200.cache import CacheManager, PagedNeed
from neurogrid_b200.engine.scheduler import FINISHED, Request, Scheduler
from neurogrid_b200.sampling import SamplingParams


def setup(pages=64, page_size=4, max_requests=4, max_seq_len=256, budget=64, chunk=None, eos=()):
    cache = CacheManager([PagedNeed(1, 16, None)], [pages], page_size, max_requests, max_seq_len)
    return cache, Scheduler(cache, max_tokens_per_step=budget, max_requests=max_requests, chunk_size=chunk,
                            eos_token_ids=eos)


def fake_token(req):
    """A next token that depends only on the request's own tokens so far."""
    return (sum(req.tokens) * 31 + len(req.tokens)) % 97 + 3


def drive(cache, sch, max_steps=10_000, to_end=True):
    """Run plans to the end the way the engine does (extend + advance stand for the step)."""
    log, finished = [], []
    for _ in range(max_steps):
        if not sch.has_work():
            break
        plan = sch.plan()
        finished += plan.failed
        for e in plan.entries:
            if not cache.is_live(e.request.id):
                cache.admit(e.request.id)
            cache.extend(e.request.id, e.count)
            cache.advance(e.request.id, e.count)
        cache.check()
        log.append(plan)
        finished += sch.commit(plan, [fake_token(e.request) for e in plan.entries if e.sample])
        cache.check()
    assert not (to_end and sch.has_work())
    return log, finished


def req(i, n, max_new=8, **kw):
    return Request(i, [(i * 7 + j) % 90 + 3 for j in range(n)], SamplingParams(temperature=0.0, max_new_tokens=max_new, **kw))


def test_fifo_budget_and_portions():
    cache, sch = setup(budget=64, chunk=48)
    for r in (req(0, 100), req(1, 50), req(2, 10)):
        sch.add(r)
    p = sch.plan()
    # request 0 gets a portion capped by chunk_size, request 1 the rest of the budget, 2 waits
    assert [(e.request.id, e.start, e.count, e.sample) for e in p.entries] == [(0, 0, 48, False), (1, 0, 16, False)]
    assert p.n_tokens == 64 and [r.id for r in sch.waiting] == [2]
    for e in p.entries:
        cache.admit(e.request.id); cache.extend(e.request.id, e.count); cache.advance(e.request.id, e.count)
    sch.commit(p, [])
    p = sch.plan()
    assert [(e.request.id, e.start, e.count, e.sample) for e in p.entries] == [(0, 48, 48, False), (1, 16, 16, False)]


def test_decode_tokens_ride_with_prompt_portions():
    cache, sch = setup(budget=32)
    sch.add(req(0, 5, max_new=20))
    log, _ = drive(cache, sch, max_steps=2, to_end=False)              # request 0 is decoding now
    sch.add(req(1, 70, max_new=2))
    p = sch.plan()
    assert [(e.request.id, e.count, e.sample) for e in p.entries] == [(0, 1, True), (1, 31, False)]


def test_everything_is_given_back_and_outputs_do_not_depend_on_the_pool():
    outs = {}
    for pages in (200, 24):                                  # 24 pages * 4 = 96 tokens: far too few for all at once
        cache, sch = setup(pages=pages, budget=48, chunk=16)
        reqs = [req(i, n, max_new=12) for i, n in enumerate([30, 17, 44, 9, 25, 38])]
        for r in reqs:
            sch.add(r)
        log, finished = drive(cache, sch)
        assert sorted(r.id for r in finished) == list(range(6))
        assert all(r.state == FINISHED and r.finish_reason == "length" and len(r.output) == 12 for r in reqs)
        assert cache.pages_free() == [pages] and cache.slots_free() == 4
        assert all(p.n_tokens <= 48 for p in log)
        outs[pages] = [r.output for r in reqs]
        if pages == 24:
            assert sum(len(p.preempted) for p in log) > 0    # the small pool did force preemptions
            assert sum(r.preemptions for r in reqs) > 0
    assert outs[200] == outs[24]


def test_preemption_takes_the_most_recently_admitted_and_requeues_it_first():
    cache, sch = setup(pages=11, page_size=4, budget=64)     # 44 tokens of room
    a, b = req(0, 18, max_new=30), req(1, 18, max_new=30)
    sch.add(a); sch.add(b)
    c = req(2, 4)
    victim = None
    for _ in range(40):
        plan = sch.plan()
        if plan.preempted:
            victim = plan.preempted
            break
        for e in plan.entries:
            if not cache.is_live(e.request.id):
                cache.admit(e.request.id)
            cache.extend(e.request.id, e.count); cache.advance(e.request.id, e.count)
        sch.commit(plan, [fake_token(e.request) for e in plan.entries if e.sample])
        if sch.waiting == type(sch.waiting)() and c.state == "waiting" and c not in sch.waiting and len(a.output) == 1:
            sch.add(c)
    assert victim is not None and victim[0] is b             # b was admitted after a
    assert b.fed == 0 and b.preemptions == 1 and not cache.is_live(b.id)
    assert sch.waiting[0] is b                               # ahead of anything that arrived later
    assert len(b.output) > 0                                 # its sampled tokens are kept for the recompute
    cache.check()


def test_a_request_that_cannot_fit_alone_finishes_with_cache_full():
    cache, sch = setup(pages=4, page_size=4, max_seq_len=256)        # 16 tokens of room
    big, small = req(0, 40), req(1, 6, max_new=3)
    sch.add(big); sch.add(small)
    log, finished = drive(cache, sch)
    assert big.finish_reason == "cache_full" and big.state == FINISHED
    assert small.finish_reason == "length" and len(small.output) == 3
    assert cache.pages_free() == [4]
    # growing beyond the pool in mid-decode ends the same way instead of hanging
    cache, sch = setup(pages=4, page_size=4)
    r = req(0, 10, max_new=50)
    sch.add(r)
    drive(cache, sch)
    assert r.finish_reason == "cache_full" and 0 < len(r.output) < 50 and cache.pages_free() == [4]


def test_stop_conditions():
    cache, sch = setup(eos=(11,), max_seq_len=20)
    r_eos, r_stop, r_len, r_ctx, r_ign = (req(0, 3, 50), req(1, 3, 50, stop_token_ids=(12,)), req(2, 3, 2),
                                          req(3, 15, 50), req(4, 3, 3, ignore_eos=True))
    toks = {0: [5, 11, 9], 1: [5, 12], 2: [5, 6, 7], 3: [4] * 50, 4: [11, 11, 11, 11]}
    for r in (r_eos, r_stop, r_len, r_ctx, r_ign):
        sch.add(r)
    # one admission wave of 4, the fifth follows
    for _ in range(100):
        if not sch.has_work():
            break
        plan = sch.plan()
        for e in plan.entries:
            if not cache.is_live(e.request.id):
                cache.admit(e.request.id)
            cache.extend(e.request.id, e.count); cache.advance(e.request.id, e.count)
        sch.commit(plan, [toks[e.request.id][len(e.request.output)] for e in plan.entries if e.sample])
    assert (r_eos.finish_reason, r_eos.output) == ("eos", [5, 11])
    assert (r_stop.finish_reason, r_stop.output) == ("stop", [5, 12])
    assert (r_len.finish_reason, r_len.output) == ("length", [5, 6])
    assert r_ctx.finish_reason == "context" and len(r_ctx.prompt) + len(r_ctx.output) == 20
    assert (r_ign.finish_reason, r_ign.output) == ("length", [11, 11, 11])
    assert cache.pages_free() == [64] and cache.slots_free() == 4


def test_slots_bound_admission():
    cache, sch = setup(max_requests=2, budget=64)
    for i in range(4):
        sch.add(req(i, 5, max_new=2))
    p = sch.plan()
    assert [e.request.id for e in p.entries] == [0, 1] and len(sch.waiting) == 2
    log, finished = drive(cache, sch)
    assert len(finished) == 4


def test_a_step_ahead_placeholders_and_late_stops():
    """The scheduler can plan the step after one whose tokens have not been read: placeholders
    stand in the outputs, a stop token found late cuts the output back and drops the token
    that was computed meanwhile, length limits are honoured without waiting."""
    from neurogrid_b200.engine.scheduler import PLACEHOLDER
    cache, sch = setup(eos=(11,), budget=64)
    a, b, c = req(0, 4, max_new=6), req(1, 3, max_new=2), req(2, 5, max_new=6)
    for r in (a, b, c):
        sch.add(r)

    def run(plan):
        for e in plan.entries:
            if not cache.is_live(e.request.id):
                cache.admit(e.request.id)
            cache.extend(e.request.id, e.count)
            cache.advance(e.request.id, e.count)

    p0 = sch.plan()                                   # the three prompts, all sampled
    run(p0)
    sch.commit_ahead(p0)
    assert [r.output for r in (a, b, c)] == [[PLACEHOLDER]] * 3 and all(r.pending == 1 for r in (a, b, c))
    p1 = sch.decode_ahead_plan()                      # decided without the tokens of p0
    assert [e.request.id for e in p1.entries] == [0, 1, 2]
    run(p1)
    sch.commit_ahead(p1)
    done = sch.finalize(p0, [5, 6, 11])               # c hits EOS on its first token
    assert [r.id for r in done] == [2] and c.output == [11] and c.finish_reason == "eos"
    assert not cache.is_live(2)
    p2 = sch.decode_ahead_plan()                      # b has its 2 tokens coming: it is left out
    assert [e.request.id for e in p2.entries] == [0]
    run(p2)
    sch.commit_ahead(p2)
    done = sch.finalize(p1, [7, 8, 9])                # c's token (9) is dropped
    assert [r.id for r in done] == [1] and b.output == [6, 8] and b.finish_reason == "length"
    assert c.output == [11]
    done = sch.finalize(p2, [12])
    assert done == [] and a.output == [5, 7, 12]
    # a prompt that waits and can be admitted stops the running ahead
    sch.add(req(3, 4))
    p3 = sch.plan()
    run(p3)
    sch.commit_ahead(p3)
    assert sch.decode_ahead_plan() is not None        # all run, nothing waits
    sch.add(req(4, 4))
    assert sch.decode_ahead_plan() is None            # a request could be admitted: decide with the tokens in hand
    cache.check()
