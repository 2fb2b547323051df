"""The scheduler's decisions, on the host with bookkeeping-only caches."""

import numpy as np
import pytest

from ayaka_py_b200.cache import CacheGroupSpec, CacheManager
from ayaka_py_b200.engine.request import Request, StopCriteria
from ayaka_py_b200.engine.scheduler import RequestRefused, Scheduler
from ayaka_py_b200.parts.base import KVNeed
from ayaka_py_b200.sampling.params import SamplingParams, derive_seed


def make(pages=65, page_size=4, max_requests=8, batch_tokens=32, prefill_chunk=16, max_len=128, eos=None):
    cache = CacheManager([CacheGroupSpec("g", KVNeed(1, 16), 1)], kv_pages=pages, page_size=page_size,
                         max_requests=max_requests, max_len=max_len, device=None)
    return Scheduler(cache, batch_tokens=batch_tokens, prefill_chunk=prefill_chunk, max_model_len=max_len,
                     eos_token_id=eos), cache


def req(i, n, max_tokens=4, **kw):
    return Request(f"r{i}", list(range(1, n + 1)), SamplingParams(temperature=0.0), StopCriteria(max_tokens=max_tokens, **kw))


def drive(sched, cache, token=lambda s: 7, max_steps=10_000, log=None):
    """Runs the loop with a fake model.  Returns finished states in order."""
    done = []
    for _ in range(max_steps):
        if not sched.has_work():
            break
        plan = sched.schedule()
        assert plan is not None, "blocked although work waits"
        cache.check_invariants()
        if log is not None:
            log.append([(e.state.request.request_id, e.start, e.count, e.sample) for e in plan.entries])
        sampled = {e.state.request.request_id: token(e.state) for e in plan.entries if e.sample}
        done += sched.update(plan, sampled)
    assert not sched.has_work()
    cache.assert_clean()
    return done


def test_portions_decode_first_and_one_unfinished_prompt():
    sched, cache = make(batch_tokens=32, prefill_chunk=16)
    for i, n in enumerate([1, 9, 33, 20]):
        sched.add(req(i, n, max_tokens=3))
    log = []
    done = drive(sched, cache, log=log)
    # step 0: r0 and r1 whole, r2 starts with what is left of the chunk / budget
    assert log[0] == [("r0", 0, 1, True), ("r1", 0, 9, True), ("r2", 0, 16, False)]
    # step 1: decodes first, then r2 goes on; r3 may not start while r2 is unfinished
    assert log[1][:2] == [("r0", 1, 1, True), ("r1", 9, 1, True)]
    assert log[1][2] == ("r2", 16, 16, False) and len(log[1]) == 3
    assert log[2][-1] == ("r2", 32, 1, True) or ("r2", 32, 1, True) in log[2]
    for step in log:
        assert sum(c for _, _, c, _ in step) <= 32
        assert len({r for r, *_ in step}) == len(step)
        unfinished = [1 for r, s, c, smp in step if not smp]
        assert len(unfinished) <= 1
    assert sorted(s.request.request_id for s in done) == ["r0", "r1", "r2", "r3"]
    assert all(s.finish_reason == "length" and s.generated == 3 for s in done)
    assert sched.stats.preemptions == 0


def test_admission_rules():
    sched, cache = make(pages=9, page_size=4, max_len=64)         # 8 usable pages = 32 tokens
    with pytest.raises(RequestRefused):
        sched.add(req(0, 60, max_tokens=10))                      # beyond the model length
    with pytest.raises(RequestRefused):
        sched.add(req(1, 30, max_tokens=8))                       # could never fit the cache
    sched.add(req(2, 8))
    with pytest.raises(RequestRefused):
        sched.add(req(2, 8))                                      # duplicate id
    with pytest.raises(ValueError):
        Request("x", [])


def test_stop_rules():
    sched, cache = make(eos=9)
    sched.add(req(0, 3, max_tokens=10, stop_token_ids=(5,), min_tokens=3))
    sched.add(req(1, 3, max_tokens=10))
    sched.add(req(2, 3, max_tokens=10, ignore_eos=True))
    # The sampler bans r0's stop id for its first min_tokens tokens (the fake model here obeys the ban);
    # the first token that may be a stop is number min_tokens + 1 (request/stream.py:130-163).
    assert sched.banned_tokens(sched.states["r0"]) == (5, 9) and sched.banned_tokens(sched.states["r1"]) == ()
    assert sched.banned_tokens(sched.states["r0"], pending=3) == ()
    tokens = {"r0": iter([1, 1, 1, 5, 5]), "r1": iter([1, 9]), "r2": iter([9] * 10)}

    def fake(s):
        token = next(tokens[s.request.request_id])
        assert token not in sched.banned_tokens(s)
        return token

    done = drive(sched, cache, token=fake)
    by = {s.request.request_id: s for s in done}
    assert by["r0"].finish_reason == "stop" and by["r0"].generated == 4      # not before min_tokens
    assert by["r1"].finish_reason == "eos" and by["r1"].generated == 2
    assert by["r2"].finish_reason == "length" and by["r2"].generated == 10


def test_slots_bound_the_running_set():
    sched, cache = make(max_requests=2)
    for i in range(5):
        sched.add(req(i, 4, max_tokens=2))
    log = []
    drive(sched, cache, log=log)
    assert max(len(step) for step in log) <= 2


def test_pages_run_out_shrink_then_preempt_then_finish():
    # 8 usable pages of 4 tokens; three requests that each grow to 20 tokens cannot all live.
    sched, cache = make(pages=9, page_size=4, batch_tokens=64, prefill_chunk=64, max_len=32)
    for i in range(3):
        sched.add(req(i, 10, max_tokens=10))
    log = []
    done = drive(sched, cache, log=log)
    assert len(done) == 3 and all(s.generated == 10 for s in done)
    assert sched.stats.preemptions >= 1 and sched.stats.recomputed_tokens > 0
    victims = [s for s in done if s.preemptions]
    assert victims and all(s.request.request_id != "r0" for s in victims)     # the oldest is never the victim
    # a preempted request recomputes its prompt and what it generated, in one go or in portions
    for s in victims:
        restarts = [e for step in log for e in step if e[0] == s.request.request_id and e[1] == 0]
        assert len(restarts) == s.preemptions + 1


def test_prefill_is_shrunk_before_anyone_is_preempted():
    sched, cache = make(pages=7, page_size=4, batch_tokens=64, prefill_chunk=64, max_len=24)   # 24 tokens
    sched.add(req(0, 8, max_tokens=4))
    drive_one = sched.schedule()
    sched.update(drive_one, {"r0": 7})
    sched.add(req(1, 20, max_tokens=2))        # needs 5 pages, 4 are free
    plan = sched.schedule()
    got = {e.state.request.request_id: (e.start, e.count, e.sample) for e in plan.entries}
    assert got["r0"] == (8, 1, True)
    assert got["r1"] == (0, 10, False)         # halved once, fits
    assert sched.stats.preemptions == 0 and sched.stats.shrunk_steps == 1
    sched.update(plan, {"r0": 7})
    done = drive(sched, cache)
    assert {s.request.request_id for s in done} == {"r0", "r1"}


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_terminate_without_leaks(seed):
    rs = np.random.RandomState(seed)
    sched, cache = make(pages=int(rs.randint(12, 40)), page_size=4, max_requests=int(rs.randint(2, 7)),
                        batch_tokens=int(rs.randint(8, 48)), prefill_chunk=int(rs.randint(2, 24)), max_len=40)
    n = 0
    pending = []
    for i in range(25):
        plen, gen = int(rs.randint(1, 30)), int(rs.randint(1, 10))
        pending.append(req(i, plen, max_tokens=gen))
    done = []
    steps = 0
    while pending or sched.has_work():
        while pending and rs.rand() < 0.5:
            sched.add(pending.pop(0))
        if not sched.has_work():
            continue
        plan = sched.schedule()
        assert plan is not None
        steps += 1
        assert steps < 5000
        assert sum(e.count for e in plan.entries) <= sched.batch_tokens
        cache.check_invariants()
        done += sched.update(plan, {e.state.request.request_id: int(rs.randint(0, 100)) for e in plan.entries if e.sample})
    cache.assert_clean()
    assert len(done) == 25
    for s in done:
        assert s.generated == s.request.stop.max_tokens and s.finish_reason == "length"
        assert len(s.tokens) == s.prompt_len + s.generated


def test_seeds():
    sched, _ = make()
    a = sched.add(Request("a", [1], SamplingParams(seed=42), StopCriteria(max_tokens=4)))
    b = sched.add(Request("b", [1], stop=StopCriteria(max_tokens=4)))
    assert a.seed == 42 and b.seed == derive_seed(1) and 0 <= b.seed < 2 ** 63


def drive_ahead(sched, cache, token, arrivals=None, max_steps=10_000, log=None):
    """The engine's loop with lookahead and a fake model: a step's tokens become
    known only after the step behind it has been planned and "launched"."""
    done, inflight, step_no = [], None, 0
    arrivals = dict(arrivals or {})
    for _ in range(max_steps):
        for r in arrivals.pop(step_no, []):
            sched.add(r)
        step_no += 1
        if inflight is None:
            if not sched.has_work():
                if not arrivals:
                    break
                continue
            plan = sched.schedule()
            assert plan is not None
            sched.advance(plan)
            inflight = plan
        current = inflight
        inflight = sched.lookahead(current)
        if inflight is not None:
            sched.advance(inflight)
        cache.check_invariants()
        if log is not None:
            log.append(("ahead" if inflight is not None else "plain", [(e.state.request.request_id, e.start, e.count) for e in current.entries]))
        # tokens of `current` arrive now; the fake model only looks at what was known when the step was planned
        sampled = {e.state.request.request_id: token(e.state, e.start + e.count) for e in current.entries if e.sample}
        done += sched.resolve(current, sampled)
    assert not sched.has_work() and inflight is None
    cache.assert_clean()
    return done


def drive_plain(sched, cache, token, arrivals=None, max_steps=10_000):
    done, step_no = [], 0
    arrivals = dict(arrivals or {})
    for _ in range(max_steps):
        for r in arrivals.pop(step_no, []):
            sched.add(r)
        step_no += 1
        if not sched.has_work():
            if not arrivals:
                break
            continue
        plan = sched.schedule()
        assert plan is not None
        sampled = {e.state.request.request_id: token(e.state, e.start + e.count) for e in plan.entries if e.sample}
        done += sched.update(plan, sampled)
    cache.assert_clean()
    return done


@pytest.mark.parametrize("seed", range(6))
def test_lookahead_gives_the_same_tokens_and_reasons(seed):
    """Planning a decode step before the tokens of the step before it are known
    changes nothing that a request sees: same tokens, same finish reasons, EOS in
    the middle of a run included; the cache ends clean."""
    rs = np.random.RandomState(seed)
    lens = rs.randint(1, 30, size=6)
    limits = rs.randint(2, 14, size=6)

    def token(state, position):                    # a function of the request and the position only
        h = (state.ordinal * 7919 + position * 104729 + seed) % 23
        return 99 if h == 0 else 5 + h             # 99 is EOS for some positions

    results = []
    for ahead in (False, True):
        sched, cache = make(pages=40, page_size=4, max_requests=4, batch_tokens=24, prefill_chunk=8, max_len=64, eos=99)
        arrivals = {0: [req(i, int(lens[i]), max_tokens=int(limits[i])) for i in range(3)],
                    5: [req(3, int(lens[3]), max_tokens=int(limits[3]))],
                    9: [req(4, int(lens[4]), max_tokens=int(limits[4]), ignore_eos=True), req(5, int(lens[5]), max_tokens=int(limits[5]))]}
        log = []
        done = drive_ahead(sched, cache, token, arrivals, log=log) if ahead else drive_plain(sched, cache, token, arrivals)
        results.append({s.request.request_id: (tuple(s.tokens), s.finish_reason) for s in done})
        if ahead:
            assert any(kind == "ahead" for kind, _ in log) or seed < 0
    assert results[0] == results[1]
    assert len(results[0]) == 6


def test_lookahead_plans_past_prompts_and_leaves_out_who_finishes():
    sched, cache = make(pages=20, page_size=4, max_requests=4, batch_tokens=8)
    sched.add(req(0, 3, max_tokens=5))
    sched.add(req(1, 2, max_tokens=2))
    plan = sched.schedule()                        # both prompts, both sampled
    assert sched.lookahead(plan) is None           # not handed over yet: nothing is on its way
    sched.advance(plan)
    ahead = sched.lookahead(plan)                  # both decode with the tokens on their way
    assert ahead is not None and ahead.decode_only and ahead.token_rows == [0, 1]
    assert [(e.state.request.request_id, e.start, e.count, e.pending) for e in ahead.entries] == [("r0", 3, 1, True), ("r1", 2, 1, True)]
    sched.advance(ahead)
    sched.resolve(plan, {"r0": 7, "r1": 7})
    plan = ahead                                   # r1 reaches max_tokens with the token on its way
    ahead = sched.lookahead(plan)                  # ... so it is left out of the next step, and r0 takes row 0 of the tokens
    assert ahead is not None and [e.state.request.request_id for e in ahead.entries] == ["r0"]
    assert ahead.token_rows == [0] and [(e.start, e.count) for e in ahead.entries] == [(4, 1)]
    sched.advance(ahead)
    done = sched.resolve(plan, {"r0": 7, "r1": 7})
    assert [s.request.request_id for s in done] == ["r1"]
    cache.check_invariants()
    plan = ahead
    sched.add(req(2, 2, max_tokens=1))             # somebody waits now: its prompt goes beside the decoding request
    ahead = sched.lookahead(plan)
    assert [(e.state.request.request_id, e.start, e.count, e.pending, e.sample) for e in ahead.entries] == \
        [("r0", 5, 1, True, True), ("r2", 0, 2, False, True)]
    assert ahead.token_rows == [0] and not ahead.decode_only
    sched.advance(ahead)
    sched.resolve(plan, {"r0": 7})
    plan = ahead
    ahead = sched.lookahead(plan)                  # r0 has one token to go and r2 one of one: r0 goes on, r2 leaves
    assert [(e.state.request.request_id, e.start) for e in ahead.entries] == [("r0", 6)] and ahead.token_rows == [0]
    sched.advance(ahead)
    sched.resolve(plan, {"r0": 7, "r2": 7})
    assert sched.lookahead(ahead) is None          # r0's last token is on its way and nobody else is there
    sched.resolve(ahead, {"r0": 7})
    assert not sched.states or sorted(sched.states) == ["r0", "r1", "r2"]
    assert not sched.has_work()
    cache.assert_clean()


def test_lookahead_goes_on_with_a_prompt_in_portions():
    sched, cache = make(pages=40, page_size=4, max_requests=4, batch_tokens=6, prefill_chunk=4, max_len=64)
    sched.add(req(0, 2, max_tokens=9))
    plan = sched.schedule()
    sched.update(plan, {"r0": 7})
    sched.add(req(1, 10, max_tokens=3))
    plan = sched.schedule()                        # r0 decodes, r1's first portion beside it
    assert [(e.state.request.request_id, e.start, e.count, e.sample) for e in plan.entries] == [("r0", 2, 1, True), ("r1", 0, 4, False)]
    sched.advance(plan)
    for start, count, sample in ((4, 4, False), (8, 2, True)):
        ahead = sched.lookahead(plan)              # r0's token is on its way; r1's next portion is known
        assert ahead.token_rows == [0]
        assert [(e.state.request.request_id, e.start, e.count, e.sample, e.pending) for e in ahead.entries][1] == ("r1", start, count, sample, False)
        sched.advance(ahead)
        sched.resolve(plan, {"r0": 7})
        cache.check_invariants()
        plan = ahead
    ahead = sched.lookahead(plan)                  # both decode now: r0's token is row 0, r1's row 1
    assert ahead.decode_only and ahead.token_rows == [0, 1] and all(e.pending for e in ahead.entries)
    sched.advance(ahead)
    sched.resolve(plan, {"r0": 7, "r1": 7})
    sched.resolve(ahead, {"r0": 7, "r1": 7})
    cache.check_invariants()


def test_lookahead_takes_nothing_away():
    # 5 usable pages of 4 tokens, two requests of 7 tokens hold 4; a third waits for 8 tokens
    sched, cache = make(pages=6, page_size=4, max_requests=3, batch_tokens=16, prefill_chunk=16, max_len=32)
    sched.add(req(0, 7, max_tokens=12))
    sched.add(req(1, 7, max_tokens=12))
    plan = sched.schedule()
    sched.update(plan, {"r0": 1, "r1": 1})
    plan = sched.schedule()
    sched.advance(plan)
    sched.add(req(2, 8, max_tokens=2))
    free, slots, waiting = cache.free_pages(0), len(cache.free_slots), [s.request.request_id for s in sched.waiting]
    assert sched.lookahead(plan) is None           # r0 and r1 need a page each at position 8 and r2 two: 1 is free
    assert (cache.free_pages(0), len(cache.free_slots)) == (free, slots)           # the admission was taken back
    assert [s.request.request_id for s in sched.waiting] == waiting and len(sched.running) == 2
    assert sched.states["r2"].slot is None
    cache.check_invariants()
    sched.resolve(plan, {"r0": 1, "r1": 1})
    assert sched.schedule() is not None            # the pass that knows the tokens decides what gives
    # more requests decoding than the budget holds: the turns are taken by the pass that knows the tokens
    sched, cache = make(pages=40, page_size=4, max_requests=4, batch_tokens=3, prefill_chunk=3, max_len=32)
    for i in range(3):
        sched.add(req(i, 1, max_tokens=6))
    plan = sched.schedule()
    sched.update(plan, {e.state.request.request_id: 1 for e in plan.entries})
    sched.batch_tokens = 2
    plan = sched.schedule()                        # two of the three decode; the third one's token is known and waits its turn
    assert len(plan.entries) == 2
    sched.advance(plan)
    assert sched.lookahead(plan) is None
    sched.resolve(plan, {e.state.request.request_id: 1 for e in plan.entries})
    assert [e.state.request.request_id for e in sched.schedule().entries] == ["r2", "r0"]


def test_lookahead_leaves_out_every_request_that_finishes_by_length():
    """Three decoding requests of which the middle one and then the last reach max_tokens: the steps
    planned ahead name the rows of the sampled tokens that the survivors take."""
    sched, cache = make(pages=40, page_size=4, max_requests=4, batch_tokens=8)
    for i, limit in enumerate([9, 3, 5]):
        sched.add(req(i, 2, max_tokens=limit))
    plan = sched.schedule()
    sched.update(plan, {"r0": 7, "r1": 7, "r2": 7})
    plan = sched.schedule()
    sched.advance(plan)
    seen = []
    for _ in range(4):
        ahead = sched.lookahead(plan)
        assert ahead is not None
        seen.append(([e.state.request.request_id for e in ahead.entries], ahead.token_rows))
        sched.advance(ahead)
        sched.resolve(plan, {e.state.request.request_id: 7 for e in plan.entries})
        cache.check_invariants()
        plan = ahead
    assert seen == [(["r0", "r1", "r2"], [0, 1, 2]), (["r0", "r2"], [0, 2]), (["r0", "r2"], [0, 1]), (["r0"], [0])]
    sched.resolve(plan, {"r0": 7})
    assert sorted(sched.states) == ["r0"]


@pytest.mark.parametrize("block", range(6))
def test_random_pressure_never_blocks(block):
    """Random prompts, budgets, arrivals and pools just large enough for the longest request alone
    (so that requests are preempted and recompute): every request finishes, no step comes back
    empty while work waits.  (Two half-recomputed prompts that held all pages between them, and a
    pass that preempted a request and then had nothing left to run, used to end the loop.)"""
    for seed in range(block * 60, block * 60 + 60):
        rs = np.random.RandomState(seed)
        page = int(rs.choice([4, 8, 16]))
        n_req = int(rs.randint(2, 9))
        plens = [int(rs.randint(1, 120)) for _ in range(n_req)]
        news = [int(rs.randint(1, 40)) for _ in range(n_req)]
        longest = max(p + n for p, n in zip(plens, news))
        pages = -(-longest // page) + 1 + int(rs.randint(0, 6))
        sched, cache = make(pages=pages, page_size=page, max_requests=int(rs.randint(2, 6)),
                            batch_tokens=int(rs.choice([8, 16, 48, 200])), prefill_chunk=int(rs.choice([4, 8, 32, 128])),
                            max_len=256)
        arrive = sorted(int(rs.randint(0, 30)) for _ in range(n_req))
        nxt, step, done = 0, 0, []
        while sched.has_work() or nxt < n_req:
            while nxt < n_req and arrive[nxt] <= step:
                sched.add(req(nxt, plens[nxt], max_tokens=news[nxt], ignore_eos=True))
                nxt += 1
            if sched.has_work():
                plan = sched.schedule()
                assert plan is not None, f"seed {seed}: blocked at step {step}"
                cache.check_invariants()
                done += sched.update(plan, {e.state.request.request_id: 7 for e in plan.entries if e.sample})
            step += 1
            assert step < 20000
        cache.assert_clean()
        assert sorted(s.request.request_id for s in done) == sorted(f"r{i}" for i in range(n_req))
        assert all(s.generated == news[int(s.request.request_id[1:])] for s in done)


def test_two_recomputing_prompts_that_fill_the_pool():
    """Both running requests are in the middle of recomputing, hold every page between them and need
    one more each: the newer one gives its pages back, the older one goes on."""
    sched, cache = make(pages=14, page_size=16, max_requests=5, batch_tokens=200, prefill_chunk=128, max_len=256)   # 13 usable
    sched.add(req(0, 115, max_tokens=32, ignore_eos=True))
    sched.add(req(1, 99, max_tokens=36, ignore_eos=True))
    done = drive(sched, cache)
    assert sorted(s.request.request_id for s in done) == ["r0", "r1"]
    assert sched.stats.preemptions > 0


def test_more_decoders_than_the_token_budget_take_turns():
    """The cursor branch of decode-first: with more decoding requests than the step's token
    budget every request advances, nobody starves, and the turns differ by at most one."""
    sched, cache = make(pages=129, page_size=4, max_requests=12, batch_tokens=5, prefill_chunk=5, max_len=64)
    for i in range(12):
        sched.add(req(i, 2, max_tokens=9))
    log = []
    done = drive(sched, cache, log=log)
    assert len(done) == 12 and all(s.generated == 9 and s.finish_reason == "length" for s in done)
    decode_steps = [step for step in log if all(start > 0 and count == 1 for _, start, count, _ in step)]
    crowded = [step for step in decode_steps if len(step) == 5]
    assert len(crowded) >= 10                                   # the budget, not the request count, bounded them
    turns = {f"r{i}": 0 for i in range(12)}
    spread = 0
    for step in log:
        assert sum(c for _, _, c, _ in step) <= 5
        for rid, start, count, _ in step:
            if start > 0:
                turns[rid] += 1
        live = [turns[r] for r in turns if turns[r] < 8]       # requests that still decode
        if len(live) > 5 and min(turns.values()) > 0:
            spread = max(spread, max(live) - min(live))
    assert spread <= 2, spread                                  # round robin: nobody runs ahead of the others


def test_abort_of_waiting_and_running_requests():
    sched, cache = make(pages=33, page_size=4, max_requests=2, batch_tokens=16, prefill_chunk=16)
    for i in range(4):
        sched.add(req(i, 6, max_tokens=8))
    plan = sched.schedule()                                     # r0, r1 run; r2, r3 wait (two slots)
    assert [e.state.request.request_id for e in plan.entries] == ["r0", "r1"]
    with pytest.raises(RuntimeError):
        sched.abort("r0")                                       # inside a reserved step
    sched.update(plan, {"r0": 7, "r1": 7})
    gone = sched.abort("r3")                                    # a waiting request: no slot, no pages
    assert gone.finish_reason == "abort" and gone.slot is None and "r3" not in sched.states
    held = cache.stats()["groups"]["g"]["free"]
    gone = sched.abort("r0")                                    # a running request: its pages and slot return
    assert gone.finish_reason == "abort" and sched.result_of(gone).token_ids == [7]
    assert cache.stats()["groups"]["g"]["free"] > held and len(cache.free_slots) == 1
    assert sched.abort("r0") is None and sched.abort("nobody") is None
    cache.check_invariants()
    done = drive(sched, cache)
    assert sorted(s.request.request_id for s in done) == ["r1", "r2"]


def test_lookahead_needs_pages_and_a_plain_decode_step():
    # 6 usable pages of 4 tokens; two requests of 7 tokens: the next token of each needs no page, the one after does
    sched, cache = make(pages=7, page_size=4, max_requests=2, batch_tokens=16, prefill_chunk=16, max_len=32)
    sched.add(req(0, 7, max_tokens=12))
    sched.add(req(1, 7, max_tokens=12))
    plan = sched.schedule()
    assert not plan.decode_only and sched.lookahead(plan) is None            # not handed over yet: nothing to look past
    sched.update(plan, {"r0": 1, "r1": 1})
    plan = sched.schedule()                                                   # decode at position 7: the pages exist
    assert plan.decode_only
    sched.advance(plan)
    ahead = sched.lookahead(plan)                                             # position 8 needs a page each: 2 are free
    assert ahead is not None and [e.start for e in ahead.entries] == [8, 8]
    sched.resolve(plan, {"r0": 1, "r1": 1})
    sched.advance(ahead)
    sched.resolve(ahead, {"r0": 1, "r1": 1})
    for _ in range(2):                                                        # positions 9 and 10: no new page
        plan = sched.schedule()
        sched.update(plan, {"r0": 1, "r1": 1})
    plan = sched.schedule()                                                   # position 11 is the last of page 2
    assert plan is not None
    sched.advance(plan)
    free_before = cache.free_pages(0)
    assert free_before == 0
    assert sched.lookahead(plan) is None                                      # position 12 needs pages that are not there
    assert cache.free_pages(0) == free_before                                 # and the refusal changed nothing
    cache.check_invariants()
    sched.resolve(plan, {"r0": 1, "r1": 1})
