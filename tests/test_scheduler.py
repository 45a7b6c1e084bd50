"""The scheduler's decisions (CPU): admission, portions under a token budget, decoding, finishing,
freeing, and what happens when pages run out."""
import random

import pytest

from cbis_b200.kernels.library import host


def make(num_pages=64, page=4, max_seqs=4, budget=16, chunk=8, positions=64, window=0):
    h = host()
    cache = h.CacheManager([h.GroupSpec(page, num_pages, window)], max_seqs)
    return cache, h.Scheduler(cache, h.SchedulerLimits(max_seqs, budget, chunk, positions))


def run_to_end(cache, sch, next_token=lambda rid, k: 100 + k, max_steps=10_000):
    """Drives the scheduler with made-up sampled tokens; returns {id: (reason, output)} and the plans."""
    done, plans, count = {}, [], {}
    for _ in range(max_steps):
        if sch.idle():
            break
        plan = sch.schedule()
        assert plan, "a step must run something while requests are left"
        assert cache.check() == ""
        plans.append([(p.request_id, p.start, list(p.tokens), p.sample) for p in plan])
        sampled = []
        for p in plan:
            if p.sample:
                k = count.get(p.request_id, 0)
                assert p.output_index == k
                count[p.request_id] = k + 1
                sampled.append((p.request_id, next_token(p.request_id, k)))
        for f in sch.update(sampled):
            done[f.request_id] = (f.reason, list(f.output))
    assert sch.idle()
    return done, plans


def test_prompt_is_cut_into_portions_beside_decoding_requests():
    cache, sch = make(budget=16, chunk=8)
    sch.add(0, list(range(5)), 3)
    plan = sch.schedule()
    assert [(p.request_id, p.start, p.tokens, p.sample) for p in plan] == [(0, 0, [0, 1, 2, 3, 4], True)]
    sch.update([(0, 50)])
    sch.add(1, list(range(20)), 2)
    plan = sch.schedule()                                   # decode token first, then a portion of the new prompt
    assert [(p.request_id, p.start, len(p.tokens), p.sample) for p in plan] == [(0, 5, 1, True), (1, 0, 8, False)]
    assert plan[0].tokens == [50]
    sch.update([(0, 51)])
    plan = sch.schedule()
    assert [(p.request_id, p.start, len(p.tokens), p.sample) for p in plan] == [(0, 6, 1, True), (1, 8, 8, False)]
    done = sch.update([(0, 52)])
    assert [(f.request_id, f.reason, f.output) for f in done] == [(0, "length", [50, 51, 52])]
    plan = sch.schedule()
    assert [(p.request_id, p.start, len(p.tokens), p.sample) for p in plan] == [(1, 16, 4, True)]
    assert cache.free_slots() == 3


def test_update_with_the_plan_pairs_the_tokens_with_the_sampling_entries():
    cache, sch = make(budget=16, chunk=8)
    sch.add(0, list(range(5)), 2)
    sch.add(1, list(range(20)), 2)
    plan = sch.schedule()                                   # request 0 whole (samples), a portion of request 1 (does not)
    assert [(p.request_id, p.sample) for p in plan] == [(0, True), (1, False)]
    with pytest.raises(ValueError, match="fewer tokens"):
        sch.update_plan(plan, [])
    with pytest.raises(ValueError, match="more tokens"):
        sch.update_plan(plan, [50, 51])
    assert sch.update_plan(plan, [50]) == []
    plan = sch.schedule()
    assert [(p.request_id, p.start, len(p.tokens), p.sample) for p in plan] == [(0, 5, 1, True), (1, 8, 8, False)]
    assert plan[0].tokens == [50]
    done = sch.update_plan(plan, [51])
    assert [(f.request_id, f.reason, f.output) for f in done] == [(0, "length", [50, 51])]


def test_budget_bounds_every_step_and_all_finish():
    cache, sch = make(budget=10, chunk=6, max_seqs=3)
    lens = [1, 7, 23, 40, 13]
    for i, n in enumerate(lens):
        sch.add(i, [i] * n, 5)
    done, plans = run_to_end(cache, sch)
    assert set(done) == set(range(5)) and all(r == "length" and len(o) == 5 for r, o in done.values())
    for plan in plans:
        assert sum(len(t) for _, _, t, _ in plan) <= 10 and len(plan) <= 3
        assert all(len(t) <= 6 for _, _, t, _ in plan)
    # every request's tokens were run exactly once, in order, prompt then its outputs but the last
    for i, n in enumerate(lens):
        fed = [t for plan in plans for rid, _, toks, _ in plan if rid == i for t in toks]
        assert fed == [i] * n + [100, 101, 102, 103]
    assert cache.free_pages(0) == 64 and cache.free_slots() == 3


def test_fifo_admission_and_slot_limit():
    cache, sch = make(max_seqs=2, budget=64, chunk=64)
    for i in range(4):
        sch.add(i, [1, 2, 3], 2)
    plan = sch.schedule()
    assert [p.request_id for p in plan] == [0, 1] and sch.num_waiting() == 2
    sch.update([(0, 9), (1, 9)])
    sch.schedule()
    sch.update([(0, 9), (1, 9)])                            # both finish
    assert [p.request_id for p in sch.schedule()] == [2, 3]


def test_eos_and_position_limit():
    cache, sch = make(positions=8, budget=16, chunk=16)
    sch.add(0, [1, 2, 3], 10, 7, False)
    sch.add(1, [1, 2, 3], 10, 7, True)
    sch.add(2, [1, 2, 3, 4, 5, 6], 10)
    done, _ = run_to_end(cache, sch, next_token=lambda rid, k: 7 if k == 1 else 5)
    assert done[0] == ("stop", [5, 7])
    assert done[1][0] == "length" and len(done[1][1]) == 6   # 3 + 6 = 9 tokens > 8 positions: the 6th cannot be fed
    assert done[2] == ("length", [5, 7, 5])                  # fed 6,7,8 tokens; the third output has no position left


def test_refusals_at_add():
    cache, sch = make(num_pages=4, page=4, positions=32)
    with pytest.raises(ValueError, match="empty prompt"):
        sch.add(0, [], 4)
    with pytest.raises(ValueError, match="exceeds the model's 32 positions"):
        sch.add(1, [0] * 33, 1)
    with pytest.raises(ValueError, match="can never fit"):
        sch.add(2, [0] * 10, 8)                              # 17 tokens need 5 pages of 4
    sch.add(3, [0] * 10, 7)                                  # 16 tokens: fits exactly
    with pytest.raises(ValueError, match="exists already"):
        sch.add(3, [0], 1)


def test_pages_run_out_newest_is_preempted_and_recomputed():
    cache, sch = make(num_pages=6, page=4, max_seqs=3, budget=32, chunk=32)
    sch.add(0, [10] * 7, 9)                                  # grows to 15 tokens: 4 pages
    sch.add(1, [11] * 7, 9)
    plan = sch.schedule()
    assert [p.request_id for p in plan] == [0, 1] and cache.free_pages(0) == 2
    sch.update([(0, 100), (1, 100)])
    history = {0: [], 1: []}
    preempted_seen = False
    for step in range(200):
        if sch.idle():
            break
        plan = sch.schedule()
        assert plan and cache.check() == ""
        sampled = []
        for p in plan:
            history[p.request_id].append((p.start, list(p.tokens)))
            if p.request_id == 1 and p.start == 0 and len(p.tokens) > 7:
                preempted_seen = True                         # recomputed: prompt and its outputs so far in one portion
                assert p.tokens[:7] == [11] * 7 and p.tokens[7:] == [100 + k for k in range(len(p.tokens) - 7)]
            if p.sample:
                sampled.append((p.request_id, 100 + p.output_index))
        sch.update(sampled)
    assert sch.idle() and sch.preemptions() >= 1 and preempted_seen
    # the older request was never disturbed: it ran each position exactly once
    starts0 = [s for s, _ in history[0]]
    assert starts0 == sorted(set(starts0))
    assert cache.free_pages(0) == 6 and cache.free_slots() == 3


def test_admission_by_what_fits_now_is_settled_by_preemption_later():
    cache, sch = make(num_pages=4, page=4, max_seqs=2, budget=32, chunk=32)
    sch.add(0, [1] * 8, 5)                                   # 12 tokens at most: 3 pages
    sch.add(1, [2] * 8, 5)
    done, plans = run_to_end(cache, sch)
    assert [rid for rid, _, _, _ in plans[0]] == [0, 1]      # both prompts fit now (2 pages each) ...
    # ... but not both at 3 pages: the newer one yields
    assert set(done) == {0, 1} and sch.preemptions() >= 1
    assert all(len(o) == 5 for _, o in done.values())
    starts0 = [st for plan in plans for rid, st, _, _ in plan if rid == 0]
    assert starts0 == sorted(set(starts0))                   # the older request never started over


def test_a_preempted_request_is_recomputed_once_not_every_few_steps():
    """The pages a preempted request gives up would let its first portion in again at once; it would then be
    recomputed and thrown out again whenever the older request crosses a page.  It comes back only when all it
    holds so far and a page more fit, and never in the step that threw it out."""
    cache, sch = make(num_pages=7, page=4, max_seqs=2, budget=32, chunk=32)
    sch.add(0, [1] * 8, 18)                                  # grows to 25 tokens: all 7 pages
    sch.add(1, [2] * 8, 18)
    done, plans = run_to_end(cache, sch)
    assert set(done) == {0, 1} and all(len(o) == 18 for _, o in done.values())
    restarts = [len(t) for plan in plans for rid, st, t, _ in plan if rid == 1 and st == 0]
    assert sch.preemptions() == 1 and len(restarts) == 2     # its first run and ONE recomputation
    for a, b in zip(plans, plans[1:]):                       # the step that preempts it does not hold it
        if any(rid == 1 for rid, *_ in a) and not any(rid == 1 for rid, *_ in b):
            assert [rid for rid, *_ in b] == [0]
    starts0 = [st for plan in plans for rid, st, _, _ in plan if rid == 0]
    assert starts0 == sorted(set(starts0))


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_with_books_kept(seed):
    rng = random.Random(seed)
    window = rng.choice([0, 0, 12])
    cache, sch = make(num_pages=rng.randint(12, 30), page=rng.choice([2, 4, 8]), max_seqs=rng.randint(1, 5),
                      budget=rng.randint(4, 24), chunk=rng.randint(2, 16), positions=48, window=window)
    want = {}
    rid = 0
    done = {}
    fed = {}
    for step in range(3000):
        if rid < 25 and rng.random() < 0.3:
            n, g = rng.randint(1, 30), rng.randint(1, 12)
            try:
                sch.add(rid, [rid] * n, g)
                want[rid] = min(g, 48 - n + 1)
            except ValueError:
                pass
            rid += 1
        if sch.idle():
            if rid >= 25:
                break
            continue
        plan = sch.schedule()
        assert plan and cache.check() == ""
        sampled = []
        for p in plan:
            if p.start == 0:
                fed[p.request_id] = []                        # (re)computed from the start
            assert p.start == len(fed[p.request_id])
            fed[p.request_id] += list(p.tokens)
            if p.sample:
                sampled.append((p.request_id, 1000 + p.output_index))
        for f in sch.update(sampled):
            done[f.request_id] = list(f.output)
    assert sch.idle() and set(done) == set(want)
    for r, out in done.items():
        assert out == [1000 + k for k in range(want[r])]
    assert cache.free_pages(0) == cache.num_pages(0) and cache.check() == ""


# ---- the step after a launched one, planned before its tokens are known -------------------------------------

def drive(cache, sch, arrivals, token, ahead):
    """Runs the scheduler as the engine does.  ``arrivals``: {step: [(id, prompt, max_new, eos)]}; ``token(id, k)``
    is request id's k-th output.  With ``ahead`` the next step is planned (schedule_ahead) before the tokens of the
    running one are given back.  Returns ({id: (reason, output)}, the rows run per step as (id, start, count),
    how many steps were planned ahead)."""
    done, steps, n_ahead, in_flight = {}, [], 0, None

    def rows(plan):
        return [(p.request_id, p.start, len(p.tokens)) for p in plan]

    def tokens(plan):
        return [token(p.request_id, p.output_index) for p in plan if p.sample]

    for step in range(5000):
        for a in arrivals.get(step, []):
            sch.add(*a)
        cur, in_flight = in_flight, None
        if cur is None:
            if sch.idle():
                if step > max(arrivals, default=0):
                    break
                continue
            cur = sch.schedule()
            assert cur and cache.check() == ""
            steps.append(rows(cur))
            if not any(p.sample for p in cur):
                continue
        if ahead:
            nxt = sch.schedule_ahead()
            assert cache.check() == ""
            if nxt:
                assert all(p.ahead and p.sample and p.tokens == [0] for p in nxt)
                sampling = [p.request_id for p in cur if p.sample]
                assert [sampling[p.source] for p in nxt] == [p.request_id for p in nxt]
                assert sch.ahead_sources() == ([] if [p.source for p in nxt] == list(range(len(nxt))) else [p.source for p in nxt])
                in_flight = nxt
                steps.append(rows(nxt))
                n_ahead += 1
        for f in sch.update_plan(cur, tokens(cur)):
            done[f.request_id] = (f.reason, list(f.output))
        if in_flight is not None and sch.idle():
            assert sch.update_plan(in_flight, tokens(in_flight)) == []
            in_flight = None
    assert sch.idle() and in_flight is None
    assert cache.free_pages(0) == cache.num_pages(0) and cache.check() == ""
    return done, steps, n_ahead


def test_steps_planned_ahead_are_the_steps_planned_in_turn():
    """Without end-of-sequence tokens every step planned ahead is, row for row, the step that schedule() plans
    after the update; with them the requests end with the same outputs, and a request that ended while its row of
    the next step was on its way is passed over when that step's tokens come back."""
    arrivals = {0: [(0, [1, 2, 3, 4, 5], 9, -1, False), (1, list(range(11)), 4, -1, False), (2, [7] * 6, 12, -1, False)]}
    tok = lambda rid, k: 100 * rid + k
    want, steps_sync, n0 = drive(*make(budget=16, chunk=8), arrivals, tok, ahead=False)
    got, steps_ahead, n1 = drive(*make(budget=16, chunk=8), arrivals, tok, ahead=True)
    assert n0 == 0 and n1 > 8
    assert got == want and steps_ahead == steps_sync
    # a request that arrives while a step planned ahead is on its way is admitted a step later, and ends the same
    later = dict(arrivals)
    later[4] = [(3, [9, 9, 9], 5, -1, False)]
    want, steps_sync, _ = drive(*make(budget=16, chunk=8), later, tok, ahead=False)
    got, steps_ahead, _ = drive(*make(budget=16, chunk=8), later, tok, ahead=True)
    assert got == want and got[3] == ("length", [300 + k for k in range(5)])
    first = lambda steps: min(i for i, st in enumerate(steps) if any(r[0] == 3 for r in st))
    assert first(steps_ahead) == first(steps_sync) + 1
    # request 0 stops at its third output, request 2 at its sixth: their rows of the steps planned ahead are for nothing
    eos = {0: [(0, [1, 2, 3, 4, 5], 9, 2, False), (1, list(range(11)), 14, -1, False)], 3: [(2, [7] * 6, 12, 205, False)]}
    want, steps_sync, _ = drive(*make(budget=16, chunk=8), eos, tok, ahead=False)
    got, steps_ahead, n1 = drive(*make(budget=16, chunk=8), eos, tok, ahead=True)
    assert want[0] == ("stop", [0, 1, 2]) and want[2] == ("stop", [200 + k for k in range(6)])
    assert got == want and n1 > 5
    in_turn = {r for s in steps_sync for r in s}
    extra = [r for s in steps_ahead for r in s if r not in in_turn]
    assert extra == [(0, 7, 1), (2, 11, 1)]              # the end-of-sequence token fed once, for nothing, each


def test_what_cannot_be_planned_ahead():
    cache, sch = make(num_pages=6, page=4, max_seqs=2, budget=16, chunk=8, positions=64)
    assert sch.schedule_ahead() == []                       # nothing runs
    sch.add(0, [1, 2, 3], 3)
    sch.add(1, list(range(12)), 6)
    plan = sch.schedule()                                   # request 0 whole, 8 tokens of request 1
    assert [(p.request_id, p.sample) for p in plan] == [(0, True), (1, False)]
    assert sch.schedule_ahead() == []                       # request 1 still has tokens to feed
    with pytest.raises(RuntimeError, match="have not come back"):
        sch.schedule()
    sch.update_plan(plan, [50])
    plan = sch.schedule()                                   # both sample now
    assert [(p.request_id, p.start, len(p.tokens), p.sample) for p in plan] == [(0, 3, 1, True), (1, 8, 4, True)]
    ahead = sch.schedule_ahead()
    assert [(p.request_id, p.start, p.tokens, p.output_index, p.ahead) for p in ahead] == [(0, 4, [0], 2, True), (1, 12, [0], 1, True)]
    assert sch.schedule_ahead() == []                       # one step ahead, not two
    sch.update_plan(plan, [51, 60])
    assert sch.schedule_ahead() == []                       # request 0's third output is its last: the step after holds one row less
    done = sch.update_plan(ahead, [52, 61])
    assert [(f.request_id, f.output) for f in done] == [(0, [50, 51, 52])]
    plan = sch.schedule()
    assert [(p.request_id, p.start, p.tokens) for p in plan] == [(1, 13, [61])]
    sch.add(2, [5, 5], 4)
    assert sch.schedule_ahead() == []                       # somebody waits for admission
    sch.update_plan(plan, [62])
    plan = sch.schedule()
    assert [(p.request_id, p.start) for p in plan] == [(1, 14), (2, 0)]
    # pages: request 1 holds 4 pages (15 tokens), request 2 one; the pool has 6; one more token for request 1 needs a fifth
    ahead = sch.schedule_ahead()
    assert [(p.request_id, p.start) for p in ahead] == [(1, 15), (2, 2)] and cache.free_pages(0) == 1
    sch.update_plan(plan, [63, 70])
    nxt = sch.schedule_ahead()                              # request 1 at 16 tokens takes the last page
    assert [(p.request_id, p.start) for p in nxt] == [(1, 16), (2, 3)] and cache.free_pages(0) == 0
    sch.update_plan(ahead, [64, 71])
    assert sch.schedule_ahead() == []                       # request 1's sixth output, its last, is on its way
    done = sch.update_plan(nxt, [65, 72])
    assert [(f.request_id, f.output) for f in done] == [(1, [60, 61, 62, 63, 64, 65])]
    assert cache.check() == "" and cache.free_pages(0) == 5      # request 2 keeps its one page


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_planned_ahead_end_like_those_planned_in_turn(seed):
    rng = random.Random(100 + seed)
    window = rng.choice([0, 0, 12])
    kw = dict(num_pages=rng.randint(12, 30), page=rng.choice([2, 4, 8]), max_seqs=rng.randint(1, 5),
              budget=rng.randint(4, 24), chunk=rng.randint(2, 16), positions=48, window=window)
    arrivals, rid = {}, 0
    for step in range(120):
        if rng.random() < 0.25:
            n, g = rng.randint(1, 30), rng.randint(1, 12)
            eos = rng.choice([-1, -1, 7])
            probe_cache, probe = make(**kw)
            try:
                probe.add(rid, [rid] * n, g, eos, False)
            except ValueError:
                continue                                     # can never fit: refused at add
            arrivals.setdefault(step, []).append((rid, [rid] * n, g, eos, False))
            rid += 1
    tok = lambda r, k: 7 if (r * 31 + k * 17) % 11 == 0 else 1000 + k
    want, _, _ = drive(*make(**kw), arrivals, tok, ahead=False)
    got, _, n_ahead = drive(*make(**kw), arrivals, tok, ahead=True)
    assert got == want and len(want) == rid
    assert n_ahead > 0 or rid == 0
