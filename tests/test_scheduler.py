"""The scheduler's decisions, with a stand-in for the step function (no GPU)."""
import random

import pytest

from lite_lang_b200.cache import CacheManager, PagedGroupSpec
from lite_lang_b200.engine.scheduler import (STRATEGIES, Request, Scheduler, peak_token_estimate)
from lite_lang_b200.sampling import SamplingParams


def make(num_pages=16, page_size=4, max_requests=4, max_len=64, budget=8, strategy="LIFOStrategy", window=None):
    m = CacheManager([PagedGroupSpec(1, 16, window, 1)], [num_pages], page_size, max_requests, max_len)
    return m, Scheduler(m, budget, max_reqs=100, busy_scale=0.6, strategy=strategy)


def req(i, n_prompt, max_new, eos=()):
    return Request(i, list(range(1, n_prompt + 1)), SamplingParams(), max_new, tuple(eos))


def run_step(m, s, token=7):
    """What the engine does around a step: run the plan, advance the cache, commit."""
    plan = s.plan()
    for p in plan:
        assert p.request.slot is not None and p.count >= 1
        m.advance(p.request.slot, m.length(p.request.slot) + p.count)
    done = s.commit(plan, [token if p.samples else None for p in plan])
    m.check_invariants()
    return plan, done


def test_prompts_are_cut_under_the_token_budget():
    m, s = make(budget=8)
    a = req(0, 19, 2)
    s.add(a)
    counts = []
    while s.has_work():
        plan, _ = run_step(m, s)
        counts.append([(p.request.id, p.start, p.count, p.samples) for p in plan])
    assert counts[0] == [(0, 0, 8, False)]
    assert counts[1] == [(0, 8, 8, False)]
    assert counts[2] == [(0, 16, 3, True)]        # the last portion gives the first new token
    assert counts[3] == [(0, 19, 1, True)]        # then one token a step
    assert a.output == [7, 7] and a.finish_reason == "length"
    assert m.num_free_pages() == 16


def test_decode_tokens_come_first_and_share_the_step_with_portions():
    m, s = make(budget=8)
    a, b = req(0, 3, 5), req(1, 20, 2)
    s.add(a)
    run_step(m, s)                 # a prefilled, first token
    s.add(b)
    plan, _ = run_step(m, s)
    assert [(p.request.id, p.count) for p in plan] == [(0, 1), (1, 7)]   # 1 + 7 = budget
    plan, _ = run_step(m, s)
    assert [(p.request.id, p.count) for p in plan] == [(0, 1), (1, 7)]
    plan, _ = run_step(m, s)
    assert [(p.request.id, p.count, p.samples) for p in plan] == [(0, 1, True), (1, 6, True)]


def test_finish_rules():
    m, s = make(budget=16)
    a, b, c = req(0, 3, 10, eos=(7,)), req(1, 3, 10, eos=(9,)), req(2, 3, 2)
    a.params = SamplingParams(ignore_eos=False)
    b.params = SamplingParams()
    for r in (a, b, c):
        s.add(r)
    _, done = run_step(m, s, token=7)
    assert [r.id for r in done] == [0] and a.finish_reason == "eos"
    _, done = run_step(m, s, token=7)
    assert [r.id for r in done] == [2] and c.finish_reason == "length"
    assert b.status == "running"
    d = req(3, 3, 10, eos=(7,))
    d.params = SamplingParams(ignore_eos=True)
    s.add(d)
    run_step(m, s, token=7)
    assert d.status == "running" and d.output == [7]


def test_model_length_ends_a_request():
    m, s = make(max_len=8, num_pages=16)
    a = req(0, 5, 100)
    s.add(a)
    while s.has_work():
        run_step(m, s)
    assert a.finish_reason == "model_len" and a.length == 8
    b = req(1, 8, 4)        # prompt + 1 > max_model_len
    s.add(b)
    assert b.finish_reason == "too_long" and not s.has_work()


def _anchors():
    import json
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "scheduler_anchors.json")
    with open(path) as fh:
        return json.load(fh)


def test_peak_estimate_equals_the_references_answers():
    """``peak_token_estimate`` on the rows (tokens held, tokens expected) that the reference built gives the
    reference's own answer (``ReadyQue._can_add_new_req``, litelang/scheduler/req_queue.py:219-232) in every
    stored case; the file was made by tests/golden/make_scheduler_anchors.py from the reference's code."""
    cases = _anchors()["admission"]
    assert len(cases) >= 100 and 0 < sum(c["admitted"] for c in cases) < len(cases)
    for c in cases:
        assert (peak_token_estimate([tuple(r) for r in c["rows"]]) <= c["pool"]) == c["admitted"], c
    assert peak_token_estimate([]) == 0


def test_admission_equals_the_references_on_its_own_inputs():
    """The scheduler's own rows and its decision, on the stored inputs.  For requests that have produced
    nothing yet the rows are the reference's (``Req.need_tokens``, req_queue.py:59-66) and so is the decision.
    For a request that has produced n tokens the reference keeps expecting its whole guess on top of what the
    request holds; this scheduler expects the guess less n, the only difference, so its row is the
    reference's with n taken off (never below zero)."""
    for c in _anchors()["admission"]:
        m = CacheManager([PagedGroupSpec(1, 16, None, 1)], [c["pool"]], 1, 16, 10 ** 6)
        s = Scheduler(m, 64, max_reqs=100, busy_scale=0.6)
        reqs = []
        for i, (n_in, n_out, max_out) in enumerate(c["requests"]):
            r = req(i, n_in, max_out)
            r.output = [1] * n_out
            reqs.append(r)
        s.running = reqs[:-1]
        s._is_busy = lambda busy=c["busy"]: busy
        rows = [(r.length, s._expected_new(r, c["busy"])) for r in reqs]
        want = [(held, max(0, expected - n_out)) for (held, expected), (_, n_out, _) in zip(c["rows"], c["requests"])]
        assert rows == want, c
        if all(n_out == 0 for _, n_out, _ in c["requests"]):
            assert s._fits(reqs[-1]) == c["admitted"], c
        else:
            assert s._fits(reqs[-1]) == (peak_token_estimate(want) <= c["pool"])
            assert s._fits(reqs[-1]) or not c["admitted"]      # whoever the reference admits is admitted here


def test_busy_is_the_references_threshold():
    # litelang/scheduler/req_queue.py:194,213-217: tokens held by running and preempted requests > pool * busy_scale
    m, s = make(num_pages=25, page_size=4, budget=8)          # 100 tokens, threshold 60
    a, b = req(0, 30, 5), req(1, 30, 5)
    s.running = [a]
    b.preemptions = 1
    s.waiting.append(b)
    assert not s._is_busy()                                   # 60 is not more than 60
    a.output = [1]
    assert s._is_busy()


def test_strategies_order_as_the_references_do():
    """The four orders in which requests leave (litelang/scheduler/pause_strategy.py:18-39), on the stored
    inputs.  The reference's LongestFirstStrategy sorts by length ascending and its ShortestFirstStrategy
    descending; here the same two orders carry names that say what they do.  The requests the reference takes
    out (``select_swapped_reqs``, :42-55) are the first of that order until more than the missing tokens are
    covered; this scheduler lets them leave one at a time, in the same order, until the pages suffice."""
    names = {"FIFOStrategy": "FIFOStrategy", "LIFOStrategy": "LIFOStrategy",
             "LongestFirstStrategy": "ShortestLeavesFirstStrategy", "ShortestFirstStrategy": "LongestLeavesFirstStrategy"}
    cases = _anchors()["preemption"]
    assert len(cases) >= 100
    for c in cases:
        reqs = []
        for i, n in enumerate(c["lengths"]):
            r = req(i, n, 10)
            r.arrival = i
            reqs.append(r)
        for ref_name, ours in names.items():
            order = [r.id for r in STRATEGIES[ours](list(reqs))]
            assert order == c["strategies"][ref_name]["order"], (ref_name, c)
            out = c["strategies"][ref_name]["out"]
            assert order[:len(out)] == out
            # one at a time until the missing tokens are covered: the same requests, or one fewer where the
            # reference's "more than" takes one more than is needed
            freed, k = 0, 0
            while freed < c["need"] and k < len(order):
                freed += c["lengths"][order[k]]
                k += 1
            assert k in (len(out), len(out) - 1), (ref_name, c)


def test_admission_waits_for_room_in_the_estimate():
    m, s = make(num_pages=8, page_size=4, budget=32)      # 32 tokens of cache
    a, b = req(0, 8, 10), req(1, 8, 10)
    s.add(a)
    s.add(b)
    plan, _ = run_step(m, s)
    # alone a always runs; with a running, b's estimate: not busy -> 6 expected each:
    # sorted equal: cumsum 8,16 ; 8+6*1=14, 16+6*2=28 <= 32 -> admitted in the same step
    assert [p.request.id for p in plan] == [0, 1]
    c = req(2, 8, 10)
    s.add(c)
    plan, _ = run_step(m, s)
    assert 2 not in [p.request.id for p in plan]           # 3 requests would peak above 32
    assert s.waiting[0] is c


def test_out_of_pages_at_decode_preempts_the_latest_arrival():
    m, s = make(num_pages=4, page_size=4, budget=16, strategy="LIFOStrategy")
    a, b = req(0, 7, 6), req(1, 7, 6)
    s.add(a)
    run_step(m, s)
    # force b in although the estimate would refuse it: admit by hand
    slot = m.open()
    b.slot, b.status, b.arrival = slot, "running", 5
    assert m.reserve(slot, 7)
    m.advance(slot, 7)
    b.computed, b.output = 7, [7]
    b.prompt = list(range(1, 8))
    s.running.append(b)
    assert m.num_free_pages() == 0
    a.computed, b.computed = a.length - 1, b.length - 1
    # both sit at 8 tokens after this step; the step after needs a third page for each
    run_step(m, s)
    plan, _ = run_step(m, s)
    assert [p.request.id for p in plan] == [0]             # b (latest) left, a went on
    assert b.status == "waiting" and b.slot is None and b.computed == 0 and b.preemptions == 1
    assert s.waiting[0] is b                               # at the front of the queue
    assert s.counters["preemptions"] == 1
    kept = list(b.output)
    # b comes back later and is recomputed from prompt + produced tokens, producing nothing twice
    while s.has_work():
        run_step(m, s)
    assert b.output[:len(kept)] == kept and len(b.output) == 6 and len(a.output) == 6
    assert a.finish_reason == b.finish_reason == "length"
    assert m.num_free_pages() == 4


def test_a_request_that_cannot_fit_alone_ends_with_cache_full():
    m, s = make(num_pages=2, page_size=4, budget=16, max_len=64)
    a = req(0, 6, 50)
    s.add(a)
    while s.has_work():
        run_step(m, s)
    assert a.finish_reason == "cache_full" and a.length == 9      # 8 cached tokens and the one drawn from them
    assert m.num_free_pages() == 2 and m.num_free_slots == 4
    b = req(1, 12, 5)           # the prompt alone needs 3 pages
    s.add(b)
    while s.has_work():
        run_step(m, s)
    assert b.finish_reason == "cache_full" and b.output == []


def test_portion_shrinks_to_the_free_pages():
    m, s = make(num_pages=4, page_size=4, budget=64)
    a = req(0, 6, 30)
    s.add(a)
    run_step(m, s)                         # a holds 2 pages
    b = req(1, 14, 2)
    s.add(b)
    s._fits = lambda cand: True            # take the estimate out of the picture
    plan, _ = run_step(m, s)
    got = {p.request.id: p.count for p in plan}
    assert got[1] == 8                     # two free pages -> 8 tokens of b's 14
    assert m.num_free_pages() == 0


def test_strategies_order_as_their_names_say():
    rs = [req(0, 5, 1), req(1, 9, 1), req(2, 2, 1)]
    for i, r in enumerate(rs):
        r.arrival = i
    assert [r.id for r in STRATEGIES["FIFOStrategy"](rs)] == [0, 1, 2]
    assert [r.id for r in STRATEGIES["LIFOStrategy"](rs)] == [2, 1, 0]
    assert [r.id for r in STRATEGIES["ShortestLeavesFirstStrategy"](rs)] == [2, 0, 1]
    assert [r.id for r in STRATEGIES["LongestLeavesFirstStrategy"](rs)] == [1, 0, 2]
    with pytest.raises(ValueError):
        make(strategy="NoSuchStrategy")


def test_waiting_queue_is_bounded():
    m, s = make()
    s.max_reqs = 2
    assert s.add(req(0, 3, 1)) and s.add(req(1, 3, 1))
    assert not s.add(req(2, 3, 1))


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("strategy", sorted(STRATEGIES))
def test_random_load_always_drains(seed, strategy):
    rng = random.Random(seed)
    m, s = make(num_pages=rng.randint(3, 10), page_size=4, max_requests=3, max_len=48,
                budget=rng.choice([2, 5, 16]), strategy=strategy, window=rng.choice([None, 6]))
    reqs = [req(i, rng.randint(1, 20), rng.randint(1, 12)) for i in range(10)]
    pending = list(reqs)
    steps = 0
    while pending or s.has_work():
        if pending and rng.random() < 0.4:
            s.add(pending.pop(0))
        if s.has_work():
            plan, _ = run_step(m, s, token=rng.randint(0, 50))
            assert sum(p.count for p in plan) <= s.budget
            assert len({p.request.id for p in plan}) == len(plan)
        steps += 1
        assert steps < 5000, "the scheduler does not make progress"
    for r in reqs:
        assert r.status == "finished" and r.slot is None
        assert r.finish_reason in ("length", "cache_full", "model_len")
        if r.finish_reason == "length":
            assert len(r.output) == r.max_new_tokens
    assert m.num_free_pages() == m.total_pages() and m.num_free_slots == 3


# ---------------------------------------------------------------- the step after the running one
def _decode_state(n=3, max_new=(6, 6, 6), eos=((), (), ())):
    m, s = make(num_pages=32, budget=8)
    reqs = [req(i, 3 + i, max_new[i], eos[i]) for i in range(n)]
    for r in reqs:
        s.add(r)
    run_step(m, s)                      # prompts; everyone has a first token
    return m, s, reqs


def test_plan_ahead_decides_a_decode_step_without_the_tokens():
    m, s, reqs = _decode_state()
    plan = s.plan()
    ahead = s.plan_ahead(plan)
    assert [(p.request.id, p.start, p.count, p.samples, p.feed) for p in ahead] == \
        [(r.id, r.length, 1, True, k) for k, r in enumerate(reqs)]
    # what the engine does: both steps advance the cache when launched, commits follow in order
    for pl in (plan, ahead):
        for p in pl:
            m.advance(p.request.slot, m.length(p.request.slot) + p.count)
    s.commit(plan, [7] * 3)
    s.commit(ahead, [8] * 3)
    assert all(r.output[-2:] == [7, 8] and r.computed == r.length - 1 for r in reqs)
    m.check_invariants()


def test_plan_ahead_leaves_out_who_ends_by_length_and_commit_ignores_who_ended_by_token():
    m, s, reqs = _decode_state(max_new=(2, 6, 6), eos=((), (9,), ()))
    plan = s.plan()                     # request 0 reaches its 2 tokens with this step
    ahead = s.plan_ahead(plan)
    assert [p.request.id for p in ahead] == [1, 2] and [p.feed for p in ahead] == [1, 2]
    for pl in (plan, ahead):
        for p in pl:
            m.advance(p.request.slot, m.length(p.request.slot) + p.count)
    done = s.commit(plan, [7, 9, 7])    # request 1 draws its eos id
    assert {r.id for r in done} == {0, 1} and reqs[1].finish_reason == "eos"
    done = s.commit(ahead, [5, 5])      # the token that was computed ahead for request 1 is dropped
    assert done == [] and reqs[1].output == [7, 9] and reqs[2].output[-2:] == [7, 5]
    m.check_invariants()
    assert s.plan_ahead(ahead) is not None      # request 2 alone goes on
    s2 = s.plan_ahead([p for p in ahead])       # (asking twice reserves nothing twice)
    assert s2 is not None
    m.check_invariants()


def test_plan_ahead_declines_when_the_outcome_matters():
    m, s, reqs = _decode_state()
    s.add(req(9, 4, 2))                 # someone waits: the next step may admit it
    assert s.plan_ahead(s.plan()) is None
    m, s, reqs = _decode_state()
    plan = s.plan()
    assert s.plan_ahead(plan[:2]) is None       # not every running request is in the step
    # no page left for one more token: the usual path decides who leaves
    m, s = make(num_pages=2, page_size=4, budget=8)
    a = req(0, 7, 5)
    s.add(a)
    run_step(m, s)                      # 7 prompt tokens: pages full after one more token
    plan = s.plan()
    assert plan and s.plan_ahead(plan) is None


def test_prefill_attention_plan_fits_the_ctas_to_the_sms():
    """The host's plan for the tcgen05 prefill attention: splits of the smallest length for which all CTAs of the
    step run at once; nothing is cut when that would not shorten the longest chain by a fifth, or when the
    uncut row blocks already exceed the slots."""
    from lite_lang_b200 import ops

    def ctas(entries, group, nkv, split_len, nsplit):
        tpb, total = 128 // group, 0
        for ctx, q in entries:
            for first in range(0, q, tpb):
                n = (ctx + min(first + tpb, q) - 1) // 64 + 1
                eff = min(nsplit, max(1, -(-n // split_len)))
                per = -(-n // eff)
                total += -(-n // per)                       # what the kernel makes of it
        return total * nkv

    blocks, nsplit, split_len = ops.attn_prefill_tc_plan([(0, 2048)], 6, None, 2, 296)
    assert (blocks, nsplit, split_len) == (98, 2, 16)
    assert ctas([(0, 2048)], 6, 2, split_len, nsplit) <= 296 < ctas([(0, 2048)], 6, 2, split_len - 1, 8)
    assert ops.attn_prefill_tc_plan([(1536, 512)] * 4, 6, None, 2, 296)[1] == 1        # equal chains: no cut
    assert ops.attn_prefill_tc_plan([(0, 8192)], 6, None, 2, 296)[1] == 1              # more row blocks than slots
    b, n, s = ops.attn_prefill_tc_plan([(7680, 512)], 6, None, 2, 296)                 # few row blocks, long context
    assert n == 8 and ctas([(7680, 512)], 6, 2, s, n) <= 296
    assert ops.attn_prefill_tc_plan([], 6, None, 2, 296) == (0, 1, 1 << 20)
    # a window shortens the chains
    assert ops.attn_prefill_tc_plan([(4096, 64)], 4, 256, 2, 296)[2] >= 4


def test_a_portion_shrinks_to_what_every_cache_group_can_take():
    """Two groups, the windowed one with few pages: a long prompt runs in portions that the smaller pool
    can hold, the window's pages come back after every step, and the prompt gets through."""
    groups = [PagedGroupSpec(1, 16, None, 1), PagedGroupSpec(1, 16, 8, 1)]
    m = CacheManager(groups, [16, 5], 4, 4, 64)
    s = Scheduler(m, 32, max_reqs=100, busy_scale=0.6)
    assert s.capacity_tokens == 64
    a = req(0, 50, 3)
    s.add(a)
    counts = []
    while s.has_work():
        plan, _ = run_step(m, s)
        counts.append([p.count for p in plan])
        assert len(counts) < 40
    assert counts[0] == [20]                      # the windowed group's 5 pages, not the budget of 32
    assert sum(c[0] for c in counts[:-2]) == 50 and a.finish_reason == "length" and len(a.output) == 3
    assert m.num_free_pages(0) == 16 and m.num_free_pages(1) == 5


def test_decode_attention_plan_follows_requests_and_context():
    """The host's plan of the decode attention (CPU: arithmetic only): CTAs for about 7/8 of the SMs, as splits of a
    cluster; several clusters a (request, kv head) for one to four requests with more than 8k tokens; a windowed
    layer is planned for its window, not for the context."""
    from lite_lang_b200.parts.attention import GQAttention

    def attn(nh, nkv, window=None):
        a = GQAttention.__new__(GQAttention)
        a.num_heads, a.num_kv_heads, a.window = nh, nkv, window
        return a

    plan = GQAttention._plan_mma
    a = attn(12, 2)
    # (row blocks, splits, one token an entry, warps, clusters a (entry, kv head))
    assert plan(a, None, 8, 4096, 148) == (8, 8, True, 4, 1)        # 8 x 2 x 8 = 128 CTAs of 4 warps
    assert plan(a, None, 1, 4096, 148) == (1, 8, True, 8, 1)
    assert plan(a, None, 16, 4096, 148) == (16, 4, True, 8, 1)
    assert plan(a, None, 64, 4096, 148) == (64, 1, True, 8, 1)
    assert plan(a, None, 8, 100, 148)[1] == 1                       # fewer than 8 tiles a split: no splits
    for entries, kv, nouter in ((1, 8192, 1), (1, 16384, 8), (1, 65536, 16), (2, 16384, 8), (4, 16384, 1),
                                (4, 32768, 4), (8, 65536, 1)):
        got = plan(a, None, entries, kv, 148)
        assert got[4] == nouter, (entries, kv, got)
        if nouter > 1:
            assert got[1] == 4 and got[3] == 8 and entries * 2 * 4 * nouter <= 148
    assert plan(attn(12, 2, window=1000), None, 1, 65536, 148) == plan(a, None, 1, 1016, 148)
    # more than 8 query heads a kv head: the other kernel (clusters = 0)
    assert plan(attn(32, 2), None, 4, 4096, 148)[4] == 0
