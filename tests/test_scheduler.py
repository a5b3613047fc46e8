"""The scheduler's decisions (no GPU): admission, portions, decoding, finishing, running out of pages."""

from __future__ import annotations

import pytest

from distie_b200.cache import CacheExhausted, CacheManager
from distie_b200.engine.scheduler import Scheduler, Sequence, SeqState
from distie_b200.parts import CacheNeed

NEED = CacheNeed(2, 16, None)


def make(pages=16, page_size=4, max_seqs=4, budget=64, chunk=None, seats=None):
    cache = CacheManager({0: NEED}, {}, num_pages=pages, page_size=page_size, max_seats=seats or max_seqs,
                         max_tokens_per_request=pages * page_size)
    return Scheduler(cache, max_seqs, budget, chunk), cache


def seq(name, prompt_len, new=4, **kw):
    return Sequence(name, list(range(1, prompt_len + 1)), new, **kw)


def run_step(sched, token=7):
    plan = sched.schedule()
    sampled = [token] * sum(1 for item in plan.items if item.samples)
    return plan, sched.complete(plan, sampled)


def test_fifo_prefill_then_decode():
    sched, _ = make()
    a, b = seq("a", 5), seq("b", 3)
    sched.submit(a), sched.submit(b)
    plan = sched.schedule()
    assert [(i.seq.request_id, len(i.token_ids), i.past_len, i.samples) for i in plan.items] == [("a", 5, 0, True), ("b", 3, 0, True)]
    assert plan.kind == "prefill"
    sched.complete(plan, [10, 11])
    plan = sched.schedule()
    assert [(i.token_ids, i.past_len) for i in plan.items] == [([10], 5), ([11], 3)] and plan.kind == "decode"


def test_max_seqs_and_submit_checks():
    sched, _ = make(max_seqs=2)
    for name in "abc":
        sched.submit(seq(name, 2))
    plan = sched.schedule()
    assert len(plan.items) == 2 and sched.num_waiting == 1
    with pytest.raises(ValueError, match="duplicate"):
        sched.submit(seq("a", 2))
    with pytest.raises(ValueError, match="non-empty"):
        sched.submit(Sequence("e", [], 3))
    with pytest.raises(ValueError, match="max_new_tokens"):
        sched.submit(Sequence("f", [1], 0))
    with pytest.raises(CacheExhausted, match="out of KV blocks"):
        sched.submit(seq("big", 60, new=8))  # 68 tokens > 16 pages of 4


def test_token_budget_cuts_prompts_into_portions():
    sched, _ = make(pages=64, budget=10)
    a, b = seq("a", 14), seq("b", 9)
    sched.submit(a), sched.submit(b)
    plan = sched.schedule()
    assert [(i.seq.request_id, len(i.token_ids), i.samples) for i in plan.items] == [("a", 10, False)]
    assert sched.num_waiting == 1, "no budget left: b waits"
    assert sched.complete(plan, []) == [] and a.num_cached == 10 and a.output_ids == []
    plan = sched.schedule()
    assert [(i.seq.request_id, len(i.token_ids), i.past_len, i.samples) for i in plan.items] == [("a", 4, 10, True), ("b", 6, 0, False)]
    sched.complete(plan, [5])
    plan = sched.schedule()  # a decodes (1 token, first), b gets its last 3
    assert [(i.seq.request_id, len(i.token_ids), i.samples) for i in plan.items] == [("a", 1, True), ("b", 3, True)]


def test_prefill_chunk_bounds_every_portion():
    sched, _ = make(pages=64, budget=64, chunk=5)
    sched.submit(seq("a", 12))
    sizes = []
    while True:
        plan = sched.schedule()
        sizes.append(len(plan.items[0].token_ids))
        done = plan.items[0].samples
        sched.complete(plan, [3] if done else [])
        if done:
            break
    assert sizes == [5, 5, 2]


def test_budget_also_bounds_admission_and_decoding_never_starves():
    sched, _ = make(pages=64, budget=3, max_seqs=4)
    for name in "abcd":
        sched.submit(seq(name, 1, new=3))
    sizes = []
    while sched.has_work():
        plan, _ = run_step(sched)
        assert all(len(i.token_ids) == 1 and i.samples for i in plan.items)
        sizes.append(len(plan.items))
    assert sizes == [3, 3, 3, 1, 1, 1], "three fill the budget; the fourth joins when they are done"


def test_waits_for_pages_and_admits_head_only():
    sched, cache = make(pages=4, page_size=4)
    a, big, small = seq("a", 9, new=2), seq("big", 8, new=2), seq("small", 2, new=2)
    for s in (a, big, small):
        sched.submit(s)
    plan = sched.schedule()
    assert [i.seq.request_id for i in plan.items] == ["a"], "big does not fit beside a; small may not overtake it"
    assert sched.num_waiting == 2


def test_finishing_frees_pages_and_eos_counts():
    sched, cache = make()
    a = seq("a", 5, new=3, eos_id=99)
    sched.submit(a)
    plan = sched.schedule()
    assert cache.free_pages() == 14
    out = sched.complete(plan, [99])
    assert out[0].finished and a.finish_reason == "eos" and a.output_ids == [99] and a.state is SeqState.FINISHED
    assert cache.free_pages() == 16 and not sched.has_work()
    b = seq("b", 2, new=2)
    sched.submit(b)
    run_step(sched), run_step(sched)
    assert b.finish_reason == "length" and len(b.output_ids) == 2 and cache.free_pages() == 16


def test_running_out_of_pages_preempts_the_newest_and_recomputes_it():
    sched, cache = make(pages=4, page_size=4, budget=64)
    a, b = seq("a", 7, new=8), seq("b", 7, new=8)
    sched.submit(a), sched.submit(b)
    run_step(sched)                      # both prefilled: 2 pages each, pool empty
    plan, _ = run_step(sched)            # token 8 of each still fits its second page
    assert len(plan.items) == 2
    plan = sched.schedule()              # token 9 needs a third page: b, the newest, is preempted
    assert [i.seq.request_id for i in plan.items] == ["a"]
    assert b.state is SeqState.WAITING and b.preemptions == 1 and b.num_cached == 0 and b.seat is None
    assert len(b.output_ids) == 2, "what it generated is kept and never emitted twice"
    assert sched.waiting()[0] is b, "a preempted request goes to the front of the queue"
    sched.complete(plan, [7])
    while a.state is not SeqState.FINISHED:
        run_step(sched)
    plan = sched.schedule()              # b comes back: prompt and its outputs from position 0
    item = plan.items[0]
    assert item.seq is b and item.past_len == 0 and item.token_ids == b.prompt_ids + b.output_ids and item.samples
    while sched.has_work():
        run_step(sched)
    assert len(b.output_ids) == 8 and cache.free_pages() == 4 and cache.free_seats == 4


def test_a_request_may_preempt_itself_and_abort_paths():
    sched, cache = make(pages=3, page_size=4)
    a, b = seq("a", 4, new=8), seq("b", 7, new=1)
    sched.submit(a), sched.submit(b)
    run_step(sched)  # b finishes at once (1 new token); a holds 1 page, then grows
    sched.abort("a")
    sched.abort("nobody")
    plan = sched.schedule()
    assert plan.items == () and a.finish_reason == "aborted" and cache.free_pages() == 3 and not sched.has_work()
    c, d = seq("c", 3), seq("d", 3)
    sched.submit(c), sched.submit(d)
    plan = sched.schedule()
    sched.abort("c")  # in flight: its result is discarded
    out = sched.complete(plan, [1, 2])
    assert [e.seq.request_id for e in out] == ["d"] and c.output_ids == []
    sched.schedule()
    assert cache.free_seats == 3


def test_forced_preemption_hook():
    sched, cache = make()
    a = seq("a", 6, new=5)
    sched.submit(a)
    run_step(sched)
    assert sched.force_preempt("a") and not sched.force_preempt("a")
    assert cache.free_pages() == 16 and a.preemptions == 1
    plan = sched.schedule()
    assert plan.items[0].token_ids == a.prompt_ids + a.output_ids


def test_complete_checks_the_number_of_tokens():
    sched, _ = make()
    sched.submit(seq("a", 2))
    plan = sched.schedule()
    with pytest.raises(ValueError):
        sched.complete(plan, [])


# -- a step ahead: the bookkeeping of a decode step launched before the tokens of the one before are known ----
def _token_for(seq, index):
    """A stand-in for the model: the token at output position `index` of a request (deterministic)."""
    return (sum(map(ord, seq.request_id)) * 31 + index * 7) % 50 + 1


def _drive(pipelined, specs, pages=24, eos=None):
    """Runs requests to the end, the plain way or a step ahead, and returns every emission in order."""
    sched, cache = make(pages=pages, page_size=4, max_seqs=4, budget=16)
    for name, prompt_len, new in specs:
        sched.submit(seq(name, prompt_len, new=new, eos_id=eos))
    emitted, in_flight = [], None

    def tokens_of(plan):
        # What the device would hand back: a token per sampling row, computed from the row's position alone.
        return [_token_for(i.seq, i.past_len + len(i.token_ids) - len(i.seq.prompt_ids)) for i in plan.items if i.samples]

    guard = 0
    while sched.has_work() or in_flight is not None:
        guard += 1
        assert guard < 500
        if in_flight is None:
            plan = sched.schedule()
            if not plan.items:
                continue
            if not pipelined or plan.kind != "decode":
                emitted += [(e.seq.request_id, e.token_id, e.finished) for e in sched.complete(plan, tokens_of(plan))]
                continue
            in_flight = plan
        plan, in_flight = in_flight, None
        if sched.can_look_ahead(plan):
            sched.assume(plan)
            following = sched.schedule()
            same = len(following.items) == len(plan.items) and all(
                a.seq is b.seq and len(b.token_ids) == 1 for a, b in zip(plan.items, following.items))
            if same:
                assert all(b.token_ids == [Scheduler.PLACEHOLDER] for b in following.items)
                in_flight = following
            out = sched.resolve(plan, tokens_of(plan))
        else:
            out = sched.complete(plan, tokens_of(plan))
        emitted += [(e.seq.request_id, e.token_id, e.finished) for e in out]
    assert cache.free_pages() == pages
    return emitted


@pytest.mark.parametrize("eos", [None, 17, 33])
def test_a_step_ahead_emits_what_the_plain_loop_emits(eos):
    specs = [("a", 5, 9), ("b", 3, 4), ("c", 11, 12), ("d", 2, 1)]
    plain = _drive(False, specs, eos=eos)
    ahead = _drive(True, specs, eos=eos)
    by_request = lambda out, r: [(t, f) for name, t, f in out if name == r]  # noqa: E731
    for name, _, _ in specs:
        assert by_request(ahead, name) == by_request(plain, name), name
    assert sum(1 for _, _, finished in ahead if finished) == len(specs)


def test_a_step_ahead_survives_preemption():
    # So few pages that the newest request is preempted while steps are in flight; nothing is emitted twice.
    specs = [("a", 6, 10), ("b", 6, 10), ("c", 6, 10)]
    plain = _drive(False, specs, pages=9)
    ahead = _drive(True, specs, pages=9)
    for name, _, _ in specs:
        assert [t for n, t, _ in ahead if n == name] == [t for n, t, _ in plain if n == name]
