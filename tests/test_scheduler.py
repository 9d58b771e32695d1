"""The scheduler's decisions on the CPU, with a stand-in for the model step (after the reference's
tests/test_scheduler.py, whose fake ``engine_step`` plays the same part, ``:29-46``)."""

import pytest

from clockwork_b200.cache import CacheManager, PrefixCache
from clockwork_b200.config import SchedulerConfig
from clockwork_b200.engine.scheduler import Scheduler
from clockwork_b200.engine.sequence import Sequence, SequenceStatus
from clockwork_b200.parts import PagedKVNeed
from clockwork_b200.sampling import SamplingParams


def make(num_pages=16, page_size=4, max_num_seqs=8, budget=32, chunk=None, watermark=0.0, prefix=False):
    cache = CacheManager({0: PagedKVNeed(1, 16, None)}, num_pages=num_pages, page_size=page_size, watermark=watermark)
    pc = PrefixCache(cache.groups[0].allocator, page_size) if prefix else None
    sched = Scheduler(SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=budget,
                                      prefill_chunk_size=chunk), cache, pc)
    return sched, cache, pc


def seq(name, n, arrival, start=0):
    return Sequence(name, list(range(start, start + n)), SamplingParams(max_tokens=100), arrival_time=float(arrival))


def fake_step(sched, cache, pc, out, finish=()):
    """What the engine does around the model: advance progress, append a token where one is sampled,
    record prompt pages, finish some sequences."""
    for p in out.portions:
        p.seq.num_computed_tokens = p.start + p.num_tokens
        cache.get(p.seq.seq_id).num_computed = p.seq.num_computed_tokens
        if p.samples:
            p.seq.append_token(1000 + len(p.seq.output_token_ids))
    if pc is not None:
        for s in out.prefill_seqs:
            n = min(s.num_computed_tokens, len(s.prompt_token_ids))
            pc.insert(s.prompt_token_ids[:n], cache.get(s.seq_id).tables[0])
    for s in sched.running:
        if s.seq_id in finish:
            s.status = SequenceStatus.FINISHED_LENGTH
    sched.free_finished()
    cache.check_invariants(pc.references() if pc else None)


def plan(out):
    return [(p.seq.seq_id, p.start, p.num_tokens, p.samples) for p in out.portions]


def test_token_budget_cuts_prompts_into_portions():
    sched, cache, _ = make(budget=10, num_pages=32)
    sched.add_seq(seq("a", 7, 0))
    sched.add_seq(seq("b", 9, 1))
    out = sched.schedule()
    assert plan(out) == [("a", 0, 7, True), ("b", 0, 3, False)] and out.num_batched_tokens == 10
    fake_step(sched, cache, None, out)
    out = sched.schedule()  # a decodes first, b takes what is left of its prompt
    assert plan(out) == [("a", 7, 1, True), ("b", 3, 6, True)]
    assert [s.seq_id for s in out.decode_seqs] == ["a"] and [s.seq_id for s in out.prefill_seqs] == ["b"]
    fake_step(sched, cache, None, out)
    assert plan(sched.schedule()) == [("a", 8, 1, True), ("b", 9, 1, True)]


def test_prefill_chunk_size_and_a_prompt_longer_than_the_budget():
    sched, cache, _ = make(budget=8, chunk=5, num_pages=32)
    sched.add_seq(seq("a", 13, 0))
    seen = []
    for _ in range(4):
        out = sched.schedule()
        seen.append(plan(out))
        fake_step(sched, cache, None, out)
    assert seen == [[("a", 0, 5, False)], [("a", 5, 5, False)], [("a", 10, 3, True)], [("a", 13, 1, True)]]


def test_decodes_come_before_waiting_prompts_and_head_blocks():
    sched, cache, _ = make(budget=6, num_pages=32)
    sched.add_seq(seq("a", 4, 0))
    fake_step(sched, cache, None, sched.schedule())
    sched.add_seq(seq("big", 20, 1))
    sched.add_seq(seq("small", 2, 2))
    out = sched.schedule()
    # a's decode, then a portion of the head of the queue; 'small' may not overtake 'big'
    assert plan(out) == [("a", 4, 1, True), ("big", 0, 5, False)]
    assert [s.seq_id for s in sched.waiting] == ["small"]


def test_max_num_seqs():
    sched, cache, _ = make(max_num_seqs=2, num_pages=32)
    for i in range(3):
        sched.add_seq(seq(f"s{i}", 3, i))
    out = sched.schedule()
    assert [p.seq.seq_id for p in out.portions] == ["s0", "s1"] and sched.stats.num_waiting == 1
    fake_step(sched, cache, None, out, finish={"s0"})
    assert [p.seq.seq_id for p in sched.schedule().portions] == ["s1", "s2"]


def test_admission_needs_pages_for_the_whole_sequence_with_the_watermark_left():
    sched, cache, _ = make(num_pages=10, page_size=4, watermark=0.2)
    sched.add_seq(seq("a", 32, 0))  # 8 pages + 2 free: fits exactly
    sched.add_seq(seq("b", 1, 1))
    out = sched.schedule()
    assert [p.seq.seq_id for p in out.portions] == ["a"]  # b would leave less than the watermark
    assert cache.num_free_pages() == [2] and [s.seq_id for s in sched.waiting] == ["b"]


def test_pages_run_out_latest_arrival_is_preempted_and_recomputed():
    sched, cache, _ = make(num_pages=6, page_size=4, budget=64)
    a, b, c = seq("a", 8, 0), seq("b", 8, 1), seq("c", 7, 2)
    for s in (a, b, c):
        sched.add_seq(s)
    fake_step(sched, cache, None, sched.schedule())
    assert cache.num_free_pages() == [0]
    out = sched.schedule()  # a needs a new page: c, the latest arrival, gives its pages up
    assert [s.seq_id for s in out.preempted] == ["c"] and c.status is SequenceStatus.PREEMPTED
    assert plan(out) == [("a", 8, 1, True), ("b", 8, 1, True)]
    assert c.num_computed_tokens == 0 and len(c) == 8 and sched.waiting[0] is c  # tokens kept, front of the queue
    assert sched.stats.num_preempted_total == 1 and "c" not in cache.requests
    fake_step(sched, cache, None, out)
    sched.add_seq(seq("d", 2, 3))
    out = sched.schedule()
    assert plan(out)[:2] == [("a", 9, 1, True), ("b", 9, 1, True)]
    assert [s.seq_id for s in sched.waiting][0] == "c"  # c is readmitted before d, when pages allow
    fake_step(sched, cache, None, out, finish={"a", "b"})
    out = sched.schedule()
    assert plan(out) == [("c", 0, 8, True), ("d", 0, 2, True)]  # recompute covers prompt and generated token


def test_a_sequence_alone_preempts_itself():
    sched, cache, _ = make(num_pages=2, page_size=4)
    a = seq("a", 8, 0)
    sched.add_seq(a)
    fake_step(sched, cache, None, sched.schedule())
    out = sched.schedule()
    assert [s.seq_id for s in out.preempted] == ["a"] and not out.portions
    assert cache.num_free_pages() == [2]


def test_prefix_hit_lowers_the_cost_and_a_refused_admission_rolls_back():
    sched, cache, pc = make(num_pages=8, page_size=4, budget=12, prefix=True)
    sched.add_seq(seq("a", 10, 0))
    fake_step(sched, cache, pc, sched.schedule(), finish={"a"})
    assert pc.tree.num_pages() == 2 and cache.num_free_pages() == [6]
    b = Sequence("b", list(range(8)) + [50, 51, 52], SamplingParams(), arrival_time=1.0)
    sched.add_seq(b)
    out = sched.schedule()
    assert plan(out) == [("b", 8, 3, True)] and b.num_cached_tokens == 8
    assert sched.stats.total_cached_tokens == 8 and cache.get("b").tables[0][:2] == [0, 1]
    fake_step(sched, cache, pc, out)
    # a third request shares the prefix but the pool has too few pages left: nothing may leak
    big = Sequence("big", list(range(8)) + list(range(100, 124)), SamplingParams(), arrival_time=2.0)
    sched.add_seq(big)
    before = [cache.groups[0].allocator.refcount(p) for p in range(8)]
    out = sched.schedule()
    assert [p.seq.seq_id for p in out.portions] == ["b"] and big.status is SequenceStatus.WAITING
    after = [cache.groups[0].allocator.refcount(p) for p in range(8)]
    assert before[:2] == after[:2] and big.num_cached_tokens == 0
    fake_step(sched, cache, pc, out, finish={"b"})
    cache.check_invariants(pc.references())


def test_abort_in_every_state():
    sched, cache, _ = make(num_pages=8, page_size=4, max_num_seqs=1)
    a, b = seq("a", 5, 0), seq("b", 5, 1)
    sched.add_seq(a)
    sched.add_seq(b)
    fake_step(sched, cache, None, sched.schedule())
    sched.abort("b")  # waiting: holds nothing
    assert b.status is SequenceStatus.FINISHED_ABORTED and not sched.waiting
    sched.abort("a")  # running: gives its pages back
    assert a.status is SequenceStatus.FINISHED_ABORTED and cache.num_free_pages() == [8]
    sched.abort("nobody")
    assert not sched.has_unfinished()


def test_preempted_requests_wait_in_rank_order_before_the_arrivals_and_can_be_aborted():
    """Two requests preempted in different steps come back in the order of their arrival, both ahead of a
    request that has never run; aborting one of them while it waits leaves nothing behind."""
    sched, cache, _ = make(num_pages=6, page_size=4, budget=64)
    a, b, c = seq("a", 8, 0), seq("b", 7, 1), seq("c", 7, 2)
    for s in (a, b, c):
        sched.add_seq(s)
    fake_step(sched, cache, None, sched.schedule())           # 2 + 2 + 2 pages: the pool is full
    out = sched.schedule()                                     # a needs a third page: c goes
    assert [s.seq_id for s in out.preempted] == ["c"]
    fake_step(sched, cache, None, out)
    for _ in range(3):
        fake_step(sched, cache, None, sched.schedule())        # a and b fill the pages they have
    out = sched.schedule()                                     # now a needs a fourth page: b goes
    assert [s.seq_id for s in out.preempted] == ["b"] and [s.seq_id for s in sched.running] == ["a"]
    sched.add_seq(seq("d", 3, 3))
    assert [s.seq_id for s in sched.waiting] == ["b", "c", "d"]  # by arrival among the preempted, d behind them
    assert sched.stats.num_waiting == 3 and sched.stats.num_running == 1 and sched.stats.num_preempted_total == 2
    sched.abort("b")
    assert b.status is SequenceStatus.FINISHED_ABORTED and [s.seq_id for s in sched.waiting] == ["c", "d"]
    fake_step(sched, cache, None, out, finish={"a"})
    out = sched.schedule()
    assert [p.seq.seq_id for p in out.portions] == ["c", "d"] and c.num_computed_tokens == 0
    fake_step(sched, cache, None, out, finish={"c", "d"})
    assert not sched.has_unfinished() and cache.num_free_pages() == [6] and cache.state.num_free == cache.state.num_slots


def test_a_scripted_session_is_deterministic():
    def run():
        sched, cache, pc = make(num_pages=12, page_size=4, budget=16, chunk=6, prefix=True, max_num_seqs=3)
        log = []
        arrivals = {0: [("a", 9, 0)], 1: [("b", 14, 0)], 2: [("c", 9, 0), ("d", 5, 40)], 5: [("e", 11, 0)]}
        n = 0
        for step in range(40):
            for name, length, start in arrivals.get(step, []):
                sched.add_seq(seq(name, length, n, start))
                n += 1
            out = sched.schedule()
            log.append((plan(out), [s.seq_id for s in out.preempted]))
            done = {s.seq_id for s in sched.running if len(s.output_token_ids) >= 6}
            fake_step(sched, cache, pc, out, finish=done)
            if not sched.has_unfinished() and step > 6:
                break
        assert not sched.has_unfinished()
        return log, sched.stats

    first, stats = run()
    second, _ = run()
    assert first == second
    assert stats.total_cached_tokens >= 8  # c shares a's first two pages
