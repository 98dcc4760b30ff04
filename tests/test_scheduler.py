"""The scheduler's decisions, on the CPU, with a fake model whose next token is a function of
the request and the position (so a recomputed request must produce the same tokens)."""
import numpy as np
import pytest

from aien_sovereign_core_mv_b200.csrc import build

host = build.load_host()


def make(pages=64, page=4, max_requests=8, **limits):
    cm = host.CacheManager(page, [host.GroupSpec(host.GroupKind.Full, 0, pages)], max_requests)
    sc = host.SchedulerConfig()
    sc.max_batch_size, sc.max_batch_tokens, sc.max_prefill_tokens, sc.prefill_chunk_size = 8, 64, 32, 16
    sc.watermark_blocks = 0
    for k, v in limits.items():
        setattr(sc, k, v)
    return cm, host.Scheduler(sc, cm)


def fake_token(rid, position):
    return 10 + (rid * 7 + position * 3) % 50


def drive(sched, cm, max_steps=2000, log=None):
    """Run to completion; returns {id: (generated, reason)}."""
    done = {}
    for _ in range(max_steps):
        if not sched.has_work():
            break
        plan = sched.plan()
        if log is not None:
            log.append(plan)
        sampled = [fake_token(e.id, e.start + len(e.tokens)) for e in plan.entries if e.wants_logits]
        if plan.entries:
            sched.commit(sampled)
        assert cm.check() == ""
        for ev in sched.take_finished():
            done[ev.id] = (list(ev.generated), ev.reason.name, ev.message)
    return done


def expected(rid, prompt_len, n):
    return [fake_token(rid, prompt_len + i) for i in range(n)]


def test_portions_budget_and_decode_every_step():
    cm, s = make()
    s.submit(1, list(range(40)), 5)
    s.submit(2, list(range(10)), 5)
    log = []
    done = drive(s, cm, log=log)
    first = log[0]
    assert [(e.id, len(e.tokens), e.start, e.wants_logits) for e in first.entries] == [(1, 16, 0, False), (2, 10, 0, True)]
    assert first.prefill_tokens == 26 and first.num_tokens == 26
    second = log[1]                                           # request 1 goes on, request 2 decodes
    assert [(e.id, len(e.tokens), e.start) for e in second.entries] == [(1, 16, 16), (2, 1, 10)]
    third = log[2]
    assert [(e.id, len(e.tokens), e.start, e.wants_logits) for e in third.entries] == [(1, 8, 32, True), (2, 1, 11, True)]
    assert done[1][0] == expected(1, 40, 5) and done[2][0] == expected(2, 10, 5)
    assert done[1][1] == "LengthLimit" and cm.num_requests == 0 and cm.free_count(0) == 64
    for p in log:
        assert p.num_tokens <= 64 and p.prefill_tokens <= 32 and len(p.entries) <= 8


def test_fifo_admission_under_the_sequence_limit():
    cm, s = make(max_batch_size=2)
    for rid in (1, 2, 3):
        s.submit(rid, [1, 2, 3], 2)
    log = []
    done = drive(s, cm, log=log)
    assert [e.id for e in log[0].entries] == [1, 2]           # the third waits its turn
    assert 3 not in [e.id for p in log[:2] for e in p.entries]
    assert set(done) == {1, 2, 3}


def test_stop_token_ends_and_is_not_emitted():
    cm, s = make()
    stop = fake_token(4, 6 + 2)                               # the third generated token
    s.submit(4, list(range(6)), 10, [stop])
    done = drive(s, cm)
    assert done[4][0] == expected(4, 6, 2) and done[4][1] == "StopToken"


def test_whole_prompt_mode():
    cm, s = make(chunk_prefill=False)
    s.submit(1, list(range(30)), 1)
    s.submit(2, list(range(40)), 1)                           # larger than max_prefill_tokens: can never run whole
    done = drive(s, cm)
    assert done[1][1] == "LengthLimit" and done[2][1] == "Aborted" and "chunk_prefill" in done[2][2]


def test_request_larger_than_the_pool_is_aborted_not_queued_forever():
    cm, s = make(pages=4)                                      # 16 tokens
    s.submit(1, list(range(30)), 4)
    s.submit(2, list(range(5)), 2)
    done = drive(s, cm)
    assert done[1][1] == "Aborted" and host.EXHAUSTED_PREFIX in done[1][2]
    assert done[2][0] == expected(2, 5, 2)


def test_admission_reserves_the_whole_input():
    """Two prompts of 20 tokens need 6 pages each (21 tokens); 8 pages hold only one at a time."""
    cm, s = make(pages=8)
    s.submit(1, list(range(20)), 3)
    s.submit(2, list(range(20)), 3)
    log = []
    done = drive(s, cm, log=log)
    assert [e.id for e in log[0].entries] == [1]
    first_of_2 = next(i for i, p in enumerate(log) if any(e.id == 2 for e in p.entries))
    assert all(s_.preempted == [] for s_ in log)               # nobody had to be thrown out
    assert first_of_2 >= 4
    assert done[1][0] == expected(1, 20, 3) and done[2][0] == expected(2, 20, 3)


def test_out_of_pages_preempts_lowest_priority_and_recomputes():
    """Decoding outgrows the pool: the lower-priority request is preempted, its pages are given
    back, and it is recomputed from prompt ++ generated; its tokens are the same as if it had
    never been interrupted, and none is emitted twice."""
    cm, s = make(pages=7, page=4)                              # 28 tokens
    s.submit(1, list(range(8)), 12, [], 5)                     # priority 5
    s.submit(2, list(range(8)), 12, [], 1)                     # priority 1: the victim
    log = []
    done = drive(s, cm, log=log)
    preempted = [p.preempted for p in log if p.preempted]
    assert preempted and all(v == [2] for v in preempted)
    assert done[1][0] == expected(1, 8, 12) and done[2][0] == expected(2, 8, 12)
    assert s.record(2).preemptions >= 1 and s.record(1).preemptions == 0
    # after the preemption the victim's next entry starts from position 0 and carries its own tokens
    k = next(i for i, p in enumerate(log) if p.preempted)
    again = next(e for p in log[k + 1:] for e in p.entries if e.id == 2)
    assert again.start == 0 and again.tokens[:8] == list(range(8)) and len(again.tokens) > 8 or again.tokens == list(range(8))
    assert s.metrics()["preemptions"] == len(preempted) and cm.free_count(0) == 7


def test_watermark_preempts_before_the_pool_is_dry():
    cm, s = make(pages=10, page=4, watermark_blocks=3)
    s.submit(1, list(range(12)), 20, [], 2)
    s.submit(2, list(range(12)), 20, [], 1)
    log = []
    done = drive(s, cm, log=log)
    assert any(p.preempted == [2] for p in log)
    assert done[1][0] == expected(1, 12, 20) and done[2][0] == expected(2, 12, 20)


def test_cancel_and_bad_calls():
    cm, s = make()
    s.submit(1, [1, 2, 3], 4)
    with pytest.raises(ValueError, match="already live"):
        s.submit(1, [1], 1)
    with pytest.raises(ValueError, match="empty prompt"):
        s.submit(9, [], 1)
    plan = s.plan()
    with pytest.raises(RuntimeError):
        s.plan()                                               # a planned step must be committed first
    with pytest.raises(ValueError, match="sampled tokens expected"):
        s.commit([])
    assert s.cancel(1) and not s.cancel(1)
    s.commit([5])                                              # the cancelled request ignores the token
    ev = s.take_finished()
    assert [e.reason.name for e in ev] == ["Cancelled"] and cm.num_requests == 0 and not s.has_work()


def test_context_limit():
    cm, s = make(max_context=12)
    s.submit(1, list(range(8)), 100)
    done = drive(s, cm)
    assert done[1][1] == "LengthLimit" and len(done[1][0]) == 4


def test_fork_shares_the_cache_and_runs_at_once():
    cm, s = make()
    s.submit(1, list(range(10)), 6)
    plan = s.plan(); s.commit([fake_token(1, 10)])             # prompt done, one token generated
    copies = s.fork(1, 2, 4, [], 0)
    assert copies == [] and cm.num_tokens(2) == 10 and cm.table(2, 0) == cm.table(1, 0)
    rec = s.record(2)
    assert rec.prompt == list(range(10)) + [fake_token(1, 10)] and rec.computed == 10 and rec.state.name == "Running"
    plan = s.plan()                                             # both decode the token they share; the tail page is copied for one
    assert [(e.id, e.start, e.tokens) for e in plan.entries] == [(1, 10, [fake_token(1, 10)]), (2, 10, [fake_token(1, 10)])]
    assert len(plan.copies) >= 1
    s.commit([fake_token(1, 11), fake_token(2, 11)])
    done = drive(s, cm)
    assert done[1][0] == expected(1, 10, 6) and done[2][0] == [fake_token(2, 11 + i) for i in range(4)]
    assert cm.free_count(0) == 64
    with pytest.raises(ValueError, match="not running"):
        s.fork(1, 3, 4, [], 0)


def drive_overlapped(sched, cm, max_steps=4000):
    """The loop of Generator.step_async without a device: step n+1 is planned while the tokens of
    step n are still unknown; they are resolved one step late."""
    done, flight = {}, None
    for _ in range(max_steps):
        if not sched.has_work() and flight is None:
            break
        plan = sched.plan()
        now = None
        if plan.entries:
            for e in plan.entries:                       # an unknown token may only be the last one of an entry
                assert all(t >= 0 for t in e.tokens[:-1])
            now = [(e.id, fake_token(e.id, e.start + len(e.tokens))) for e in plan.entries if e.wants_logits]
            sched.commit_deferred()
        if flight:
            sched.resolve(flight)
        flight = now
        assert cm.check() == ""
        for ev in sched.take_finished():
            assert all(t >= 0 for t in ev.generated)
            done[ev.id] = (list(ev.generated), ev.reason.name, ev.message)
    return done


def test_overlapped_steps_give_the_same_tokens():
    """Lengths, stop ids met early, late and at the length limit, a pool so small that requests are
    preempted with a token still unknown: the overlapped loop ends every request like the plain loop."""
    rng = np.random.default_rng(3)
    for trial in range(30):
        pages = int(rng.integers(10, 40))
        reqs = []
        for rid in range(1, int(rng.integers(2, 9))):
            plen, n = int(rng.integers(1, 30)), int(rng.integers(1, 25))
            stop_at = int(rng.integers(0, n + 3))          # sometimes beyond the length limit: never met
            stops = [fake_token(rid, plen + stop_at)] if rng.random() < 0.6 else []
            reqs.append((rid, plen, n, stops))
        outcomes = []
        for drive_fn in (drive, drive_overlapped):
            cm, s = make(pages=pages, page=4, max_requests=8)
            for rid, plen, n, stops in reqs:
                s.submit(rid, [int(t) for t in rng.integers(0, 9, plen)], n, stops, 0)
            outcomes.append(drive_fn(s, cm))
            assert cm.free_count(0) == pages and not s.has_work()
        plain, overlapped = outcomes
        assert {k: v[:2] for k, v in plain.items()} == {k: v[:2] for k, v in overlapped.items()}, trial


def test_deferred_commit_rules():
    cm, s = make()
    s.submit(1, list(range(6)), 3, [fake_token(1, 7)], 0)
    s.plan(); s.commit_deferred()                           # prompt; first token unknown
    plan = s.plan()
    assert plan.entries[0].tokens == [-1] and plan.entries[0].start == 6
    s.commit_deferred()
    with pytest.raises(RuntimeError, match="not resolved"):
        s.fork(1, 2, 4, [], 0)
    s.resolve([(1, fake_token(1, 6))])                      # the first token comes in: request goes on
    assert s.record(1).generated == [fake_token(1, 6), -1] and s.record(1).unresolved == 1
    s.plan(); s.commit_deferred()                           # third token planned: the length limit is reached, unresolved
    assert s.record(1).draining and s.plan().entries == []
    s.resolve([(1, fake_token(1, 7))])                      # ... but the second token was the stop id
    ev = s.take_finished()
    assert len(ev) == 1 and ev[0].reason.name == "StopToken" and ev[0].generated == [fake_token(1, 6)]
    s.resolve([(1, 5)])                                     # the value of the dropped token arrives: ignored
    assert cm.free_count(0) == 64 and not s.has_work()


def test_rollback_of_a_failed_step_restores_lengths_and_the_step_can_be_planned_again():
    cm, s = make()
    s.submit(1, list(range(20)), 4)
    s.submit(2, list(range(5)), 4)
    p0 = s.plan()
    s.commit([fake_token(e.id, e.start + len(e.tokens)) for e in p0.entries if e.wants_logits])
    held = {1: cm.num_tokens(1), 2: cm.num_tokens(2)}
    free = cm.free_count(0)
    p1 = s.plan()                                             # request 1: rest of the prompt; request 2: one token
    assert cm.num_tokens(1) == 20 and cm.num_tokens(2) == 6
    s.rollback()                                              # the launch failed
    assert {1: cm.num_tokens(1), 2: cm.num_tokens(2)} == held and cm.free_count(0) == free and cm.check() == ""
    with pytest.raises(RuntimeError):
        s.rollback()                                          # nothing is planned now
    p2 = s.plan()                                             # the same step again
    assert [(e.id, list(e.tokens), e.start) for e in p2.entries] == [(e.id, list(e.tokens), e.start) for e in p1.entries]
    s.commit([fake_token(e.id, e.start + len(e.tokens)) for e in p2.entries if e.wants_logits])
    done = drive(s, cm)
    assert done[1][0] == expected(1, 20, 4) and done[2][0] == expected(2, 5, 4)


def test_rollback_of_the_step_that_admitted_a_request():
    cm, s = make()
    s.submit(7, list(range(9)), 3)
    s.plan()
    s.rollback()
    assert cm.num_tokens(7) == 0 and cm.free_count(0) == 64 and cm.check() == ""
    done = drive(s, cm)
    assert done[7][0] == expected(7, 9, 3) and cm.num_requests == 0


def test_restart_running_recomputes_from_known_tokens_only():
    cm, s = make()
    s.submit(1, list(range(6)), 6)
    s.submit(2, list(range(3)), 6)
    for _ in range(2):                                        # two steps resolved in the ordinary way
        p = s.plan()
        s.commit([fake_token(e.id, e.start + len(e.tokens)) for e in p.entries if e.wants_logits])
    p = s.plan()
    s.commit_deferred()                                       # a third whose tokens never arrive
    assert s.record(1).unresolved == 1
    s.restart_running()
    assert cm.num_requests == 0 and cm.free_count(0) == 64 and cm.check() == ""
    r = s.record(1)
    assert r.unresolved == 0 and list(r.generated) == expected(1, 6, 2) and r.computed == 0 and r.preemptions == 1
    s.resolve_for([(e.id, 99, e.arrival) for e in p.entries])    # late values of the dropped step change nothing
    assert list(s.record(1).generated) == expected(1, 6, 2)
    done = drive(s, cm)
    assert done[1][0] == expected(1, 6, 6) and done[2][0] == expected(2, 3, 6)


def test_prompt_at_or_beyond_the_context_limit_is_aborted_and_blocks_nobody():
    cm, s = make(pages=64, page=4, max_context=32)
    s.submit(1, list(range(100)), 4)                          # would need 25 pages of a block table that holds 8
    s.submit(2, list(range(32)), 4)                           # no room for a single new token either
    s.submit(3, list(range(10)), 4)
    ev = {e.id: e for e in s.take_finished()}
    assert ev[1].reason.name == "Aborted" and "context limit" in ev[1].message and ev[2].reason.name == "Aborted"
    done = drive(s, cm)
    assert done[3][0] == expected(3, 10, 4) and cm.check() == "" and cm.num_requests == 0


def test_a_value_of_an_earlier_submission_never_reaches_a_new_request_with_the_same_id():
    cm, s = make()
    s.submit(5, list(range(4)), 8)
    p = s.plan()
    s.commit_deferred()                                       # its first token is still on the device
    assert s.cancel(5)
    s.submit(5, list(range(7)), 8)                            # the id is used again before that token arrives
    s.resolve_for([(e.id, 42, e.arrival) for e in p.entries if e.wants_logits])     # dropped: another submission
    assert list(s.record(5).generated) == []
    s.take_finished()
    done = drive(s, cm)
    assert done[5][0] == expected(5, 7, 8)


def test_steps_cut_to_whole_tiles():
    """align_step_tokens: a portion that is not its input's last gives up what overhangs the last whole tile
    of the step (a quarter of itself at most); the end of an input and plain decode steps are left alone,
    nobody else is given the tokens held back, and the requests produce what they produce without it."""
    def run(align):
        cm, s = make(pages=256, max_batch_tokens=64, max_prefill_tokens=32, prefill_chunk_size=32, align_step_tokens=align)
        s.submit(1, list(range(6)), 12)              # decoding from the second step on
        s.submit(2, list(range(7)), 12)
        s.submit(3, list(range(100)), 4)             # the long input: portions of 32 beside two decode tokens
        s.submit(4, list(range(50)), 4)              # waits for prefill room
        log = []
        done = drive(s, cm, log=log)
        return log, done
    plain_log, plain_done = run(0)
    log, done = run(16)
    assert done == plain_done and set(done) == {1, 2, 3, 4}
    # without the option some step holds 32 + 2 = 34 tokens
    assert any(p.num_tokens == 34 for p in plain_log)
    for p in log:
        sizes = {e.id: len(e.tokens) for e in p.entries}
        longest = max(sizes.values())
        ends = any(e.wants_logits and len(e.tokens) > 1 for e in p.entries)
        if longest > 1 and not ends and longest >= 4 * (p.num_tokens % 16 or 16):
            assert p.num_tokens % 16 == 0, (p.num_tokens, sizes)
        assert p.num_tokens <= 64 and p.prefill_tokens <= 32
    # the portion beside the two decoding requests: 30 tokens, not 32
    assert any({1, 2, 3} <= {e.id for e in p.entries} and p.num_tokens == 32 and max(len(e.tokens) for e in p.entries) == 30 for p in log)
    with pytest.raises(Exception):
        make(align_step_tokens=-1)
