"""The cache manager: no page lost, held twice or freed twice, under random orders of
requests; appends are all-or-nothing; the page arithmetic predicts what appends take; windows
give pages back; forks share and copy on write; state slots."""
import random

import numpy as np
import pytest

from aien_sovereign_core_mv_b200.csrc import build

host = build.load_host()
Full, Window, State = host.GroupKind.Full, host.GroupKind.Window, host.GroupKind.State


def manager(page=4, pages=16, max_requests=8, window=0, state=False):
    groups = [host.GroupSpec(Full, 0, pages)]
    if window:
        groups.append(host.GroupSpec(Window, window, pages))
    if state:
        groups.append(host.GroupSpec(State, 0, max_requests))
    return host.CacheManager(page, groups, max_requests)


def test_first_pages_and_lifo_reuse():
    cm = manager()
    cm.add_request(1)
    cm.append([(1, 9)])
    assert cm.table(1, 0) == [0, 1, 2]                      # page 0 is handed out first
    cm.add_request(2)
    cm.append([(2, 4)])
    assert cm.table(2, 0) == [3]
    cm.free_request(1)
    cm.add_request(3)
    cm.append([(3, 5)])
    assert cm.table(3, 0) == [0, 1]                         # the stack hands a freed request's pages on in the order it held them
    assert cm.check() == ""


def test_exhaustion_changes_nothing_and_exact_fit_works():
    cm = manager(page=4, pages=4)
    cm.add_request(1); cm.add_request(2)
    cm.append([(1, 7)])
    before = (cm.table(1, 0), cm.free_count(0), cm.num_tokens(1))
    with pytest.raises(RuntimeError, match=host.EXHAUSTED_PREFIX):
        cm.append([(1, 2), (2, 9)])                          # the batch as a whole does not fit
    assert (cm.table(1, 0), cm.free_count(0), cm.num_tokens(1)) == before and cm.num_tokens(2) == 0
    assert not cm.can_append([(1, 2), (2, 9)]) and cm.can_append([(1, 1), (2, 8)])
    cm.append([(1, 1), (2, 8)])                              # exact fit
    assert cm.free_count(0) == 0 and cm.check() == ""
    with pytest.raises(RuntimeError, match=host.EXHAUSTED_PREFIX):
        cm.append([(2, 1)])
    cm.free_request(1)
    cm.append([(2, 1)])                                      # retry after a free works
    assert cm.check() == ""


def test_pages_needed_predicts_appends():
    rng = random.Random(3)
    cm = manager(page=4, pages=64, window=10)
    live = {}
    for step in range(300):
        rid = rng.randrange(6)
        if rid not in live:
            assert cm.pages_needed(rid, 5) == [2, 2]         # unknown request: from empty
            cm.add_request(rid); live[rid] = 0
        n = rng.choice([1, 1, 2, 3, 7, 16])
        need = cm.pages_needed(rid, n)
        free_before = [cm.free_count(g) for g in range(2)]
        try:
            cm.append([(rid, n)])
        except RuntimeError:
            cm.free_request(rid); del live[rid]
            continue
        live[rid] += n
        for g in range(2):
            taken = free_before[g] - cm.free_count(g)
            assert max(0, taken) == need[g], (step, g, taken, need)
        assert cm.check() == ""
        if rng.random() < 0.1:
            cm.free_request(rid); del live[rid]


def test_window_gives_pages_back():
    cm = manager(page=4, pages=16, window=6)
    cm.add_request(1)
    for _ in range(40):
        cm.append([(1, 1)])
    full, win = cm.table(1, 0), cm.table(1, 1)
    assert len(full) == 10 and all(p >= 0 for p in full)
    held = [p for p in win if p >= 0]
    assert len(held) <= 3 and win[:7] == [-1] * 7           # only the pages the last 6 keys touch
    assert cm.slot_of(1, 1, 39) >= 0 and cm.slot_of(1, 1, 34) >= 0 and cm.slot_of(1, 1, 20) == -1
    assert cm.metrics()["window_releases"] >= 7 and cm.check() == ""
    # a long request fits a window group far smaller than itself
    cm2 = host.CacheManager(4, [host.GroupSpec(Window, 6, 4)], 2)
    cm2.add_request(1)
    for _ in range(100):
        cm2.append([(1, 1)])
    assert cm2.check() == ""
    cm2.append([(1, 5)])                                     # a portion: needs the pages of window + portion
    with pytest.raises(RuntimeError, match=host.EXHAUSTED_PREFIX):
        cm2.append([(1, 12)])
    assert cm2.num_tokens(1) == 105 and cm2.check() == ""


def test_fork_shares_and_copies_on_write():
    cm = manager(page=4, pages=16, state=True)
    cm.add_request(1)
    cm.append([(1, 10)])                                     # pages 0,1,2 ; the tail page holds 2 tokens
    copies = cm.fork(1, 2, -1)
    assert copies == [(1, cm.state_slot(1, 1), cm.state_slot(2, 1))]      # the state slot is copied
    assert cm.table(2, 0) == cm.table(1, 0) and all(cm.refcount(0, p) == 2 for p in cm.table(1, 0))
    copies = cm.append([(2, 1)])                             # child writes into the shared tail: copy first
    assert len(copies) == 1 and copies[0][0] == 0 and copies[0][1] == cm.table(1, 0)[2] and copies[0][2] == cm.table(2, 0)[2]
    assert cm.table(2, 0)[:2] == cm.table(1, 0)[:2] and cm.table(2, 0)[2] != cm.table(1, 0)[2]
    assert cm.append([(1, 1)]) == []                         # the parent's tail is private again
    cm.free_request(1)
    assert all(cm.refcount(0, p) == 1 for p in cm.table(2, 0)) and cm.check() == ""
    with pytest.raises(ValueError, match="itself"):
        cm.fork(2, 2, -1)
    with pytest.raises(ValueError, match="fixed-size state"):
        cm.fork(2, 3, 4)                                     # state cannot be forked in the past
    assert not cm.has(3) and cm.check() == ""
    cm3 = manager(page=4, pages=16)
    cm3.add_request(1); cm3.append([(1, 10)])
    cm3.fork(1, 2, 6)                                        # fork at token 6: two pages shared, child holds 6
    assert cm3.num_tokens(2) == 6 and cm3.table(2, 0) == cm3.table(1, 0)[:2]
    assert len(cm3.append([(2, 3)])) == 1 and cm3.check() == ""


def test_truncate():
    cm = manager(page=4, pages=8, window=0)
    cm.add_request(1); cm.append([(1, 14)])
    cm.truncate(1, 5)
    assert cm.num_tokens(1) == 5 and len(cm.table(1, 0)) == 2 and cm.free_count(0) == 6 and cm.check() == ""
    with pytest.raises(ValueError):
        cm.truncate(1, 9)
    cmw = manager(page=4, pages=8, window=6)
    cmw.add_request(1)
    for _ in range(30):
        cmw.append([(1, 1)])
    with pytest.raises(ValueError, match="left the window"):
        cmw.truncate(1, 10)
    cmw.truncate(1, 29)                                      # the last token's window is still held
    assert cmw.check() == ""


def test_rows_and_state_slots_run_out_cleanly():
    cm = manager(max_requests=2, state=True)
    cm.add_request(1); cm.add_request(2)
    assert {cm.state_slot(1, 1), cm.state_slot(2, 1)} == {0, 1} and {cm.row_of(1), cm.row_of(2)} == {0, 1}
    with pytest.raises(RuntimeError, match=host.EXHAUSTED_PREFIX):
        cm.add_request(3)
    with pytest.raises(ValueError, match="already exists"):
        cm.add_request(1)
    cm.free_request(1)
    cm.add_request(3)
    assert cm.check() == ""
    with pytest.raises(IndexError):
        cm.num_tokens(99)


def test_fill_meta():
    cm = manager(page=4, pages=16, state=True)
    cm.add_request(5); cm.add_request(6)
    cm.append([(5, 6)])
    cm.append([(5, 3), (6, 1)])
    buf = np.full(200, -7, dtype=np.int32)
    max_ctx = cm.fill_meta([5, 6], [3, 1], buf, 0, 10, 20, 30, [(40, 60, 4), (-1, 70, 0)])
    assert max_ctx == 9
    assert buf[0:4].tolist() == [6, 7, 8, 0]                 # positions
    assert buf[10:14].tolist() == [0, 0, 0, 1]               # which entry a token belongs to
    assert buf[20:23].tolist() == [0, 3, 4] and buf[30:32].tolist() == [9, 1]
    t5, t6 = cm.table(5, 0), cm.table(6, 0)
    assert buf[40:48].tolist() == t5 + [-1] * (4 - len(t5)) + t6 + [-1] * 3
    assert buf[60:64].tolist() == [cm.slot_of(5, 0, 6), cm.slot_of(5, 0, 7), cm.slot_of(5, 0, 8), cm.slot_of(6, 0, 0)]
    assert buf[70:72].tolist() == [cm.state_slot(5, 1), cm.state_slot(6, 1)]
    assert (buf[72:] == -7).all()
    with pytest.raises(IndexError):
        cm.fill_meta([5], [3], buf, 198, 10, 20, 30, [(40, 60, 4), (-1, 70, 0)])


@pytest.mark.parametrize("seed", range(6))
def test_random_lifecycles_against_a_model(seed):
    """Random adds, appends, forks, truncates and frees; a Python model of ownership must agree
    with the manager's tables, and the invariants must hold after every operation."""
    rng = random.Random(seed)
    page, pages = 4, 24
    cm = manager(page=page, pages=pages, max_requests=6)
    tokens = {}                                              # request -> token count
    owners = {}                                              # request -> list of pages (model)
    for step in range(600):
        op = rng.random()
        live = list(tokens)
        if op < 0.15 and len(live) < 6:
            rid = rng.randrange(1000, 2000)
            if rid in tokens:
                continue
            cm.add_request(rid); tokens[rid] = 0; owners[rid] = []
        elif op < 0.65 and live:
            batch = [(r, rng.choice([1, 1, 2, 5, 9])) for r in rng.sample(live, rng.randint(1, len(live)))]
            try:
                copies = cm.append(batch)
            except RuntimeError:
                assert [cm.num_tokens(r) for r, _ in batch] == [tokens[r] for r, _ in batch]
                victim = max(live, key=lambda r: tokens[r])
                cm.free_request(victim); del tokens[victim]; del owners[victim]
                continue
            for r, n in batch:
                tokens[r] += n
                owners[r] = cm.table(r, 0)
            for g, src, dst in copies:
                assert src != dst and cm.refcount(0, dst) == 1
        elif op < 0.75 and live and len(live) < 6:
            parent = rng.choice(live)
            child = rng.randrange(2000, 3000)
            if child in tokens:
                continue
            at = rng.randint(0, tokens[parent])
            cm.fork(parent, child, at)
            tokens[child] = at; owners[child] = cm.table(child, 0)
            assert owners[child] == owners[parent][:(at + page - 1) // page]
        elif op < 0.85 and live:
            r = rng.choice(live)
            n = rng.randint(0, tokens[r])
            cm.truncate(r, n); tokens[r] = n; owners[r] = cm.table(r, 0)
        elif live:
            r = rng.choice(live)
            cm.free_request(r); del tokens[r]; del owners[r]
        assert cm.check() == "", (step, cm.check())
        held = {}
        for r, pgs in owners.items():
            assert cm.num_tokens(r) == tokens[r] and len(pgs) == (tokens[r] + page - 1) // page
            for p in pgs:
                held[p] = held.get(p, 0) + 1
        assert all(cm.refcount(0, p) == c for p, c in held.items())       # held exactly as often as counted
        assert cm.free_count(0) + len(held) == pages                      # nothing lost, nothing twice
    for r in list(tokens):
        cm.free_request(r)
    assert cm.free_count(0) == pages and cm.check() == ""
