"""The engine against the plain implementation under every way of cutting the work, in float32
and in bfloat16: whole requests; most in one step and the last 32 tokens one by one; portions
of changing size down to two tokens; mixed batches with so few pages that they are reused;
long decoding; the first tokens; fork with copy-on-write."""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

DTYPES = [("float32", H.FP32_TOL), ("bfloat16", H.BF16_TOL)]
LENGTHS = {"A": [7, 13, 29, 150], "B": [1, 17, 40, 63, 131], "C": [5, 33, 90], "D": [3, 70, 45]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for which in H.TINY:
        d = H.make_folder(root, which)
        reqs = {i + 1: H.tokens_for(which, n, 1000 + 17 * i + n) for i, n in enumerate(LENGTHS[which])}
        want = {rid: H.plain_logits(d, toks) for rid, toks in reqs.items()}
        out[which] = (d, reqs, want)
    return out


def check(collected, want, tol, what):
    assert collected, f"{what}: nothing was collected"
    for rid, rows in collected.items():
        pos = sorted(rows)
        got = np.stack([rows[p] for p in pos])
        H.assert_close(got, want[rid][pos], tol, f"{what} request {rid} (positions {pos[0]}..{pos[-1]})")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", list(H.TINY))
def test_whole_requests(models, which, dtype, tol):
    d, reqs, want = models[which]
    eng = H.engine_for(d, dtype, H.PAGE_SIZE[which], 256)
    steps = [([(rid, toks, list(range(len(toks))))], [rid]) for rid, toks in reqs.items()]
    check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} whole")
    assert eng.cache_state()["check"] == "" and eng.cache_state()["requests"] == 0


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_last_32_one_by_one(models, which, dtype, tol):
    d, reqs, want = models[which]
    eng = H.engine_for(d, dtype, H.PAGE_SIZE[which], 256)
    rid = max(reqs, key=lambda r: len(reqs[r]))
    toks = reqs[rid]
    cut = len(toks) - 32
    steps = [([(rid, toks[:cut], [cut - 1])], [])]
    steps += [([(rid, [toks[i]], [0])], []) for i in range(cut, len(toks))]
    check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} last-32")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "D"])
def test_changing_portions(models, which, dtype, tol):
    d, reqs, want = models[which]
    eng = H.engine_for(d, dtype, H.PAGE_SIZE[which], 256)
    sizes = [7, 2, 13, 3, 2, 29, 5, 2, 16, 17, 1, 8]
    for rid, toks in reqs.items():
        steps, at, k = [], 0, rid
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            steps.append(([(rid, toks[at:at + n], list(range(n)))], []))
            at += n
            k += 1
        steps[-1] = (steps[-1][0], [rid])
        check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} portions request {rid}")


def mixed_steps(reqs, rng, max_live=4):
    """Up to `max_live` requests at a time: portions of some beside single tokens of others; a
    request may sit a step out; finished ones are ended and the next one starts."""
    waiting = list(reqs)
    live, done_at = {}, {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            toks, at = reqs[rid], live[rid]
            if rng.random() < 0.2 and len(live) > 1:
                continue                                   # left out of this step
            left = len(toks) - at
            mode = rng.integers(0, 3)
            n = 1 if mode == 0 else (2 if mode == 1 else int(rng.integers(2, 24)))
            n = min(n, left)
            entries.append((rid, toks[at:at + n], list(range(n))))
            live[rid] = at + n
            if live[rid] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append((entries, end))
    return steps


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_mixed_with_page_reuse(models, which, dtype, tol):
    d, _, _ = models[which]
    rng = np.random.default_rng(7)
    lens = [int(x) for x in rng.integers(3, 120, 9)]
    reqs = {i + 1: H.tokens_for(which, n, 500 + i) for i, n in enumerate(lens)}
    want = {rid: H.plain_logits(d, toks) for rid, toks in reqs.items()}
    ps = H.PAGE_SIZE[which]
    pool = sum(sorted(((n + 63) // 64) * 64 for n in lens)[-4:])          # four largest, each rounded to 64
    eng = H.engine_for(d, dtype, ps, pool)
    steps = mixed_steps(reqs, rng)
    assert max(len(e) for e, _ in steps) >= 3
    check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} mixed")
    st = eng.cache_state()
    assert st["check"] == "" and st["requests"] == 0
    assert st["metrics"]["pages_allocated"] > pool // ps, "the pool was never reused"


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_long_decoding(models, dtype, tol):
    which = "B"
    d, _, _ = models[which]
    toks = H.tokens_for(which, 400, 99)
    want = H.plain_logits(d, toks)
    eng = H.engine_for(d, dtype, H.PAGE_SIZE[which], 448)
    steps = [([(1, toks[:16], [15])], [])] + [([(1, [t], [0])], []) for t in toks[16:]]
    check(H.run_steps(eng, steps), {1: want}, tol, f"{which} {dtype} long decode")


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_first_tokens(models, dtype, tol):
    """Position 0 alone, then 1, 2, 3: the start of a sequence and of its first page."""
    for which in ("A", "B"):
        d, reqs, want = models[which]
        rid = 2
        toks = reqs[rid][:6]
        eng = H.engine_for(d, dtype, H.PAGE_SIZE[which], 64)
        steps = [([(rid, [t], [0])], []) for t in toks]
        check(H.run_steps(eng, steps), want, tol, f"{which} {dtype} first tokens")


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_batch_row_equals_single(models, dtype, tol):
    """A request's logits do not depend on what else is in the batch."""
    which = "B"
    d, reqs, want = models[which]
    eng = H.engine_for(d, dtype, H.PAGE_SIZE[which], 512)
    ids = [r for r in reqs if len(reqs[r]) >= 17][:3]
    steps = [([(r, reqs[r][:16], [15]) for r in ids], [])]
    steps.append(([(r, [reqs[r][16]], [0]) for r in ids], ids))
    together = H.run_steps(eng, steps)
    check(together, want, tol, "batched")
    alone = {}
    for r in ids:
        alone.update(H.run_steps(eng, [([(r, reqs[r][:16], [15])], []), ([(r, [reqs[r][16]], [0])], [r])]))
    bound = 1e-5 if dtype == "float32" else 2e-2
    for r in ids:
        for p in together[r]:
            assert H.rel_err(together[r][p], alone[r][p]) <= bound


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_fork_copy_on_write(models, dtype, tol):
    """Fork at token 20 (inside a page): both go on with different tokens; neither sees the other."""
    which = "B"
    d, reqs, _ = models[which]
    base = reqs[4][:40]
    child_tail = H.tokens_for(which, 12, 4242)
    want_parent = H.plain_logits(d, base)
    want_child = H.plain_logits(d, base[:20] + child_tail)
    eng = H.engine_for(d, dtype, H.PAGE_SIZE[which], 256)
    got = H.run_steps(eng, [([(1, base[:30], list(range(30)))], [])])
    eng.fork(1, 2, 20)
    assert eng.num_tokens(2) == 20
    got2 = H.run_steps(eng, [([(2, child_tail[:5], list(range(5))), (1, base[30:33], [0, 1, 2])], [])])
    got3 = H.run_steps(eng, [([(1, base[33:], list(range(7))), (2, child_tail[5:], list(range(7)))], [])])
    H.assert_close(np.stack([got[1][p] for p in range(30)]), want_parent[:30], tol, "parent before fork")
    H.assert_close(np.stack([got2[2][p] for p in range(5)]), want_child[20:25], tol, "child after fork")
    H.assert_close(np.stack([got2[1][p] for p in range(3)]), want_parent[30:33], tol, "parent after fork")
    H.assert_close(np.stack([got3[1][p] for p in range(7)]), want_parent[33:40], tol, "parent later")
    H.assert_close(np.stack([got3[2][p] for p in range(7)]), want_child[25:32], tol, "child later")
    assert eng.cache_state()["metrics"]["cow_copies"] >= 1
    eng.end_request(1)
    eng.end_request(2)
    assert eng.cache_state()["check"] == ""


def test_step_refusals(models):
    d, reqs, _ = models["A"]
    eng = H.engine_for(d, "float32", 16, 64, max_batch_tokens=128)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.step([(1, [256], [0])])
    with pytest.raises(ValueError, match="wanted place"):
        eng.step([(1, [1, 2], [2])])
    with pytest.raises(RuntimeError, match="KV pool exhausted"):
        eng.step([(1, list(range(65)), [])])
    assert eng.cache_state()["requests"] == 0 and eng.cache_state()["free_pages"] == [4]
    eng.step([(1, list(range(64)), [])])          # exact fit works after the refusal
    with pytest.raises(RuntimeError, match="KV pool exhausted"):
        eng.step([(1, [5], [0])])
    assert eng.num_tokens(1) == 64
    eng.end_request(1)
    assert eng.cache_state()["free_pages"] == [4]


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_steps_of_a_repeated_shape_reissue_recorded_launches(models, dtype, tol):
    """Mixed steps whose host numbers repeat (two decoded tokens beside a five-token portion, six
    times, contexts growing, pages changing) run once through the Python parts and afterwards as
    the recorded launches: the same bits as an engine that records nothing, and the plain logits."""
    d, reqs, want = models["A"]
    a = H.engine_for(d, dtype, H.PAGE_SIZE["A"], 256)
    b = H.engine_for(d, dtype, H.PAGE_SIZE["A"], 256, replay_steps=False)
    t1, t2, t3 = reqs[4][:40], reqs[3][:29], reqs[4][:150]
    steps = [([(1, t1[:20], []), (2, t2[:10], []), (3, t3[:100], [])], [])]
    for k in range(6):
        steps.append(([(1, [t1[20 + k]], [0]), (2, [t2[10 + k]], [0]), (3, t3[100 + 5 * k:105 + 5 * k], [4])], []))
    steps.append(([(3, t3[130:], list(range(20)))], [1, 2, 3]))
    got_a, got_b = H.run_steps(a, steps), H.run_steps(b, steps)
    assert a.steps_replayed >= 4 and b.steps_replayed == 0      # one of the six crosses into a second key chunk
    for rid in got_a:
        for p in got_a[rid]:
            assert np.array_equal(got_a[rid][p], got_b[rid][p]), f"request {rid} position {p}: replayed launches differ"
    check(got_a, {1: want[4], 2: want[3], 3: want[4]}, tol, f"A {dtype} repeated shapes")
    assert a.cache_state()["check"] == "" and a.cache_state()["requests"] == 0
