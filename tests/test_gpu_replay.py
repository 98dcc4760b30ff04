"""bin/trace_run as a user drives it: a subprocess fed JSON steps, logits compared with the plain
implementation.  The same requests whole, with the last 32 tokens one by one, in portions of
changing size, and mixed so that pages are reused; in float32 and bfloat16."""
import os

import numpy as np
import pytest

import helpers as H
from test_gpu_engine import mixed_steps

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    root = tmp_path_factory.mktemp("replay")
    out = {}
    for which in ("A", "B"):
        d = H.make_folder(root, which)
        lens = [70, 33, 100, 5, 64, 129]
        reqs = {f"r{i}": H.tokens_for(which, n, 40 + i) for i, n in enumerate(lens)}
        out[which] = (d, reqs, {k: H.plain_logits(d, v) for k, v in reqs.items()})
    return root, out


def to_trace(steps):
    return [{"step": i, "entries": [{"id": rid, "tokens": [int(t) for t in toks], "want": list(want)} for rid, toks, want in entries],
             "end": list(end)} for i, (entries, end) in enumerate(steps)]


def collect(trace, outputs):
    got, held = {}, {}
    for s in trace:
        r = 0
        for e in s["entries"]:
            base = held.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = outputs[s["step"]][r]
                r += 1
            held[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            held.pop(rid, None)
    return got


@pytest.mark.parametrize("dtype,tol", [("float32", H.FP32_TOL), ("bfloat16", H.BF16_TOL)])
@pytest.mark.parametrize("which", ["A", "B"])
def test_trace_replay_every_cutting(folder, which, dtype, tol, tmp_path):
    root, models = folder
    d, reqs, want = models[which]
    rng = np.random.default_rng(5)
    steps = []
    for rid, toks in list(reqs.items())[:3]:                                   # whole
        steps.append(([(rid + "w", toks, range(len(toks)))], [rid + "w"]))
    rid, toks = "r2", reqs["r2"]                                                 # last 32 one by one
    steps.append(([(rid + "d", toks[:-32], [len(toks) - 33])], []))
    steps += [([(rid + "d", [t], [0])], []) for t in toks[-32:]]
    steps[-1] = (steps[-1][0], [rid + "d"])
    rid, toks = "r5", reqs["r5"]                                                 # portions of changing size
    at, sizes, k = 0, [7, 2, 13, 3, 2, 29, 5, 2, 16, 17], 0
    while at < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - at)
        steps.append(([(rid + "p", toks[at:at + n], range(n))], []))
        at += n; k += 1
    steps[-1] = (steps[-1][0], [rid + "p"])
    steps += mixed_steps({k + "m": v for k, v in reqs.items()}, rng)            # mixed, pages reused
    trace = to_trace(steps)
    pool = sum(sorted(((len(v) + 63) // 64) * 64 for v in reqs.values())[-4:])
    outputs = H.run_trace(d, dtype, str(tmp_path / "out"), pool, trace, page_size=H.PAGE_SIZE[which])
    got = collect(trace, outputs)
    assert len(got) == 3 + 1 + 1 + len(reqs)
    for rid, rows in got.items():
        pos = sorted(rows)
        H.assert_close(np.stack([rows[p] for p in pos]), want[rid[:-1]][pos], tol, f"{which} {dtype} trace request {rid}")
    wanted_steps = [s["step"] for s in trace if any(e["want"] for e in s["entries"])]
    assert sorted(outputs) == wanted_steps


def test_trace_replay_default_page_size_and_empty_want(folder, tmp_path):
    root, models = folder
    d, reqs, want = models["A"]
    toks = reqs["r0"]
    trace = [
        {"step": 0, "entries": [{"id": 1, "tokens": toks[:40], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": 1, "tokens": toks[40:], "want": [len(toks) - 41]}, {"id": "b", "tokens": reqs["r3"], "want": [4]}], "end": [1]},
        {"step": 2, "entries": [], "end": ["b"]},
    ]
    out = H.run_trace(d, "float32", str(tmp_path / "o"), 192, trace)
    assert sorted(out) == [1] and out[1].shape == (2, 256)
    H.assert_close(out[1][0], want["r0"][-1], H.FP32_TOL, "last row")
    H.assert_close(out[1][1], want["r3"][4], H.FP32_TOL, "second request")
