"""Generation through the Python entry point and the command line: greedy tokens equal the plain
implementation's, sampling follows the plain sampler, preempted requests repeat nothing."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers as H
import plain_model as pm

pytestmark = pytest.mark.gpu


def plain_greedy(folder, prompt, n, stops=()):
    cfg, w = pm.load_model_folder(folder)
    seq, out = list(prompt), []
    for _ in range(n):
        t = pm.argmax_token(pm.decoder_forward(cfg, w, seq)[-1])
        if t in stops:
            break
        seq.append(t); out.append(t)
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return {w: H.make_folder(root, w) for w in ("A", "B")}


@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_float32_equals_plain(folders, which):
    from aien_sovereign_core_mv_b200.engine.generate import Generator, generate, generate_tokens
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d = folders[which]
    lens = [7, 13, 29] if which == "A" else [1, 17, 40, 63]
    prompts = [H.tokens_for(which, n, 900 + n) for n in lens]
    n_new = 8 if which == "A" else 12
    want = [plain_greedy(d, p, n_new) for p in prompts]
    eng = H.engine_for(d, "float32", H.PAGE_SIZE[which], 512, prefill_chunk_size=16, max_prefill_tokens=32)
    got = generate(eng, prompts, SamplingParams(temperature=0.0, max_tokens=n_new, stop_token_ids=[]))
    assert got == want
    assert eng.cache_state()["requests"] == 0 and eng.cache_state()["check"] == ""
    assert generate_tokens(eng, 5, prompts[1], n_new, 0.0, []) == want[1]          # the reference's signature
    # the model's own stop ids end a request; the stop id is not emitted
    stop = want[0][3]
    res = Generator(eng).generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=n_new, stop_token_ids=[stop]))
    assert res[0].tokens == want[0][:want[0].index(stop)] and res[0].finish_reason == "stop"


def test_greedy_generation_bfloat16_follows_its_own_logits(folders):
    """bfloat16 may pick another token where two logits are close; along its own path every chosen
    token must be the argmax of the engine's logits for that path, recomputed whole."""
    from aien_sovereign_core_mv_b200.engine.generate import generate
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d = folders["B"]
    prompts = [H.tokens_for("B", n, 300 + n) for n in (5, 31, 64)]
    eng = H.engine_for(d, "bfloat16", 8, 512)
    got = generate(eng, prompts, SamplingParams(temperature=0.0, max_tokens=20, stop_token_ids=[]))
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert len(g) == 20
        ref = H.plain_logits(d, p + g)
        for j, tok in enumerate(g):
            row = ref[len(p) + j - 1]
            assert row[tok] >= row.max() - H.BF16_TOL * 2 * np.abs(row).max(), (i, j)


def test_sampling_through_the_entry_point_matches_the_plain_sampler(folders):
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams, philox_uniform
    d = folders["A"]
    cfg, w = pm.load_model_folder(d)
    prompts = [H.tokens_for("A", n, 700 + n) for n in (17, 40)]
    params = [SamplingParams(temperature=0.7, top_p=0.95, top_k=0, max_tokens=12, stop_token_ids=[], seed=11),
              SamplingParams(temperature=1.1, top_p=0.8, top_k=20, max_tokens=12, stop_token_ids=[], seed=12)]
    eng = H.engine_for(d, "float32", 16, 256)
    res = Generator(eng).generate(prompts, params, request_ids=[41, 42])
    again = Generator(eng).generate(prompts[::-1], params[::-1], request_ids=[42, 41])      # other batch order: same draws
    assert [r.tokens for r in res] == [r.tokens for r in again[::-1]]
    for rid, p, sp, r in zip([41, 42], prompts, params, res):
        seq = list(p)
        for tok in r.tokens:
            logits = pm.decoder_forward(cfg, w, seq)[-1]
            u = philox_uniform(sp.seed, rid, len(seq))
            kept, _ = pm.kept_set(logits, sp.temperature, sp.top_p, sp.top_k)
            assert tok in kept
            # the engine's float32 logits differ from the plain ones by up to FP32_TOL: only a draw on an edge may move
            assert pm.sample_token(logits, sp.temperature, sp.top_p, sp.top_k, u) == tok or \
                H.knife_edge(logits, sp.temperature, sp.top_p, sp.top_k, u, eps=20 * H.FP32_TOL), (rid, len(seq))
            seq.append(tok)
        assert len(r.tokens) == 12 and len(set(r.tokens)) > 1


def test_preemption_repeats_nothing(folders):
    """A pool too small for both requests to finish: one is preempted and recomputed; both get
    exactly the tokens they get alone."""
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d = folders["A"]
    prompts = [H.tokens_for("A", 20, 1), H.tokens_for("A", 20, 2)]
    want = [plain_greedy(d, p, 30) for p in prompts]
    eng = H.engine_for(d, "float32", 16, 80, watermark_blocks=0)             # 5 pages of 16
    gen = Generator(eng)
    sp = SamplingParams(temperature=0.0, max_tokens=30, stop_token_ids=[])
    res = gen.generate(prompts, sp, request_ids=[1, 2])
    assert [r.tokens for r in res] == want
    assert sum(r.preemptions for r in res) >= 1
    assert eng.cache_state()["free_pages"] == [5]


def test_fork_through_the_generator(folders):
    """A request branches after a few tokens: the greedy child on the shared pages repeats the
    parent's continuation, a sampling child goes its own way, and the parent is not disturbed."""
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d = folders["A"]
    prompt = H.tokens_for("A", 21, 77)                       # ends inside a page: the tail page is copied on write
    want = plain_greedy(d, prompt, 14)
    eng = H.engine_for(d, "float32", 16, 512)
    gen = Generator(eng)
    gen.submit(1, prompt, SamplingParams(temperature=0.0, max_tokens=14, stop_token_ids=[]))
    done = {}
    while len(gen.scheduler.record(1).generated) < 5:
        for r in gen.step():
            done[r.request_id] = r
    made = len(gen.scheduler.record(1).generated)
    gen.fork(1, 2, SamplingParams(temperature=0.0, max_tokens=14 - made, stop_token_ids=[]))
    gen.fork(1, 3, SamplingParams(temperature=1.3, top_p=1.0, top_k=0, max_tokens=6, stop_token_ids=[], seed=5))
    done.update(gen.run())
    assert done[1].tokens == want and done[2].tokens == want[made:]
    assert len(done[3].tokens) == 6 and done[3].tokens != want[made:made + 6]
    assert eng.cache_state()["requests"] == 0 and eng.cache_state()["check"] == ""


def test_overlapped_steps_equal_step_by_step(folders):
    """Generation with steps that overlap (the tokens of step n reach the host while step n+1
    runs) against the step-by-step loop: same tokens and reasons, with stop ids met at different
    places, different lengths, sampling, and a pool small enough to preempt."""
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d = folders["A"]
    prompts = [H.tokens_for("A", n, 40 + n) for n in (9, 23, 31, 5)]
    free_run = [plain_greedy(d, p, 12) for p in prompts[:3]]
    params = [SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[free_run[0][4]]),           # stops early
              SamplingParams(temperature=0.0, max_tokens=7, stop_token_ids=[free_run[1][6]]),            # the stop id would be the last token
              SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[]),
              SamplingParams(temperature=0.9, top_p=0.9, top_k=30, max_tokens=15, stop_token_ids=[], seed=3)]
    out = {}
    for overlap in (False, True):
        eng = H.engine_for(d, "float32", 16, 96, watermark_blocks=0, async_scheduling=overlap)       # 6 pages: someone gets preempted
        res = Generator(eng).generate(prompts, params, request_ids=[1, 2, 3, 4])
        out[overlap] = [(r.tokens, r.finish_reason) for r in res]
        assert eng.cache_state()["requests"] == 0 and eng.cache_state()["check"] == ""
    assert out[True] == out[False]
    cut = lambda toks, stop: toks[:toks.index(stop)]
    assert out[True][0] == (cut(free_run[0], free_run[0][4]), "stop") and out[True][1] == (cut(free_run[1], free_run[1][6]), "stop")
    assert out[True][2] == (free_run[2], "length") and len(out[True][3][0]) == 15


def test_command_line(folders, tmp_path):
    d = folders["A"]
    prompt = H.tokens_for("A", 13, 3)
    want = plain_greedy(d, prompt, 6)
    cmd = [os.path.join(H.ROOT, "bin", "aien-b200"), "generate", "--model-dir", d, "--dtype", "float32", "--prompt-ids",
           ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0", "--stop-token-ids", "", "--logprobs", "--json"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["tokens"] == [want]
    # greedy: the log softmax at the maximum, one per token, never positive
    assert len(rec["logprobs"]) == 1 and len(rec["logprobs"][0]) == 6 and all(-20.0 < v <= 0.0 for v in rec["logprobs"][0])
    bad = subprocess.run([cmd[0], "generate", "--model-dir", str(tmp_path), "--prompt-ids", "1"], capture_output=True, text=True, timeout=600)
    assert bad.returncode != 0 and "config.json" in bad.stderr


# ------------------------------------------------------------------ a kernel wait that runs out
def _break_one_step(monkeypatch, K, at_call):
    """Makes the `at_call`-th reading of the wait words report that the streamed product gave up,
    without touching the device: the words themselves stay zero."""
    real = K.wait_error_message
    calls = {"n": 0}

    def fake(words):
        calls["n"] += 1
        return real((0, 7, 0, 0)) if calls["n"] == at_call else real(words)

    monkeypatch.setattr(K, "wait_error_message", fake)
    return calls


def test_a_failed_wait_raises_from_step_and_the_cache_is_rolled_back(folders, monkeypatch):
    from aien_sovereign_core_mv_b200 import kernels as K
    d = folders["A"]
    toks = H.tokens_for("A", 40, 5)
    eng = H.engine_for(d, "float32", 16, 256)
    eng.step([(1, toks[:20], [])])
    eng.check_waits()
    _break_one_step(monkeypatch, K, 1)
    logits = eng.step([(1, toks[20:30], [9]), (2, toks[:5], [4])])
    with pytest.raises(K.KernelError, match="gemv_stream .code 7."):
        eng.check_waits()                                     # the caller looks before it uses the logits
    assert eng.num_tokens(1) == 20 and not eng.has_request(2) and eng.cache_state()["check"] == ""
    again = eng.step([(1, toks[20:30], [9]), (2, toks[:5], [4])]).cpu().numpy()    # the same step, now clean
    eng.check_waits()
    want = H.plain_logits(d, toks[:30])
    H.assert_close(again[0], want[29], H.FP32_TOL, "after the rollback")


@pytest.mark.parametrize("overlap", [False, True])
def test_a_failed_wait_raises_from_generation_and_nothing_is_lost(folders, monkeypatch, overlap):
    """Step by step the failed step is rolled back (cache lengths as before) and planned again; with
    overlapping steps everything that runs is queued again and recomputed from the tokens known so
    far.  Either way the tokens that come out are those of an undisturbed run."""
    from aien_sovereign_core_mv_b200 import kernels as K
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d = folders["B"]
    prompts = [H.tokens_for("B", n, 70 + n) for n in (9, 33, 18)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, stop_token_ids=[])
    eng = H.engine_for(d, "float32", 8, 512, prefill_chunk_size=16, max_prefill_tokens=32, async_scheduling=overlap)
    want = [r.tokens for r in Generator(eng).generate(prompts, sp)]
    gen = Generator(eng)
    for i, p in enumerate(prompts):
        gen.submit(100 + i, p, sp)
    _break_one_step(monkeypatch, K, 4)
    done, raised = {}, 0
    for _ in range(200):
        if not (gen.scheduler.has_work() or gen._inflight is not None):
            break
        held = {r: eng.num_tokens(r) for r in (100, 101, 102) if eng.has_request(r)}
        try:
            for r in gen.advance():
                done[r.request_id] = r
        except K.KernelError as e:
            raised += 1
            assert "gemv_stream" in str(e) and eng.cache_state()["check"] == ""
            if overlap:
                assert eng.cache_state()["requests"] == 0              # all queued again, their pages given back
            else:
                assert {r: eng.num_tokens(r) for r in held} == held    # lengths as before the step
    for r in gen.flush():
        done[r.request_id] = r
    assert raised == 1 and [done[100 + i].tokens for i in range(3)] == want
    assert eng.cache_state()["requests"] == 0 and eng.cache_state()["check"] == ""


def test_prompts_beyond_the_context_limit_are_aborted_and_the_rest_runs(folders):
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d = folders["A"]
    eng = H.engine_for(d, "float32", 16, 1024, max_context=64, prefill_chunk_size=32)
    gen = Generator(eng)
    sp = SamplingParams(temperature=0.0, max_tokens=4, stop_token_ids=[])
    res = gen.generate([H.tokens_for("A", 100, 1), H.tokens_for("A", 12, 2), H.tokens_for("A", 64, 3)], sp)
    assert res[0].finish_reason == "aborted" and "context limit" in res[0].message and res[0].tokens == []
    assert res[2].finish_reason == "aborted"
    assert res[1].finish_reason == "length" and res[1].tokens == plain_greedy(d, H.tokens_for("A", 12, 2), 4)
    assert eng.cache_state()["requests"] == 0 and eng.cache_state()["check"] == ""


@pytest.mark.parametrize("overlap", [False, True])
def test_logprobs_come_back_with_the_tokens(folders, overlap):
    """Greedy: the log softmax of the logits at the chosen token (crates/aien-inference-abi/src/
    tensor.rs:299-318); sampled: ln(p / kept mass).  One per token, also when a stop id ends the
    request (the stop id brings neither a token nor a logprob)."""
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    d = folders["A"]
    cfg, w = pm.load_model_folder(d)
    prompts = [H.tokens_for("A", n, 40 + n) for n in (9, 21)]
    eng = H.engine_for(d, "float32", 16, 256, async_scheduling=overlap)
    params = [SamplingParams(temperature=0.0, max_tokens=6, stop_token_ids=[], logprobs=True),
              SamplingParams(temperature=0.9, top_p=0.7, max_tokens=6, stop_token_ids=[], seed=3, logprobs=True)]
    res = Generator(eng).generate(prompts, params, request_ids=[1, 2])
    plain = Generator(eng).generate(prompts, [SamplingParams(temperature=0.0, max_tokens=6, stop_token_ids=[]), params[1]], request_ids=[1, 2])
    assert plain[0].logprobs is None and plain[0].tokens == res[0].tokens and plain[1].tokens == res[1].tokens
    for r, p, sp in zip(res, prompts, params):
        assert len(r.logprobs) == len(r.tokens) == 6
        seq = list(p)
        for tok, lp in zip(r.tokens, r.logprobs):
            logits = pm.decoder_forward(cfg, w, seq)[-1]
            if sp.greedy:
                want = logits[tok] - logits.max() - np.log(np.exp(logits - logits.max()).sum())
            else:
                kept, probs = pm.kept_set(logits, sp.temperature, sp.top_p, sp.top_k)
                want = np.log(probs[tok] / sum(probs[i] for i in kept))
            assert abs(lp - want) < 2e-3, (r.request_id, len(seq), lp, want)
            seq.append(tok)
    stop = res[0].tokens[3]
    cut = Generator(eng).generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=6, stop_token_ids=[stop], logprobs=True))[0]
    assert cut.tokens == res[0].tokens[:res[0].tokens.index(stop)] and len(cut.logprobs) == len(cut.tokens)
    assert all(abs(a - b) < 1e-5 for a, b in zip(cut.logprobs, res[0].logprobs))
