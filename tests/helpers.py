"""Shared pieces of the tests: tiny configurations, model folders, comparisons.

The tiny configurations differ in every size and option: head counts and groups, head sizes,
widths and vocabularies that are no power of two, number of layers, the norms' eps, rotary
base and scaling, q/k norm, tied or untied head, page size.
"""
import json
import os
import subprocess
import sys

import numpy as np

import plain_model as pm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TINY = {
    # Llama-style: nq*hd == hidden, untied head, no q/k norm
    "A": dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=160, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256,
              hidden_act="silu", eos_token_id=2),
    # Qwen3-style: nq*hd != hidden, tied head, q/k norm
    "B": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=8, num_key_value_heads=2, head_dim=32, intermediate_size=288, vocab_size=512,
              rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512,
              hidden_act="silu", eos_token_id=[1, 2]),
    # odd everything: head size 48, 6 heads in 3 groups, width 72, vocabulary 333, one layer
    "C": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=1, hidden_size=72,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=200, vocab_size=333,
              rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=1024,
              hidden_act="silu", eos_token_id=0),
    # Llama with llama3 rotary scaling, one kv head (multi-query), head size 80
    "D": dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=160,
              num_attention_heads=2, num_key_value_heads=1, head_dim=80, intermediate_size=112, vocab_size=300,
              rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=2048,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64),
              hidden_act="silu", eos_token_id=1),
}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16, "D": 32}
SEED = {"A": 0, "B": 1, "C": 2, "D": 3}

FP32_TOL = 1e-4      # x max|logit| : the float32 engine against the plain implementation
BF16_TOL = 3e-2      # x max|logit| : the bfloat16 engine against the plain implementation


def make_folder(tmp_path, which, seed=None, init_std=None):
    """Write a random model folder with the engine's own writer; returns its path."""
    from aien_sovereign_core_mv_b200 import write_random_model
    d = os.path.join(str(tmp_path), f"tiny{which}")
    write_random_model(d, TINY[which], SEED[which] if seed is None else seed, init_std)
    return d


def plain_logits(model_dir, ids):
    config, weights = pm.load_model_folder(model_dir)
    return pm.decoder_forward(config, weights, ids)


def tokens_for(which, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, TINY[which]["vocab_size"], n)]


def rel_err(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def assert_close(got, want, tol, what=""):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    diff = np.abs(got - want)
    scale = max(np.abs(want).max(), 1e-30)
    if diff.max() > tol * scale:
        idx = np.unravel_index(diff.argmax(), diff.shape)
        rows = np.where(diff.max(axis=-1) > tol * scale)[0] if diff.ndim == 2 else []
        raise AssertionError(
            f"{what}: max|d|={diff.max():.3e} at {idx} (got {got[idx]:.6f}, want {want[idx]:.6f}), "
            f"bound {tol * scale:.3e}; first wrong row {rows[0] if len(rows) else '-'} of {got.shape[0] if got.ndim == 2 else 1}")


def engine_for(model_dir, dtype, page_size, pool_tokens, max_requests=8, max_batch_tokens=None, **kw):
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    ec = EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=pool_tokens, max_requests=max_requests,
                      max_batch_tokens=max_batch_tokens or max(pool_tokens, 64), **kw)
    return Engine.from_folder(model_dir, ec)


def run_steps(engine, steps):
    """steps: list of (entries, end) with entries [(id, tokens, want)].  Returns, per request,
    {position: logits row} collected from the wanted places."""
    out = {}
    held = {}
    for entries, end in steps:
        logits = engine.step(entries).cpu().numpy() if entries else None
        r = 0
        for rid, toks, want in entries:
            base = held.get(rid, 0)
            for w in want:
                out.setdefault(rid, {})[base + w] = logits[r]
                r += 1
            held[rid] = base + len(toks)
        for rid in end:
            engine.end_request(rid)
            held.pop(rid, None)
    return out


def run_trace(model_dir, dtype, out_dir, max_tokens, steps, page_size=None, timeout=900):
    """Drive bin/trace_run with `steps` (list of dicts); returns {step: array [wanted, vocab]}."""
    cmd = [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run answered {line!r} to step {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for s in steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if os.path.exists(path):
            out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(-1, vocab)
    return out


def knife_edge(logits, temperature, top_p, top_k, u, eps=2e-6):
    """Whether the draw `u` for these logits sits on an edge that float32 exponentials may legitimately
    move: u times the kept mass within `eps` (of the mass) of a boundary between two kept tokens, or a
    cumulative mass in the nucleus order within `eps` of top_p (one token more or fewer is kept).
    Only such a draw may differ between the device sampler and the plain float64 one."""
    kept, probs = pm.kept_set(logits, temperature, top_p, top_k)
    mass = sum(probs[i] for i in kept)
    cum = 0.0
    for i in kept:
        cum += probs[i]
        if abs(cum - u * mass) <= eps * mass:
            return True
    if 0.0 < top_p < 1.0:
        allowed = [i for i in range(len(probs)) if probs[i] > 0.0]
        order = sorted(allowed, key=lambda i: (-probs[i], i))
        cum = 0.0
        for i in order:
            cum += probs[i]
            if abs(cum - top_p) <= eps:
                return True
            if cum > top_p + eps:
                break
    return False
