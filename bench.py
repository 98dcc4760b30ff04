#!/usr/bin/env python3
"""Headline measurement: decode tokens per second of the Qwen3-8B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--prompt-len L] [--prefill-tokens T] [--layers N] [--workload decode|llama3_8b|serving|mixed_step]

A step is one decode step of a batch of requests that each hold a 1,024-token prompt (context
limit 4,096, pages of 16 tokens), random bfloat16 weights, synthetic uniform token ids.  One JSON
line is printed:

* ``value``      decoded tokens per second at the default batch, timed on the device with CUDA
                 events around exactly K steps after W warm-up steps;
* ``e2e``        the same through the Python entry point (scheduler, sampling, token ids from and
                 to the host every step);
* ``prefill``    one 2,048-token prompt in one step: tokens per second and the fraction of the
                 bfloat16 tensor peak its flops reach;
* ``roofline``   bytes a decode step must read (every weight once, the cache of the live
                 requests) per second against the measured copy bandwidth;
* ``points``     decode tokens per second at batch 1 and 64.

Peaks come from ``MEASURED_PEAKS.json`` beside this file when present, else from the fallback
measured earlier on the same pool (6.65 TB/s, 1.59 PFLOP/s).  The weights of one step (15 GB) are
far larger than the 126 MB L2, so consecutive steps cannot be served from cache.  Every decode
run first fills its requests' cache by prefill, pauses 0.3 s and then takes its W warm-up steps: the
fill runs at the power cap and leaves the SM clock low for some 70 ms, which 20 timed steps straight
after it would measure instead of decoding (steps of 4.2 ms that settle at 3.5 ms).
``--workload llama3_8b`` prints the same line for the Llama-3-8B shape with 16 requests decoding at
contexts that end at 8,192 tokens (the cache, 17 GB a step, outweighs the weights) and a 2,048-token
prefill; ``--workload serving`` runs continuous batching of 32 requests on the Qwen3-4B shape and adds
the distribution of step times.  Every line carries ``wait_errors``: how many of the kernels' bounded
waits ran out during the timed regions (0, or the number is void).
``--impl reference`` reports that the reference (a Rust workspace) cannot be installed here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960,
    hidden_act="silu", attention_bias=False, eos_token_id=151645,
)
LLAMA3_8B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=32, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
    rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=8192,
    hidden_act="silu", attention_bias=False, eos_token_id=128001,
)
PAGE, PREFILL_TOKENS = 16, 2048
SETTLE_S = 0.3           # pause between a cache fill (a prefill at the power cap) and the decode steps after it
# prompt_len None: as long as lets the timed steps end exactly at `context` tokens
WORKLOADS = {
    "decode": dict(cfg=QWEN3_8B, label="Qwen3-8B shape, random weights", prompt_len=1024, context=4096, batch=8, seed=2, points=(1, 64)),
    "llama3_8b": dict(cfg=LLAMA3_8B, label="Llama-3-8B shape, random weights", prompt_len=None, context=8192, batch=16, seed=4, points=()),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    if os.path.exists(path):
        try:
            with open(path) as f:
                p = json.load(f)
            hbm = float(p.get("hbm_gbs", hbm))
            tf = float(p.get("bf16_tflops", tf))
            src = "measured"
        except Exception:
            pass
    return hbm, tf, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, layers_run):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Q = cfg["num_attention_heads"] * cfg["head_dim"]
    KV = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (Q + 2 * KV) * H + H * Q + 2 * I * H + H * I
    linear_params = per_layer * layers_run + V * H                       # matrices a decode step reads
    norm_params = layers_run * (2 * H + (2 * cfg["head_dim"] if cfg["architectures"][0] == "Qwen3ForCausalLM" else 0)) + H
    kv_bytes_per_token = 2 * KV * 2 * layers_run
    return dict(per_layer=per_layer, linear_params=linear_params, weight_bytes=2 * (linear_params + norm_params),
                kv_bytes_per_token=kv_bytes_per_token, Q=Q, KV=KV)


QWEN3_4B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=2560,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=9728, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960,
    hidden_act="silu", attention_bias=False, eos_token_id=151645,
)


def _dist(ms):
    """p50 / p90 / max of a list of step times in ms."""
    if not ms:
        return None
    v = sorted(ms)
    pick = lambda q: v[min(len(v) - 1, int(q * len(v)))]
    return {"n": len(v), "p50_ms": round(pick(0.5), 3), "p90_ms": round(pick(0.9), 3), "max_ms": round(v[-1], 3),
            "mean_ms": round(sum(v) / len(v), 3)}


def serving_workload(align_step_tokens: int = 0) -> int:
    """Continuous batching through the public entry point: 32 requests with uniform-random prompt
    lengths in [64, 4096], prompts cut into portions under a 512-token budget, 256 greedy tokens
    each (Qwen3-4B shape, random bfloat16 weights, seed 3).  Wall-clock time of the whole job, and
    the distribution of step times: the time from one turn of the generation loop to the next,
    which with overlapping steps is what a step adds to the job; steps that carry a portion of a
    prompt apart from steps that only decode."""
    import numpy as np
    import torch
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    from aien_sovereign_core_mv_b200 import kernels as K
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams
    ec = EngineConfig(dtype="bfloat16", page_size=16, max_cache_tokens=32 * 4400, max_requests=32, max_batch_tokens=1024,
                      max_context=8192, max_batch_size=32, max_prefill_tokens=512, prefill_chunk_size=512,
                      align_step_tokens=align_step_tokens)
    engine = Engine.from_config(QWEN3_4B, seed=3, engine_config=ec, init_std=0.02, device_init=True)
    rng = np.random.default_rng(3)
    lens = rng.integers(64, 4097, 32)
    prompts = [rng.integers(0, QWEN3_4B["vocab_size"], int(n)).tolist() for n in lens]
    sp = SamplingParams(temperature=0.0, max_tokens=256, stop_token_ids=[])

    def job(first_id, timed):
        gen = Generator(engine)
        for i, p in enumerate(prompts):
            gen.submit(first_id + i, p, sp)
        torch.cuda.synchronize()
        done, kinds, stamps = {}, [], [time.perf_counter()]
        while gen.scheduler.has_work() or gen._inflight is not None:
            before = gen.steps
            for r in gen.advance():
                done[r.request_id] = r
            if gen.steps > before:
                kinds.append(gen.last_plan)
                stamps.append(time.perf_counter())
        torch.cuda.synchronize()
        stamps[-1] = time.perf_counter()
        return gen, done, kinds, stamps

    job(10000, False)                     # untimed: every step shape is met once (recorded launches, captured graphs)
    K.read_wait_errors()
    sampler = ClockSampler()
    sampler.start()
    gen, done, kinds, stamps = job(100, True)
    clocks = sampler.stop()
    wait_errors = sum(1 for w in K.read_wait_errors() if w != 0)
    dt = stamps[-1] - stamps[0]
    step_ms = [(b - a) * 1e3 for a, b in zip(stamps, stamps[1:])]
    with_prompt = [t for t, k in zip(step_ms, kinds) if k[0] > 0]
    decode_only = [t for t, k in zip(step_ms, kinds) if k[0] == 0]
    m = gen.scheduler.metrics()
    new = sum(len(r.tokens) for r in done.values())
    print(json.dumps({
        "metric": "serving_generated_tokens_per_s", "value": round(new / dt, 1), "unit": "tokens/s", "n_gpus": 1,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "total_tokens_per_s": round((int(lens.sum()) + new) / dt, 1), "seconds": round(dt, 3), "steps": int(m["steps"]),
        "preemptions": int(m["preemptions"]), "requests": len(done), "prompt_tokens": int(lens.sum()), "generated_tokens": new,
        "step_ms": {"all": _dist(step_ms), "with_prompt_portion": _dist(with_prompt), "decode_only": _dist(decode_only)},
        "clocks": clocks, "wait_errors": int(wait_errors),
        "config": {"model": "Qwen3-4B shape, random weights", "layers": 36, "hidden": 2560, "heads": 32, "kv_heads": 8, "head_dim": 128,
                   "intermediate": 9728, "vocab": 151936, "requests": 32, "prompt_len": "uniform 64..4096",
                   "prefill_budget": 512, "align_step_tokens": align_step_tokens, "new_tokens": 256, "context": 8192, "page_size": 16, "seed": 3,
                   "timing": "second run of the job; the first, untimed, meets every step shape once"},
    }))
    return 0


def mixed_step_workload() -> int:
    """One step of the kind a chunked-prefill server runs all day, timed alone on the device: a
    512-token portion of a prompt at offset 2,048 beside 24 requests that decode one token each at
    contexts of 500 tokens (Qwen3-4B shape, random bfloat16 weights, seed 3).  The timed step lies
    between cudaProfilerStart and cudaProfilerStop, so `ncu --profile-from-start off` lists its
    launches and nothing else."""
    import torch
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    from aien_sovereign_core_mv_b200 import kernels as K
    ec = EngineConfig(dtype="bfloat16", page_size=16, max_cache_tokens=40 * 1024, max_requests=32, max_batch_tokens=1024,
                      max_context=8192, max_batch_size=32, max_prefill_tokens=512, prefill_chunk_size=512)
    eng = Engine.from_config(QWEN3_4B, seed=3, engine_config=ec, init_std=0.02, device_init=True)
    V = QWEN3_4B["vocab_size"]
    toks = lambda n, s: [(7 * i + s) % V for i in range(n)]
    decodes, portion, offset, ctx = 24, 512, 1024, 500
    for r in range(0, decodes, 2):
        eng.step([(r, toks(ctx, r), []), (r + 1, toks(ctx, r + 1), [])])
    for k in range(offset // portion):
        eng.step([(500, toks(portion, k), [])])

    def mixed(s):
        return eng.step([(r, [s + r], [0]) for r in range(decodes)] + [(500, toks(portion, 9 + s), [portion - 1])])

    times = []
    for rep in range(5):            # every repetition moves the portion 512 tokens on (the first writes the launches
        torch.cuda.synchronize()    # down, the others re-issue them); the third, at offset 2,048, is the profiled one
        if rep == 2:
            torch.cuda.profiler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        mixed(rep)
        e1.record()
        torch.cuda.synchronize()
        if rep == 2:
            torch.cuda.profiler.stop()
        times.append(round(e0.elapsed_time(e1), 3))
    eng.check_waits()
    wait_errors = sum(1 for w in K.read_wait_errors() if w != 0)
    print(json.dumps({
        "metric": "mixed_step_ms", "value": times[2], "unit": "ms", "n_gpus": 1, "higher_is_better": False, "dtype": "bf16",
        "data": "synthetic", "impl": "ours", "steps_ms": times, "wait_errors": wait_errors,
        "config": {"model": "Qwen3-4B shape, random weights", "layers": 36, "hidden": 2560, "heads": 32, "kv_heads": 8, "head_dim": 128,
                   "intermediate": 9728, "vocab": 151936, "portion_tokens": portion, "portion_offset": "1024 + 512 per step; value: the step at 2048",
                   "decoding_requests": decodes, "decode_context": ctx, "page_size": 16, "seed": 3},
    }))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=0, help="requests decoding together (0: the workload's own: 8, or 16 for llama3_8b)")
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (0 = all)")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="decode workload: tokens each request holds before the timed steps (default 1,024); the context limit "
                         "grows with it, and the points at batch 1 and 64 are left out")
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help="length of the prompt whose one-step prefill is timed (default 2,048); another length leaves out the points")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature of the end-to-end run (0: greedy)")
    ap.add_argument("--top-p", type=float, default=1.0, help="nucleus of the end-to-end run")
    ap.add_argument("--top-k", type=int, default=0, help="top-k of the end-to-end run")
    ap.add_argument("--align-step-tokens", type=int, default=0,
                    help="serving workload: the scheduler cuts portions so that a step's tokens fill whole tiles of this many rows")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "llama3_8b", "serving", "mixed_step"],
                    help="decode: the headline decode-step measurement (Qwen3-8B shape, 1,024-token prompts); llama3_8b: the same "
                         "line for the Llama-3-8B shape, 16 requests at contexts ending at 8,192 tokens; serving: continuous batching "
                         "of 32 requests on the Qwen3-4B shape (prompts of 64..4096 tokens, portions of 512, 256 new tokens each); "
                         "mixed_step: one step of a 512-token portion beside 24 decoding requests on that shape, timed alone")
    ap.add_argument("--fill", default="prefill", choices=["prefill", "cache"],
                    help="how requests get their prompt: real prefill, or (development only) cache pages "
                         "filled with random keys/values without running the model")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace without setup.py/pyproject.toml; pip cannot install it and no cargo/rustc exists here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    warmup, steps = max(3, args.warmup), max(1, args.steps)
    if args.workload == "serving":
        return serving_workload(args.align_step_tokens)
    if args.workload == "mixed_step":
        return mixed_step_workload()

    import numpy as np
    import torch
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    from aien_sovereign_core_mv_b200 import kernels as K
    from aien_sovereign_core_mv_b200.engine.generate import Generator
    from aien_sovereign_core_mv_b200.sampling import SamplingParams

    wl = dict(WORKLOADS[args.workload])
    if args.prompt_len > 0 and wl["prompt_len"]:
        wl["prompt_len"] = args.prompt_len
        wl["context"] = max(wl["context"], args.prompt_len + warmup + steps + 64)
        wl["points"] = ()
    batch_main = args.batch or wl["batch"]
    ptok = args.prefill_tokens if args.prefill_tokens > 0 else PREFILL_TOKENS
    if ptok != PREFILL_TOKENS:
        wl["context"] = max(wl["context"], ptok + 64)
        wl["points"] = ()
    cfg = dict(wl["cfg"])
    layers_cfg = cfg["num_hidden_layers"]
    layers_run = args.layers or layers_cfg
    cfg["num_hidden_layers"] = layers_run
    nums = model_numbers(cfg, layers_run)
    hbm_gbs, bf16_tflops, peak_src = peaks()
    CONTEXT, SEED = wl["context"], wl["seed"]
    # the timed steps end at `context` tokens when the workload gives no prompt length
    PROMPT_LEN = wl["prompt_len"] or CONTEXT - (warmup + steps)
    max_batch = max([batch_main, *wl["points"]])
    pool_tokens = max_batch * (PROMPT_LEN + warmup + steps + 64) + ptok
    ec = EngineConfig(dtype="bfloat16", page_size=PAGE, max_cache_tokens=pool_tokens, max_requests=max_batch,
                      max_batch_tokens=max(PREFILL_TOKENS, ptok), max_context=CONTEXT + (0 if wl["prompt_len"] else 64), max_batch_size=max_batch,
                      max_prefill_tokens=max(PREFILL_TOKENS, ptok), prefill_chunk_size=max(PREFILL_TOKENS, ptok))
    t_load = time.time()
    engine = Engine.from_config(cfg, seed=SEED, engine_config=ec, init_std=0.02, device_init=True)
    torch.cuda.synchronize()
    load_s = time.time() - t_load
    rng = np.random.default_rng(SEED)
    V = cfg["vocab_size"]
    if args.fill == "cache":
        for planes in engine.storage:
            for st in planes.values():
                st.normal_(0.0, 0.5)
    wait_errors = 0

    def count_wait_errors():
        """After a timed region (the device is idle): how many kernels left an error word."""
        nonlocal wait_errors
        wait_errors += sum(1 for w in K.read_wait_errors() if w != 0)

    def settle():
        """Filling the cache is a prefill at the power cap, and the SM clock stays low for some 70 ms
        after it: decode steps of 4.2 ms, then 3.8, then the 3.5 ms that decoding sustains for as
        long as it goes on.  A short pause between the fill and the warm-up steps lets the timed
        steps run at the clocks that decoding itself settles at."""
        torch.cuda.synchronize()
        time.sleep(SETTLE_S)

    def fill_requests(batch, first_id):
        """Each request gets a PROMPT_LEN-token prompt by real prefill: portions of at most 2,048
        tokens, several requests in a step where they fit."""
        ids = list(range(first_id, first_id + batch))
        if args.fill == "cache":
            for rid in ids:
                engine.cache.add_request(rid)
            engine.cache.append([(rid, PROMPT_LEN) for rid in ids])
            return ids
        ents, used = [], 0
        for rid in ids:
            left = PROMPT_LEN
            while left > 0:
                n = min(left, PREFILL_TOKENS - used)
                ents.append((rid, rng.integers(0, V, n), []))
                used += n
                left -= n
                if used == PREFILL_TOKENS:
                    engine.step(ents)
                    ents, used = [], 0
        if ents:
            engine.step(ents)
        return ids

    def decode_run(batch, first_id, n_warm, n_steps, sample_clocks=False):
        ids = fill_requests(batch, first_id)
        settle()
        toks = rng.integers(0, V, (n_warm + n_steps, batch))
        for s in range(n_warm):
            engine.step([(rid, [int(toks[s, j])], [0]) for j, rid in enumerate(ids)])
        torch.cuda.synchronize()
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
            time.sleep(0.25)
        launches0 = K.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(n_warm, n_warm + n_steps):
            engine.step([(rid, [int(toks[s, j])], [0]) for j, rid in enumerate(ids)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if sample_clocks else None
        launches = K.launch_count() - launches0
        engine.check_waits()
        count_wait_errors()
        ctx_mid = PROMPT_LEN + n_warm + n_steps // 2
        for rid in ids:
            engine.end_request(rid)
        return ms, clocks, launches, ctx_mid

    def prefill_run():
        """One 2,048-token prompt in one step: three untimed runs, then four timed ones, each after
        a pause of 0.3 s, because the peak it is set against is a burst figure too (back to back, a
        25 ms GEMM-bound step runs into the power cap after the third or fourth repetition, as a
        cuBLAS loop does); the median of the four."""
        ptoks = rng.integers(0, V, ptok)
        times = []
        for rep in range(7):
            torch.cuda.synchronize()
            if rep >= 3:
                time.sleep(0.3)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([(9000 + rep, ptoks, [ptok - 1])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            engine.end_request(9000 + rep)
        engine.check_waits()
        count_wait_errors()
        pms = float(np.median(times[3:]))
        T = ptok
        flops = 2.0 * (nums["linear_params"] - V * cfg["hidden_size"]) * T + 2.0 * V * cfg["hidden_size"] \
            + layers_run * 4.0 * nums["Q"] * T * (T + 1) / 2
        return {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3), "runs_ms": [round(t, 2) for t in times],
                "frac": round(flops / (pms / 1e3) / (bf16_tflops * 1e12), 4), "peak": f"{bf16_tflops} TFLOP/s bf16, of {peak_src}"}

    # the prefill is timed before the decode runs, as a burst, like the peak it is set against
    prefill = None if args.skip_prefill else prefill_run()

    # ---- headline: decode at the workload's batch
    ms, clocks, launches, ctx_mid = decode_run(batch_main, 1000, warmup, steps, sample_clocks=True)
    ms_per_step = ms / steps
    value = batch_main * steps / (ms / 1e3)
    step_bytes = nums["weight_bytes"] + batch_main * ctx_mid * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    points = {}
    if not args.skip_points:
        for b in wl["points"]:                     # the same number of timed steps as the headline
            pms, _, _, _ = decode_run(b, 2000 + 100 * b, warmup, steps)
            points[f"decode_b{b}"] = round(b * steps / (pms / 1e3), 1)

    e2e = None
    if not args.skip_e2e:
        # The same K decode steps through the public entry point: every step the scheduler plans,
        # token ids and block tables go host->device from pinned memory, the chosen ids come back.
        gen = Generator(engine)
        prompts = [rng.integers(0, V, PROMPT_LEN).tolist() for _ in range(batch_main)]
        sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, seed=SEED, max_tokens=4 * warmup + steps + 64, stop_token_ids=[])
        for i, p in enumerate(prompts):
            gen.submit(5000 + i, p, sp)
        def all_decoding():
            m = gen.scheduler.metrics()
            return m["prefill_tokens"] >= batch_main * PROMPT_LEN and gen.scheduler.num_running == batch_main
        while not all_decoding():
            gen.advance()
        gen.flush()
        settle()
        for _ in range(warmup):
            gen.advance()
        gen.flush()
        torch.cuda.synchronize()
        h0, d0, s0 = gen.h2d_bytes, gen.d2h_bytes, gen.steps
        dec0 = gen.scheduler.metrics()["decode_tokens"]
        t0 = time.perf_counter()
        for _ in range(steps):
            gen.advance()          # with async_scheduling (the default) step n+1 is launched before step n's ids are read
        gen.flush()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        count_wait_errors()
        n_steps = max(1, gen.steps - s0)
        new_tokens = gen.scheduler.metrics()["decode_tokens"] - dec0
        for i in range(batch_main):
            gen.scheduler.cancel(5000 + i)
        e2e = {"value": round(new_tokens / dt, 1), "unit": "tokens/s", "steps": n_steps, "pause_after_prefill_s": SETTLE_S,
               "sampling": {"temperature": args.temperature, "top_p": args.top_p, "top_k": args.top_k},
               "h2d_bytes_per_step": int((gen.h2d_bytes - h0) / n_steps), "d2h_bytes_per_step": int((gen.d2h_bytes - d0) / n_steps)}

    out = {
        "metric": "decode_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": wl["label"], "layers": layers_cfg, "layers_run": layers_run,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": V,
            "global_batch": batch_main, "seq_len": PROMPT_LEN, "context": CONTEXT, "page_size": PAGE,
            "parallelism": "single GPU", "prefill_tokens": ptok, "seed": SEED,
            "l2": "inputs larger than L2: 15 GB of weights per step", "fill": args.fill,
        },
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "wait_errors": int(wait_errors),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4), "of": peak_src, "bytes_per_step": int(step_bytes)},
        "points": points, "load_s": round(load_s, 1),
    }
    if args.workload == "decode":
        out["reference_gb10"] = {"tokens_per_s": 7.0, "source": "docs/campaigns/open-model-qwen3/RESULT-v7.md:67-68 (Qwen3-8B, GB10, one request)"}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
