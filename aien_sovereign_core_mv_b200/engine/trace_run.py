"""Trace replay: feeds given token ids through the model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--page-size P]

It samples nothing and owns no model code: it builds the same :class:`Engine` that generation
uses and calls its ``step``.  Steps are read from standard input, one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted it writes ``<out>/<step>.f32``: float32 little-endian
``[wanted, vocab]`` in the order of the entries and of each ``want``.  After every step it
prints ``done <step>`` and flushes.  ``end`` lists requests whose pages are given back after
the step.  The cache pool holds ``--max-tokens`` tokens (whole pages), so pages are reused.

The nearest thing in the reference is its teacher-forced ``logits_per_step`` helper
(crates/aien-inference-runtime/tests/drift/mod.rs:46-92).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens the cache pool holds")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default 16)")
    ap.add_argument("--max-requests", type=int, default=8, help="requests live at a time (default 8)")
    args = ap.parse_args(argv)

    print("trace_run: loading the engine (native code is compiled at first use)", file=sys.stderr, flush=True)
    import numpy as np
    import torch
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig

    os.makedirs(args.out, exist_ok=True)
    page = args.page_size
    pool_tokens = ((args.max_tokens + page - 1) // page) * page
    ec = EngineConfig(dtype=args.dtype, page_size=page, max_cache_tokens=pool_tokens, max_requests=args.max_requests,
                      max_batch_tokens=max(pool_tokens, 64), max_context=0)
    engine = Engine.from_folder(args.model, ec)       # its context limit is the model's, or the pool if that is smaller
    print("trace_run: ready", file=sys.stderr, flush=True)

    ids = {}                                  # trace ids (any JSON scalar) -> engine request ids
    next_id = 1
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            key = json.dumps(e["id"])
            if key not in ids:
                ids[key] = next_id
                next_id += 1
            entries.append((ids[key], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                arr = logits.to("cpu").numpy().astype("<f4", copy=False)
                engine.check_waits()                  # a kernel wait that ran out makes the step fail, not write
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
                engine.check_waits()
        for rid in rec.get("end", []):
            key = json.dumps(rid)
            if key in ids:
                engine.end_request(ids.pop(key))
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    sys.exit(main())
