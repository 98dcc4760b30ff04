"""Command line of the engine.

    aien-b200 generate --model-dir DIR --prompt-ids 1,2,3 [--max-tokens N] [--temperature T] ...
    aien-b200 random-model --config config.json --seed 0 --out DIR
    aien-b200 replay --model DIR --dtype float32 --out DIR --max-tokens N   (= bin/trace_run)
    aien-b200 info --model-dir DIR

Option names follow the reference where it has them: ``--model-dir``, ``--max-context``,
``--max-tokens-cap`` and ``--batch-slots`` are its server's flags (crates/aien-serve-http/src/
main.rs:123-206); ``--temperature``, ``--top-p``, ``--top-k``, ``--max-tokens``, ``--seed`` and
``--stop-token-ids`` are its generation parameters (crates/aien-abi-core/src/lib.rs:470-487,
crates/aien-inference-abi/src/qwen3_moe_omega.rs:3135-3160).  The model folder is also taken from
``AIEN_MODEL_DIR`` and the context cap from ``AIEN_KV_CONTEXT_TOKENS`` as the reference's daemon
does (crates/aien-cli/src/commands.rs:1057-1070, crates/aien-runtime/src/shared_kv.rs:321).  The
engine works on token ids; tokenizers are outside it.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def _engine_args(ap):
    ap.add_argument("--model-dir", default=os.environ.get("AIEN_MODEL_DIR"), help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-context", type=int, default=int(os.environ.get("AIEN_KV_CONTEXT_TOKENS", "0")),
                    help="longest request in tokens (0: the model's max_position_embeddings)")
    ap.add_argument("--batch-slots", type=int, default=64, help="requests live at a time")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--num-pages", type=int, default=0, help="cache pages (0: enough for batch-slots x max-context, capped)")
    ap.add_argument("--max-batch-tokens", type=int, default=4096)
    ap.add_argument("--prefill-chunk-size", type=int, default=512)
    ap.add_argument("--strict-config", action="store_true", help="refuse unknown config.json keys as the reference does")


def _build_engine(args):
    from . import Engine, EngineConfig
    if not args.model_dir:
        raise SystemExit("no model folder: give --model-dir or set AIEN_MODEL_DIR")
    from .config.model_config import read_config_json
    raw = read_config_json(args.model_dir)
    ctx = args.max_context or int(raw.get("max_position_embeddings", 4096))
    pages = args.num_pages or min(args.batch_slots * ((ctx + args.page_size - 1) // args.page_size), (1 << 20))
    ec = EngineConfig(dtype=args.dtype, page_size=args.page_size, num_pages=pages, max_requests=args.batch_slots,
                      max_context=ctx, max_batch_tokens=args.max_batch_tokens, max_batch_size=args.batch_slots,
                      max_prefill_tokens=min(args.max_batch_tokens, 2048), prefill_chunk_size=args.prefill_chunk_size)
    return Engine.from_folder(args.model_dir, ec, strict=args.strict_config)


def cmd_generate(args) -> int:
    from .engine.generate import Generator
    from .sampling import SamplingParams
    prompts = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts:
        raise SystemExit("no prompt: give --prompt-ids 1,2,3 (repeatable) or --prompt-file")
    engine = _build_engine(args)
    cap = args.max_tokens_cap or args.max_tokens
    sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, max_tokens=min(args.max_tokens, cap),
                        stop_token_ids=_ids(args.stop_token_ids) if args.stop_token_ids is not None else None, seed=args.seed,
                        logprobs=args.logprobs)
    gen = Generator(engine)
    t0 = time.perf_counter()
    results = gen.generate(prompts, sp)
    dt = time.perf_counter() - t0
    if args.json:
        out = {"tokens": [r.tokens for r in results], "finish_reasons": [r.finish_reason for r in results],
               "seconds": round(dt, 4), "steps": gen.steps}
        if args.logprobs:
            out["logprobs"] = [r.logprobs for r in results]
        print(json.dumps(out))
    else:
        for i, r in enumerate(results):
            print(f"[{i}] {r.finish_reason}: {' '.join(map(str, r.tokens))}")
            if args.logprobs and r.logprobs is not None:
                print(f"[{i}] logprobs: {' '.join(f'{v:.4f}' for v in r.logprobs)}")
        n = sum(len(r.tokens) for r in results)
        print(f"{n} tokens in {dt:.3f} s ({n / dt:.1f} tokens/s, {gen.steps} steps)", file=sys.stderr)
    return 0


def cmd_random_model(args) -> int:
    from . import write_random_model
    with open(args.config) as f:
        raw = json.load(f)
    out = write_random_model(args.out, raw, args.seed, args.init_std)
    print(out)
    return 0


def cmd_info(args) -> int:
    from . import model_spec_for
    from .config.model_config import read_config_json, read_generation_config
    from .models import Decoder
    cfg, spec = model_spec_for(read_config_json(args.model_dir), read_generation_config(args.model_dir), args.strict_config)
    model = Decoder(spec)
    params = sum(int(__import__("math").prod(shape)) for shape, _ in model.catalog().values())
    print(json.dumps({"architecture": spec.architecture, "layers": len(spec.layers), "hidden_size": spec.hidden_size,
                      "vocab_size": spec.vocab_size, "parameters": params, "cache_groups": [n.kind for n in model.group_needs],
                      "stop_token_ids": list(spec.stop_token_ids)}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aien-b200", description="B200 inference engine for the dense Llama / Qwen3 decoder")
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate token ids from prompt token ids")
    _engine_args(g)
    g.add_argument("--prompt-ids", "-p", action="append", default=[], help="comma- or space-separated token ids (repeatable)")
    g.add_argument("--prompt-file", help="one prompt per line, token ids")
    g.add_argument("--max-tokens", type=int, default=512)
    g.add_argument("--max-tokens-cap", type=int, default=0)
    g.add_argument("--temperature", type=float, default=0.7)
    g.add_argument("--top-p", type=float, default=0.95)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--stop-token-ids", default=None, help="default: the model's end-of-sequence ids")
    g.add_argument("--logprobs", action="store_true", help="the log-probability of every generated token with it")
    g.add_argument("--json", action="store_true")
    g.set_defaults(fn=cmd_generate)
    r = sub.add_parser("random-model", help="write config.json + model.safetensors with random weights")
    r.add_argument("--config", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--init-std", type=float, default=None)
    r.set_defaults(fn=cmd_random_model)
    i = sub.add_parser("info", help="what the registry builds for a model folder")
    _engine_args(i)
    i.set_defaults(fn=cmd_info)
    t = sub.add_parser("replay", help="trace replay (same as bin/trace_run)", add_help=False)
    t.set_defaults(fn=None)
    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .engine.trace_run import main as replay_main
        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    try:
        return args.fn(args)
    except (ValueError, RuntimeError, KeyError) as e:
        print(f"aien-b200: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
