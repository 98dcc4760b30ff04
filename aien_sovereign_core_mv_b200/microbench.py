"""Single kernels at model shapes, for timing and for profiler captures.

    python -m aien_sovereign_core_mv_b200.microbench gemv --n 24576 --k 4096 --m 1 --epilogue 1
    python -m aien_sovereign_core_mv_b200.microbench gemm --m 2048 --n 24576 --k 4096 --epilogue 1
    python -m aien_sovereign_core_mv_b200.microbench attn-decode --batch 1 --ctx 1030 --impl stream
    python -m aien_sovereign_core_mv_b200.microbench attn-prefill --tokens 2048 --impl tc
    python -m aien_sovereign_core_mv_b200.microbench qk --tokens 2048
    python -m aien_sovereign_core_mv_b200.microbench sample --rows 8 --top-p 0.95
    python -m aien_sovereign_core_mv_b200.microbench all

Every case launches its kernel a few times eagerly (what a profiler captures) and then times a
CUDA graph of back-to-back launches over rotating weight copies larger than L2, with CUDA events.
Attention cases use 32 query heads, 8 kv heads, head size 128, pages of 16 (the Qwen3-8B shape)
unless told otherwise.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import kernels as K


def _time_graph(fn, n: int) -> float:
    fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / n


def gemv_case(n: int, k: int, m: int, epilogue: int, reps: int = 20) -> None:
    copies = max(2, int(1.5e9 // (n * k * 2)))
    ws = [torch.randn(n, k, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(m, n // 2 if epilogue else n, device="cuda", dtype=torch.bfloat16)
    for i in range(3):
        K.gemv(a, ws[i % copies], out, epilogue=epilogue)
    us = _time_graph(lambda i: K.gemv(a, ws[i % copies], out, epilogue=epilogue), reps)
    print(f"gemv[{K.GEMV_IMPL}] N={n} K={k} M={m} epilogue={epilogue}: {us:8.2f} us  {n * k * 2 / us / 1e3:7.0f} GB/s of weights", flush=True)


def gemm_case(m: int, n: int, k: int, epilogue: int, reps: int = 10, splits: int = 1) -> None:
    """splits 1: bfloat16 output; > 1: float32 partial products over that many ranges of K; -1: as many
    ranges as the engine asks for when its consumer can add partial products (kernels.gemm_tc_splits)."""
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    if splits < 0:
        splits = K.gemm_tc_splits(m, n, k)
    ranges = K.gemm_tc_ranges(k, splits) if splits > 1 else 1
    if ranges > 1:
        out = torch.empty(ranges, m, n, device="cuda", dtype=torch.float32)
    else:
        out = torch.empty(m, n // 2 if epilogue else n, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        K.gemm_tc(a, w, out, epilogue=epilogue)
    us = _time_graph(lambda i: K.gemm_tc(a, w, out, epilogue=epilogue), reps)
    print(f"gemm_tc M={m} N={n} K={k} epilogue={epilogue} ranges={ranges}: {us:9.1f} us  {2.0 * m * n * k / us / 1e6:7.1f} TFLOP/s  (error flag {K.gemm_tc_error()})", flush=True)


def _paged_cache(batch: int, ctx: int, nkv: int, hd: int, page: int, layout: str = "shuffled"):
    """layout: where a request's pages lie in the pool.  "shuffled": anywhere (the worst case);
    "sequential": one after the other, as a fresh pool hands them out; "runs4": shuffled runs of 4."""
    pages_per = (ctx + page - 1) // page
    n_pages = batch * pages_per + 4
    kc = torch.randn(n_pages * page, nkv, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    width = max(256, pages_per + 1)
    bt = torch.full((batch, width), -1, dtype=torch.int32)
    if layout == "sequential":
        order = torch.arange(batch * pages_per)
    elif layout == "runs4":
        runs = torch.randperm(n_pages // 4)[:(batch * pages_per + 3) // 4]
        order = (runs[:, None] * 4 + torch.arange(4)[None]).reshape(-1)[:batch * pages_per]
    else:
        order = torch.randperm(n_pages)[:batch * pages_per]
    bt[:, :pages_per] = order.view(batch, pages_per).to(torch.int32)
    return kc, vc, bt.cuda(), width


def attn_decode_case(batch: int, ctx: int, nq: int = 32, nkv: int = 8, hd: int = 128, page: int = 16, reps: int = 40,
                     impl: str = "stream") -> None:
    kc, vc, bt, width = _paged_cache(batch, ctx, nkv, hd, page)
    q = torch.randn(batch, nq * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    splits = 1
    while splits * K.DECODE_CHUNK < ctx:
        splits *= 2
    po = torch.empty(batch * nq * splits * hd, device="cuda")
    pml = torch.empty(batch * nq * splits * 2, device="cuda")
    pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device="cuda")

    def run(_=0):
        K.paged_attention_decode(q, kc, vc, bt, width, None, pos, out, po, pml, nq, nkv, hd, page, 0, 1 / math.sqrt(hd), splits, impl=impl)

    for _ in range(3):
        run()
    us = _time_graph(run, reps)
    mb = batch * ctx * nkv * hd * 2 * 2 / 1e6
    print(f"attn-decode[{impl}] batch={batch} ctx={ctx} page={page} ({nq}q/{nkv}kv x {hd}): {us:8.2f} us  {mb:.1f} MB of K/V  {mb / us * 1e3:7.0f} GB/s"
          f"  (error flag {K.attention_decode_stream_error()})", flush=True)


def attn_prefill_case(tokens: int, offset: int = 0, nq: int = 32, nkv: int = 8, hd: int = 128, page: int = 16, reps: int = 10,
                      impl: str = "tc", layout: str = "shuffled", splits: int = 0) -> None:
    """splits: 0 lets the launch cut the keys into ranges where it sees fit (it is given the room), -1 gives
    it no room, n > 0 asks for n ranges."""
    ctx = offset + tokens
    kc, vc, bt, width = _paged_cache(1, ctx, nkv, hd, page, layout)
    q = torch.randn(tokens, nq * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    n_tiles = (tokens + K.PREFILL_TILE - 1) // K.PREFILL_TILE
    args = (i32([0, tokens]), i32([ctx]), i32([0] * n_tiles), i32([t * K.PREFILL_TILE for t in range(n_tiles)]), n_tiles)

    room = n_tiles * K.PREFILL_TILE * nq * splits * (hd + 2) * 4 if splits > 0 else K.prefill_split_scratch_bytes(n_tiles, nq, hd, ctx) if splits == 0 else 0
    scratch = torch.empty(room // 4, device="cuda") if room else None

    def run(_=0):
        K.paged_attention_prefill(q, kc, vc, bt, width, *args, out, nq, nkv, hd, page, 0, 1 / math.sqrt(hd), impl=impl,
                                  scratch=scratch, max_ctx=ctx, splits=max(splits, 0))

    for _ in range(3):
        run()
    us = _time_graph(run, reps)
    flops = 4.0 * nq * hd * (tokens * (tokens + 1) / 2 + tokens * offset)
    print(f"attn-prefill[{impl}] tokens={tokens} offset={offset} page={page} {layout} splits={splits} ({nq}q/{nkv}kv x {hd}): {us:8.1f} us  {flops / us / 1e6:7.1f} TFLOP/s"
          f"  (error flag {K.attention_prefill_tc_error()})", flush=True)


def qk_case(tokens: int, parts: int = 0, nq: int = 32, nkv: int = 8, hd: int = 128, reps: int = 20) -> None:
    """q/k norm + rotation + cache write on the projections of `tokens` tokens (bfloat16 rows, or
    `parts` float32 partial products as a product cut over K leaves them)."""
    width = (nq + 2 * nkv) * hd
    if parts == 0:
        buf = torch.randn(tokens, width, device="cuda").to(torch.bfloat16)
    else:
        buf = torch.randn(parts, tokens, width, device="cuda")
    q, k, v = buf[..., :nq * hd], buf[..., nq * hd:(nq + nkv) * hd], buf[..., (nq + nkv) * hd:]
    q_out = torch.empty(tokens, nq * hd, dtype=torch.bfloat16, device="cuda")
    qw = torch.ones(hd, dtype=torch.bfloat16, device="cuda"); kw = torch.ones(hd, dtype=torch.bfloat16, device="cuda")
    cos = torch.empty(tokens, hd // 2, device="cuda"); sin = torch.empty(tokens, hd // 2, device="cuda")
    inv = torch.tensor([1e6 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    K.rope_table(torch.arange(tokens, dtype=torch.int32, device="cuda"), inv, cos, sin)
    slot_map = torch.arange(tokens, dtype=torch.int32, device="cuda")
    kc = torch.zeros(tokens + 8, nkv, hd, dtype=torch.bfloat16, device="cuda"); vc = torch.zeros_like(kc)

    def run(_=0):
        K.qk_norm_rope_kv_write(q, k, v, hd, qw, kw, 1e-6, cos, sin, hd, slot_map, kc, vc, q_out=q_out)

    for _ in range(3):
        run()
    us = _time_graph(run, reps)
    moved = buf.numel() * buf.element_size() + tokens * width * 2
    print(f"qk tokens={tokens} parts={parts} ({nq}q/{nkv}kv x {hd}): {us:8.2f} us  {moved / us / 1e3:7.0f} GB/s read + written", flush=True)


def sample_case(rows: int, vocab: int, temperature: float, top_p: float, top_k: int, peaked: bool = True, reps: int = 10) -> None:
    """One sampling launch over `rows` rows of logits; `peaked`: a handful of tokens far above the rest, like a language model's."""
    logits = (torch.randn(rows, vocab, device="cuda") * 2).float()
    if peaked:
        idx = torch.randint(0, vocab, (rows, 40), device="cuda")
        logits.scatter_(1, idx, torch.rand(rows, 40, device="cuda") * 8 + 10)
    ids = torch.empty(rows, dtype=torch.int32, device="cuda")
    scratch = torch.empty(rows * vocab, device="cuda")
    t = torch.full((rows,), temperature, device="cuda"); tp = torch.full((rows,), top_p, device="cuda")
    tk = torch.full((rows,), top_k, dtype=torch.int32, device="cuda")
    seeds = torch.arange(rows, dtype=torch.int64, device="cuda"); rid = torch.arange(rows, dtype=torch.int64, device="cuda")
    pos = torch.full((rows,), 100, dtype=torch.int32, device="cuda")

    def run(_=0):
        K.sample_rows(logits, t, tp, tk, seeds, rid, pos, scratch, ids)

    for _ in range(3):
        run()
    us = _time_graph(run, reps)
    print(f"sample rows={rows} vocab={vocab} T={temperature} top_p={top_p} top_k={top_k} {'peaked' if peaked else 'flat'}: {us:8.1f} us", flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="microbench", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="case", required=True)
    p = sub.add_parser("gemv")
    p.add_argument("--n", type=int, default=24576); p.add_argument("--k", type=int, default=4096)
    p.add_argument("--m", type=int, default=1); p.add_argument("--epilogue", type=int, default=0)
    p = sub.add_parser("gemm")
    p.add_argument("--m", type=int, default=2048); p.add_argument("--n", type=int, default=24576)
    p.add_argument("--k", type=int, default=4096); p.add_argument("--epilogue", type=int, default=0)
    p.add_argument("--splits", type=int, default=1, help="ranges of K into float32 partial products; -1: what the engine would ask for")
    p = sub.add_parser("attn-decode")
    p.add_argument("--batch", type=int, default=1); p.add_argument("--ctx", type=int, default=1030)
    p.add_argument("--impl", default="stream", choices=["stream", "direct"]); p.add_argument("--page", type=int, default=16)
    p = sub.add_parser("attn-prefill")
    p.add_argument("--tokens", type=int, default=2048); p.add_argument("--offset", type=int, default=0)
    p.add_argument("--impl", default="tc", choices=["tc", "mma"]); p.add_argument("--page", type=int, default=16)
    p.add_argument("--layout", default="shuffled", choices=["shuffled", "sequential", "runs4"], help="where the request's pages lie in the pool")
    p.add_argument("--splits", type=int, default=0, help="ranges the keys of a tile are cut into: 0 as the launch chooses, -1 never, n > 0 exactly n")
    p = sub.add_parser("qk")
    p.add_argument("--tokens", type=int, default=2048); p.add_argument("--parts", type=int, default=0)
    p = sub.add_parser("sample")
    p.add_argument("--rows", type=int, default=8); p.add_argument("--vocab", type=int, default=151936)
    p.add_argument("--temperature", type=float, default=0.7); p.add_argument("--top-p", type=float, default=0.95)
    p.add_argument("--top-k", type=int, default=0); p.add_argument("--flat", action="store_true")
    sub.add_parser("all")
    args = ap.parse_args(argv)
    K.lib()
    if args.case == "gemv":
        gemv_case(args.n, args.k, args.m, args.epilogue)
    elif args.case == "gemm":
        gemm_case(args.m, args.n, args.k, args.epilogue, splits=args.splits)
    elif args.case == "attn-decode":
        attn_decode_case(args.batch, args.ctx, page=args.page, impl=args.impl)
    elif args.case == "attn-prefill":
        attn_prefill_case(args.tokens, args.offset, page=args.page, impl=args.impl, layout=args.layout, splits=args.splits)
    elif args.case == "qk":
        qk_case(args.tokens, args.parts)
    elif args.case == "sample":
        sample_case(args.rows, args.vocab, args.temperature, args.top_p, args.top_k, peaked=not args.flat)
    else:
        shapes = {"qkv": (6144, 4096, 0), "o": (4096, 4096, 0), "gate_up": (24576, 4096, 1), "down": (4096, 12288, 0), "head": (151936, 4096, 0)}
        for m in (1, 8, 16):
            for name, (n, k, epi) in shapes.items():
                gemv_case(n, k, m, epi)
        for m in (64, 256, 2048, 8192):
            for name, (n, k, epi) in shapes.items():
                if name != "head":
                    gemm_case(m, n, k, epi)
        for impl in ("stream", "direct"):
            for b in (1, 8, 64):
                attn_decode_case(b, 1030, impl=impl)
            attn_decode_case(16, 8192, impl=impl)
        for t, off in ((2048, 0), (512, 1536), (8192, 0)):
            for impl in ("tc", "mma"):
                attn_prefill_case(t, off, impl=impl)
        for t, parts in ((8, 0), (64, 6), (512, 0), (2048, 0)):
            qk_case(t, parts)
        for tp, tk in ((0.95, 0), (0.95, 50), (1.0, 0)):
            sample_case(8, 151936, 0.7, tp, tk)
    return 0


if __name__ == "__main__":
    sys.exit(main())
