"""The engine at the layer sizes of the real models (Qwen3-8B, Llama-3-8B and Llama-3.2-1B shapes, two layers, a
small vocabulary so that the plain implementation stays fast): the kernels meet their production
shapes here (K = 4096 / 12288 / 14336, 32 query heads in groups of 4, head size 128), whole, in portions and
decoding, in float32 and bfloat16."""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

SHAPES = {
    "qwen3_8b": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=4096,
                     num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=2048,
                     rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096,
                     hidden_act="silu", eos_token_id=1),
    "llama3_8b": dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=4096,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=1000,
                      rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=8192,
                      hidden_act="silu", eos_token_id=1),
    # heads of 64 at production widths, tied embeddings, scaled rotation (the Llama-3.2-1B layer shape)
    "llama32_1b": dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=2048,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=1504,
                       rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072,
                       rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                     "original_max_position_embeddings": 8192},
                       hidden_act="silu", eos_token_id=1),
}


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    from aien_sovereign_core_mv_b200 import write_random_model
    root = tmp_path_factory.mktemp("big")
    out = {}
    for name, cfg in SHAPES.items():
        d = write_random_model(str(root / name), cfg, seed=2, init_std=0.02)
        toks = [int(t) for t in np.random.default_rng(5).integers(0, cfg["vocab_size"], 200)]
        out[name] = (d, toks, H.plain_logits(d, toks))
    return out


@pytest.mark.parametrize("dtype,tol", [("float32", H.FP32_TOL), ("bfloat16", H.BF16_TOL)])
@pytest.mark.parametrize("name", list(SHAPES))
def test_production_layer_sizes(big, name, dtype, tol):
    d, toks, want = big[name]
    eng = H.engine_for(d, dtype, 16, 1024, max_requests=16, max_batch_tokens=256)
    # whole; then 150 tokens in portions of 64 + 64 + 22 followed by 50 single tokens; then a batch of decoding requests
    got = H.run_steps(eng, [([(1, toks, list(range(len(toks))))], [1])])
    H.assert_close(np.stack([got[1][p] for p in range(len(toks))]), want, tol, f"{name} {dtype} whole")
    steps = [([(2, toks[:64], [63])], []), ([(2, toks[64:128], [0, 63])], []), ([(2, toks[128:150], [21])], [])]
    steps += [([(2, [t], [0])], []) for t in toks[150:]]
    got = H.run_steps(eng, steps)
    pos = sorted(got[2])
    H.assert_close(np.stack([got[2][p] for p in pos]), want[pos], tol, f"{name} {dtype} portions + decode")
    eng.end_request(2)
    # twelve requests decoding together (the small-batch product with two token tiles) beside one portion
    ids = list(range(10, 22))
    H.run_steps(eng, [([(r, toks[:20 + r], []) for r in ids[:6]], []), ([(r, toks[:20 + r], []) for r in ids[6:]], [])])
    got = H.run_steps(eng, [([(r, [toks[20 + r]], [0]) for r in ids], []),
                            ([(r, [toks[21 + r]], [0]) for r in ids] + [(99, toks[:40], [39])], ids + [99])])
    for r in ids:
        H.assert_close(np.stack([got[r][0], got[r][1]]), want[[20 + r, 21 + r]], tol, f"{name} {dtype} batched decode, request {r}")
    H.assert_close(got[99][39], want[39], tol, f"{name} {dtype} portion beside decodes")
    assert eng.cache_state()["check"] == "" and eng.cache_state()["requests"] == 0


def test_norm_spread_over_the_products_around_it(big, monkeypatch):
    """Decode steps of few tokens run no norm kernel between two products: the product before adds
    the residual and prepares the norm, the product after finishes it.  Same logits within the
    bfloat16 tolerance, three launches fewer per layer but the first norm of the first layer."""
    from aien_sovereign_core_mv_b200 import kernels as K
    from aien_sovereign_core_mv_b200.parts import norm as norm_part
    d, toks, want = big["qwen3_8b"]
    res = {}
    for fuse in (True, False):
        monkeypatch.setattr(norm_part, "_FUSE", fuse)
        eng = H.engine_for(d, "bfloat16", 16, 1024, max_requests=16, max_batch_tokens=256, use_cuda_graphs=False)
        H.run_steps(eng, [([(1, toks[:100], [])], [])])
        before = K.launch_count()
        got = H.run_steps(eng, [([(1, [t], [0])], []) for t in toks[100:110]])
        res[fuse] = (np.stack([got[1][p] for p in sorted(got[1])]), K.launch_count() - before)
        eng.end_request(1)
        assert K.gemv_stream_error() == 0
    layers = SHAPES["qwen3_8b"]["num_hidden_layers"]
    assert res[False][1] - res[True][1] == 10 * (2 * layers - 1)
    for fuse in (True, False):
        H.assert_close(res[fuse][0], want[100:110], H.BF16_TOL, f"decode, fused={fuse}")


def test_long_context_bfloat16_follows_float32():
    """9,000 tokens through the production layer sizes: prompt portions at offsets far into the
    context, then single tokens over 71 key chunks.  The engine allows contexts of 17,000 tokens, so its
    decode steps are laid out for 128 chunks a token, where the chunks are merged by a kernel of its own.
    The plain implementation is too slow here, so the bfloat16 kernels are held against the engine's own
    32-bit path, itself checked above."""
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    import torch
    cfg = dict(SHAPES["qwen3_8b"], max_position_embeddings=32768)
    n = 9000
    toks = [int(t) for t in np.random.default_rng(1).integers(0, cfg["vocab_size"], n + 12)]
    out = {}
    for dtype in ("float32", "bfloat16"):
        ec = EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=n + 2048, max_requests=4, max_batch_tokens=2048, max_context=n + 8000)
        eng = Engine.from_config(cfg, seed=3, engine_config=ec, init_std=0.02, device_init=True)
        rows = []
        for i in range(0, n, 2048):
            part = toks[i:i + 2048]
            lg = eng.step([(1, part, [0, len(part) - 1])])
            rows += [lg[0].float().cpu().numpy(), lg[1].float().cpu().numpy()]
        for t in toks[n:]:
            rows.append(eng.step([(1, [t], [0])])[0].float().cpu().numpy())
        out[dtype] = np.stack(rows)
        assert eng.cache_state()["check"] == ""
        del eng
        torch.cuda.empty_cache()
    H.assert_close(out["bfloat16"], out["float32"], H.BF16_TOL, "long context, bfloat16 against float32")


# ------------------------------------------------------------------ the schedules of serving, against the plain implementation
@pytest.fixture(scope="module")
def prefixes(tmp_path_factory):
    """One sequence of 1,030 tokens through the plain implementation (Qwen3-8B layer shape, two
    layers).  Every request of the tests below holds a prefix of it, so the plain logits of one
    forward pass serve all of them: the model is causal."""
    from aien_sovereign_core_mv_b200 import write_random_model
    d = write_random_model(str(tmp_path_factory.mktemp("prefixes") / "m"), SHAPES["qwen3_8b"], seed=2, init_std=0.02)
    toks = [int(t) for t in np.random.default_rng(11).integers(0, SHAPES["qwen3_8b"]["vocab_size"], 1030)]
    return d, toks, H.plain_logits(d, toks)


def _prefill_prefixes(eng, toks, lengths, first_id, budget=2048):
    """Requests first_id.. hold toks[:L] for L in lengths; several requests a step under `budget` tokens."""
    step, used = [], 0
    for i, L in enumerate(lengths):
        if used + L > budget and step:
            eng.step(step)
            step, used = [], 0
        step.append((first_id + i, toks[:L], []))
        used += L
    if step:
        eng.step(step)


@pytest.mark.parametrize("dtype,tol", [("float32", H.FP32_TOL), ("bfloat16", H.BF16_TOL)])
@pytest.mark.parametrize("batch", [40, 64])
def test_many_requests_decoding_together_at_unequal_contexts(prefixes, batch, dtype, tol):
    """What a decode step of a large batch runs: the tile product at 32 / 64 rows with its partial
    products summed by the norm, q/k and row-gather kernels, and the decode attention's cut of all
    (token, kv head) pairs into equal ranges, with contexts from 33 to 700 tokens."""
    d, toks, want = prefixes
    eng = H.engine_for(d, dtype, 16, batch * 720, max_requests=64, max_batch_tokens=2048)
    lengths = [33 + (667 * i) // (batch - 1) for i in range(batch)]
    lengths[1::2] = lengths[1::2][::-1]                      # neighbours in the batch differ widely
    ids = list(range(1, batch + 1))
    _prefill_prefixes(eng, toks, lengths, 1)
    for s in range(3):
        logits = eng.step([(r, [toks[L + s]], [0]) for r, L in zip(ids, lengths)]).cpu().numpy()
        eng.check_waits()
        for row, L in enumerate(lengths):
            H.assert_close(logits[row], want[L + s], tol, f"{dtype} batch {batch}, step {s}, request {row + 1} at context {L + s + 1}")
    for r in ids:
        eng.end_request(r)
    assert eng.cache_state()["check"] == "" and eng.cache_state()["requests"] == 0


@pytest.mark.parametrize("dtype,tol", [("float32", H.FP32_TOL), ("bfloat16", H.BF16_TOL)])
def test_a_long_portion_beside_many_single_tokens(prefixes, dtype, tol):
    """The step a chunked-prefill server runs all day: a 512-token portion that starts at offset 512
    (four query tiles, keys from earlier pages) beside 24 requests that bring one token each
    (the split-key kernel over a list of tokens), products at 536 rows."""
    d, toks, want = prefixes
    eng = H.engine_for(d, dtype, 16, 1024 + 24 * 640, max_requests=32, max_batch_tokens=2048)
    lengths = [20 + 25 * i for i in range(24)]               # 20 .. 595
    _prefill_prefixes(eng, toks, lengths, 10)
    eng.step([(1, toks[:512], [])])
    wanted = [0, 127, 128, 300, 511]
    entries = [(10 + i, [toks[L]], [0]) for i, L in enumerate(lengths[:12])]
    entries.append((1, toks[512:1024], wanted))
    entries += [(22 + i, [toks[L]], [0]) for i, L in enumerate(lengths[12:])]
    logits = eng.step(entries).cpu().numpy()
    eng.check_waits()
    row = 0
    for rid, tk, wnt in entries:
        for w in wnt:
            pos = 512 + w if rid == 1 else lengths[rid - 10]
            H.assert_close(logits[row], want[pos], tol, f"{dtype} mixed step, request {rid}, position {pos}")
            row += 1
    assert eng.cache_state()["check"] == ""


@pytest.fixture(scope="module")
def long_request(tmp_path_factory):
    """4,200 tokens through one layer of the Qwen3-8B shape in the plain implementation."""
    from aien_sovereign_core_mv_b200 import write_random_model
    cfg = dict(SHAPES["qwen3_8b"], num_hidden_layers=1, max_position_embeddings=8192)
    d = write_random_model(str(tmp_path_factory.mktemp("long") / "m"), cfg, seed=5, init_std=0.02)
    toks = [int(t) for t in np.random.default_rng(12).integers(0, cfg["vocab_size"], 4200)]
    rows = [0, 1, 2047, 2048, 2049, 3000, 4095] + list(range(4096, 4200))
    return d, toks, rows, H.plain_logits(d, toks)[rows]


@pytest.mark.parametrize("dtype,tol", [("float32", H.FP32_TOL), ("bfloat16", H.BF16_TOL)])
def test_a_request_of_4200_tokens(long_request, dtype, tol):
    """2,048 + 2,048 tokens as two portions, then 104 single tokens: the portion at an offset reads
    16 earlier key blocks, the single tokens attend over 33 key chunks, and the 32-bit attention
    kernel walks the same length; each is held to the plain implementation, not to one another."""
    d, toks, rows, want = long_request
    eng = H.engine_for(d, dtype, 16, 4352, max_requests=2, max_batch_tokens=2048, max_context=4352)
    got = [eng.step([(1, toks[:2048], [0, 1, 2047])]).cpu().numpy(),
           eng.step([(1, toks[2048:4096], [0, 1, 952, 2047])]).cpu().numpy()]
    for t in toks[4096:]:
        got.append(eng.step([(1, [t], [0])]).cpu().numpy())
    eng.check_waits()
    H.assert_close(np.concatenate(got), want, tol, f"{dtype} 4,200-token request (rows {rows[:7]} and 4096..4199)")
    assert eng.cache_state()["check"] == ""


def test_a_short_last_portion_of_a_long_request_is_cut_over_key_ranges(long_request):
    """3,944 tokens in two portions, then the last 256 as one: two query tiles over 33 key blocks, which
    the tcgen05 prefill kernel cuts into key ranges on separate CTAs and merges.  Held to the plain
    implementation at rows of both tiles."""
    d, toks, rows, want = long_request
    eng = H.engine_for(d, "bfloat16", 16, 4352, max_requests=2, max_batch_tokens=2048, max_context=4352)
    eng.step([(1, toks[:2048], [])])
    eng.step([(1, toks[2048:3944], [])])
    got = eng.step([(1, toks[3944:], [r - 3944 for r in rows if r >= 3944])]).cpu().numpy()
    eng.check_waits()
    H.assert_close(got, want[[i for i, r in enumerate(rows) if r >= 3944]], H.BF16_TOL, "last 256 tokens of 4,200 as one portion")
    assert eng.cache_state()["check"] == ""
