"""Each part alone against its plain restatement, and the generality of the arrangement: a toy
mixer with state of its own, a toy feed-forward with routing and a toy position encoding are
registered from here, built by the generic decoder and stepped by the engine, with no change to
the framework's files; a run list that names a layer twice and lets a run read another run's
cache."""
import dataclasses
import math

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as pm

pytestmark = pytest.mark.gpu


def make_ctx(dtype, positions, seq_of_token, q_start, ctx_len, groups=(), nbytes=1 << 24):
    from aien_sovereign_core_mv_b200.parts import StepContext, Workspace
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    T, S = len(positions), len(ctx_len)
    ws = Workspace(nbytes, nbytes, torch.device("cuda"))
    ws.begin_layer()
    tiles_s, tiles_q = [], []
    for s in range(S):
        for t in range((q_start[s + 1] - q_start[s] + 127) // 128):
            tiles_s.append(s); tiles_q.append(128 * t)
    return StepContext(dtype=dtype, num_tokens=T, num_seqs=S, token_ids=i32([0] * T), positions=i32(positions),
                       seq_of_token=i32(seq_of_token), q_start=i32(q_start), ctx_len=i32(ctx_len), groups=list(groups),
                       workspace=ws, max_q_len=max(q_start[i + 1] - q_start[i] for i in range(S)), max_ctx_len=max(ctx_len),
                       decode_only=(T == S), prefill_tiles=(i32(tiles_s), i32(tiles_q), len(tiles_s)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from aien_sovereign_core_mv_b200.registry import make_part
    norm = make_part("norm", "rmsnorm", size=72, eps=3e-6)
    g = torch.Generator().manual_seed(0)
    w = (torch.rand(72, generator=g) * 0.4 + 0.8).to(torch.bfloat16)
    norm.bind({"weight": w.cuda()})
    x = torch.randn(5, 72, generator=g).cuda(); d = torch.randn(5, 72, generator=g).to(dtype).cuda()
    ctx = make_ctx(dtype, [0, 1, 2, 3, 4], [0] * 5, [0, 5], [5])
    x0 = x.clone()
    h = norm.forward(ctx, x, d)
    xs = (x0.double() + d.double()).cpu().numpy()
    H.assert_close(x.cpu().numpy(), xs, 1e-6, "residual sum")
    H.assert_close(h.float().cpu().numpy(), pm.rms_norm(xs, w.double().numpy(), 3e-6), 2e-5 if dtype == torch.float32 else 1e-2, "norm part")


def test_rotary_part_tables_and_scaling():
    from aien_sovereign_core_mv_b200.registry import make_part
    scaling = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    for sc in (None, scaling):
        rot = make_part("position", "rotary", head_dim=48, theta=500000.0, scaling=sc)
        pos = [0, 5, 63, 64, 1000, 4095]
        ctx = make_ctx(torch.float32, pos, [0] * 6, [0, 6], [4096])
        cos, sin, rdim = rot.rotary(ctx)
        assert rdim == 48 and rot.rotary(ctx)[0] is cos                 # built once per step
        inv = pm.rope_inv_freq(48, 500000.0, sc)
        ang = np.asarray(pos, dtype=np.float64)[:, None] * inv[None]
        assert np.abs(cos.cpu().numpy() - np.cos(ang)).max() <= 1.2e-7 and np.abs(sin.cpu().numpy() - np.sin(ang)).max() <= 1.2e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [3, 40])
def test_feed_forward_part(dtype, T):
    from aien_sovereign_core_mv_b200.registry import make_part
    ff = make_part("feed_forward", "swiglu", hidden_size=72, intermediate_size=200)
    g = torch.Generator().manual_seed(1)
    ws = {n: (torch.randn(s, generator=g) / math.sqrt(s[1])).to(torch.bfloat16) for n, (s, _) in ff.param_shapes().items()}
    ff.bind({n: (t.cuda() if dtype == torch.bfloat16 else t.float().cuda()) for n, t in ws.items()})
    h = torch.randn(T, 72, generator=g).to(dtype).cuda()
    ctx = make_ctx(dtype, list(range(T)), [0] * T, [0, T], [T])
    y = ff.forward(ctx, h)
    y = y.sum(0) if y.dim() == 3 else y                                   # split-K partial products add up
    hd = h.double().cpu().numpy()
    a = pm.swiglu(hd @ ws["gate_proj"].double().numpy().T, hd @ ws["up_proj"].double().numpy().T)
    if dtype == torch.bfloat16:
        a = pm.round_bf16(a)
    H.assert_close(y.float().cpu().numpy(), a @ ws["down_proj"].double().numpy().T, 2e-5 if dtype == torch.float32 else 1.5e-2, "swiglu part")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 9])
def test_attention_mixer_alone(dtype, window):
    """The mixer with hand-made cache views: a portion of 11 tokens after 6 cached ones, beside a
    single token of another request."""
    from aien_sovereign_core_mv_b200.parts import GroupView, RunBinding
    from aien_sovereign_core_mv_b200.registry import make_part
    Hd, nq, nkv, hd, page = 80, 6, 3, 16, 4
    rot = make_part("position", "rotary", head_dim=hd, theta=10000.0)
    att = make_part("mixer", "paged_attention", position=rot, hidden_size=Hd, num_heads=nq, num_kv_heads=nkv, head_dim=hd,
                    qk_norm=True, qk_norm_eps=1e-6, window=window)
    g = torch.Generator().manual_seed(2)
    ws = {}
    for n, (s, kind) in att.param_shapes().items():
        ws[n] = ((torch.rand(s, generator=g) * 0.4 + 0.8) if kind == "norm" else torch.randn(s, generator=g) / math.sqrt(s[-1])).to(torch.bfloat16)
    att.bind({n: (t.cuda() if dtype == torch.bfloat16 else t.float().cuda()) for n, t in ws.items()})
    lens = [17, 9]
    hs = [torch.randn(n, Hd, generator=g).to(torch.bfloat16) for n in lens]
    storage = {n: torch.zeros(1, 16 * page, nkv, hd, dtype=dtype, device="cuda") for n in ("k", "v")}
    tables = [[3, 0, 7, 5, 9], [2, 8, 1]]
    bt = torch.full((2, 6), -1, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = torch.tensor(t)
    slot = lambda s, p: tables[s][p // page] * page + p % page

    def run(entries):      # entries: (seq, first position, count)
        pos, sot, qs, cl, sm, rows = [], [], [0], [], [], []
        for i, (s, p0, n) in enumerate(entries):
            pos += list(range(p0, p0 + n)); sot += [i] * n; qs.append(qs[-1] + n); cl.append(p0 + n)
            sm += [slot(s, p) for p in range(p0, p0 + n)]
            rows.append(hs[s][p0:p0 + n])
        gv = GroupView("window" if window else "full", page, window, 6,
                       torch.stack([bt[s] for s, _, _ in entries]).cuda(), torch.tensor(sm, dtype=torch.int32).cuda(), storage)
        ctx = make_ctx(dtype, pos, sot, qs, cl, [gv])
        y = att.forward(ctx, torch.cat(rows).to(dtype).cuda(), RunBinding(0, 0, True))
        return (y.sum(0) if y.dim() == 3 else y).float().cpu().numpy()

    run([(0, 0, 6), (1, 0, 8)])
    got = run([(0, 6, 11), (1, 8, 1)])
    want = []
    for s, (lo, hi) in zip((0, 1), ((6, 17), (8, 9))):
        x = hs[s].double().numpy()
        T = len(x)
        q = pm.rms_norm((x @ ws["q_proj"].double().numpy().T).reshape(T, nq, hd), ws["q_norm"].double().numpy(), 1e-6)
        k = pm.rms_norm((x @ ws["k_proj"].double().numpy().T).reshape(T, nkv, hd), ws["k_norm"].double().numpy(), 1e-6)
        v = (x @ ws["v_proj"].double().numpy().T).reshape(T, nkv, hd)
        inv = pm.rope_inv_freq(hd, 10000.0)
        q, k = pm.apply_rope(q, range(T), inv), pm.apply_rope(k, range(T), inv)
        o = pm.attention(q, k, v, np.arange(T), window or None).reshape(T, nq * hd)
        want.append((o @ ws["o_proj"].double().numpy().T)[lo:hi])
    H.assert_close(got, np.concatenate(want), 1e-4 if dtype == torch.float32 else 3e-2, "attention mixer")


# ---------------------------------------------------------------------------- toy parts
def register_toy_parts():
    from aien_sovereign_core_mv_b200 import register_feed_forward, register_mixer, register_position
    from aien_sovereign_core_mv_b200.parts import CacheNeed, FeedForward, Mixer, Position

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        """y[t] = mean of h[0..t] of the same request: the state is (sum, count), one slot per request."""

        def __init__(self, hidden_size, position=None):
            self.hidden_size = hidden_size

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.hidden_size + 1,), state_dtype="float32")

        def forward(self, ctx, h, run):
            """All on the device, by the contract of fixed-size state (parts/base.py, GroupView): the
            slot of request s is slot_map[s]; its portion is q_start[s]..q_start[s+1]; a portion that
            starts at position 0 starts from nothing.  Nothing is read on the host, so decode steps of
            a model with this mixer are captured in CUDA graphs like any other."""
            group = ctx.groups[run.group]
            state = group.storage["state"][run.slot]            # [slots + 1, H+1]
            S, T = ctx.num_seqs, ctx.num_tokens
            seq = ctx.seq_of_token[:T].long()
            first = ctx.q_start[:S].long()
            last = ctx.q_start[1:S + 1].long() - 1
            slots = group.slot_map[:S].long()
            fresh = (ctx.positions[:T].long()[first] == 0)
            base = torch.where(fresh[:, None], torch.zeros((), device=h.device), state[slots]).double()      # [S, H+1]
            hd = h.double()
            csum = torch.cumsum(hd, 0)
            within = csum - (csum[first] - hd[first])[seq]       # running sums inside each portion
            sums = base[seq, :-1] + within
            counts = base[seq, -1] + (torch.arange(T, device=h.device) - first[seq] + 1).double()
            state[slots] = torch.cat([sums[last], counts[last, None]], 1).float()
            return (sums / counts[:, None]).to(h.dtype)

    @register_feed_forward("toy_routed")
    class Routed(FeedForward):
        """Two experts (plain matrices); a token goes to the expert with the larger router logit."""

        def __init__(self, hidden_size):
            self.hidden_size = hidden_size

        def param_shapes(self):
            Hd = self.hidden_size
            return {"router": ((2, Hd), "matrix"), "expert0": ((Hd, Hd), "matrix"), "expert1": ((Hd, Hd), "matrix")}

        def bind(self, tensors):
            self.t = {k: v.float() for k, v in tensors.items()}

        def forward(self, ctx, h):
            x = h.float()
            pick = (x @ self.t["router"].T).argmax(-1)
            y = torch.where((pick == 0)[:, None], x @ self.t["expert0"].T, x @ self.t["expert1"].T)
            return y.to(h.dtype)

    @register_position("toy_additive")
    class Additive(Position):
        """No rotation: adds 0.01 * position to the first value of every query head."""

        def __init__(self, head_dim):
            self.head_dim = head_dim

        def rotary(self, ctx):
            return None

        def apply(self, ctx, q, group, run):
            q[:, ::self.head_dim] += (0.01 * ctx.positions.float()).to(q.dtype)[:, None]


def toy_spec():
    from aien_sovereign_core_mv_b200 import LayerSpec, ModelSpec, PartSpec, RunEntry
    Hd, V = 48, 97
    norm = PartSpec("rmsnorm", {"eps": 1e-5})
    rot = PartSpec("rotary", {"head_dim": 16, "theta": 10000.0})
    att = PartSpec("paged_attention", {"hidden_size": Hd, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16})
    layers = (
        LayerSpec("prenorm", PartSpec("toy_running_mean", {"hidden_size": Hd}), PartSpec("swiglu", {"hidden_size": Hd, "intermediate_size": 64}),
                  norm, PartSpec("none", {}), "l0."),
        LayerSpec("prenorm", att, PartSpec("toy_routed", {"hidden_size": Hd}), norm, rot, "l1."),
        LayerSpec("prenorm", att, PartSpec("swiglu", {"hidden_size": Hd, "intermediate_size": 64}), norm,
                  PartSpec("toy_additive", {"head_dim": 16}), "l2."),
    )
    # layer 1 runs twice (second time on its own cache), then layer 2 reads the cache layer 1 wrote first
    run_list = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(1, 2), RunEntry(2, 1, False))
    return ModelSpec("Toy", Hd, V, layers, run_list, PartSpec("table", {"name": "emb"}), PartSpec("rmsnorm", {"eps": 1e-5, "name": "fn"}),
                     PartSpec("linear", {"name": "head", "tied": False}), 256)


def toy_plain(w, ids):
    Hd, hd, nq = 48, 16, 3
    T = len(ids)
    x = w["emb"][ids]
    inv = pm.rope_inv_freq(hd, 10000.0)
    caches = {}

    def attn(prefix, h, position_kind, cache_key, writes):
        q = pm.linear(h, w[prefix + "mixer.q_proj"]).reshape(T, nq, hd)
        if writes:
            k = pm.linear(h, w[prefix + "mixer.k_proj"]).reshape(T, 1, hd)
            v = pm.linear(h, w[prefix + "mixer.v_proj"]).reshape(T, 1, hd)
            if position_kind == "rotary":
                k = pm.apply_rope(k, range(T), inv)
            caches[cache_key] = (k, v)
        k, v = caches[cache_key]
        if position_kind == "rotary":
            q = pm.apply_rope(q, range(T), inv)
        else:
            q = q.copy(); q[:, :, 0] += pm.f32(0.01 * np.arange(T, dtype=np.float32))[:, None]
        return pm.linear(pm.attention(q, k, v, np.arange(T)).reshape(T, nq * hd), w[prefix + "mixer.o_proj"])

    def swiglu_ff(prefix, h):
        return pm.linear(pm.swiglu(pm.linear(h, w[prefix + "feed_forward.gate_proj"]), pm.linear(h, w[prefix + "feed_forward.up_proj"])),
                         w[prefix + "feed_forward.down_proj"])

    def routed_ff(prefix, h):
        pick = (h @ w[prefix + "feed_forward.router"].T).argmax(-1)
        return np.where((pick == 0)[:, None], h @ w[prefix + "feed_forward.expert0"].T, h @ w[prefix + "feed_forward.expert1"].T)

    runs = [("l0.", "mean", swiglu_ff, None, None, None), ("l1.", "attn", routed_ff, "rotary", 1, True),
            ("l1.", "attn", routed_ff, "rotary", 2, True), ("l2.", "attn", swiglu_ff, "additive", 1, False)]
    for prefix, kind, ff, pk, ck, writes in runs:
        h = pm.rms_norm(x, w[prefix + "norm_in.weight"], 1e-5)
        a = pm.f32(np.cumsum(h, 0) / np.arange(1, T + 1)[:, None]) if kind == "mean" else attn(prefix, h, pk, ck, writes)
        x = pm.f32(x + a)
        x = pm.f32(x + ff(prefix, pm.rms_norm(x, w[prefix + "norm_post.weight"], 1e-5)))
    return pm.linear(pm.rms_norm(x, w["fn"], 1e-5), w["head"])


def test_toy_parts_register_build_and_step():
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    from aien_sovereign_core_mv_b200.models import Decoder
    from aien_sovereign_core_mv_b200.weights import random_tensors
    register_toy_parts()
    model = Decoder(toy_spec())
    assert [n.kind for n in model.group_needs] == ["state", "full"] and model.group_slots == [1, 2]
    assert [(b.group, b.slot, b.writes) for b in model.bindings] == [(0, 0, True), (1, 0, True), (1, 1, True), (1, 0, False)]
    tensors = dict(random_tensors(model.catalog(), 5))
    assert "l1.feed_forward.router" in tensors and "l2.mixer.k_proj" in tensors
    model.bind((n, t.float()) for n, t in tensors.items())
    eng = Engine(model, None, EngineConfig(dtype="float32", page_size=4, max_cache_tokens=128, max_requests=4, max_batch_tokens=64,
                                            max_context=64))
    w = {n: t.double().numpy() for n, t in tensors.items()}
    reqs = {1: H.tokens_for("A", 23, 1), 2: H.tokens_for("A", 9, 2), 3: H.tokens_for("A", 14, 3)}
    reqs = {r: [t % 97 for t in toks] for r, toks in reqs.items()}
    want = {r: toy_plain(w, toks) for r, toks in reqs.items()}
    whole = H.run_steps(eng, [([(r, toks, list(range(len(toks))))], [r]) for r, toks in reqs.items()])
    for r in reqs:
        H.assert_close(np.stack([whole[r][p] for p in range(len(reqs[r]))]), want[r], H.FP32_TOL, f"toy model whole, request {r}")
    # the same in portions and single tokens, two requests at a time: the state slots carry over
    steps = [([(1, reqs[1][:5], range(5)), (2, reqs[2][:2], range(2))], []),
             ([(1, reqs[1][5:6], [0]), (2, reqs[2][2:9], range(7))], [2]),
             ([(1, reqs[1][6:20], range(14)), (3, reqs[3][:1], [0])], []),
             ([(3, reqs[3][1:], range(13)), (1, reqs[1][20:], range(3))], [1, 3])]
    cut = H.run_steps(eng, steps)
    for r in reqs:
        H.assert_close(np.stack([cut[r][p] for p in range(len(reqs[r]))]), want[r], H.FP32_TOL, f"toy model in portions, request {r}")
    # fork copies the state slot: the child goes on as the parent would
    H.run_steps(eng, [([(7, reqs[1][:10], [])], [])])
    eng.fork(7, 8)
    a = H.run_steps(eng, [([(7, reqs[1][10:14], range(4)), (8, reqs[1][10:14], range(4))], [7, 8])])
    H.assert_close(np.stack([a[8][p] for p in range(4)]), want[1][10:14], H.FP32_TOL, "forked child")
    H.assert_close(np.stack([a[7][p] for p in range(4)]), want[1][10:14], H.FP32_TOL, "parent after fork")
    assert eng.cache_state()["check"] == "" and eng.cache_state()["requests"] == 0


def test_windowed_attention_model_frees_pages():
    """A model whose layers alternate between all keys and a window of 12: two cache groups with
    pages of their own; the windowed group gives pages back while the request runs."""
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig, LayerSpec, ModelSpec, PartSpec, model_spec_for
    from aien_sovereign_core_mv_b200.models import Decoder
    from aien_sovereign_core_mv_b200.weights import random_tensors
    raw = dict(H.TINY["A"]); raw["num_hidden_layers"] = 3
    _, spec = model_spec_for(raw)
    layers = list(spec.layers)
    wp = dict(layers[1].mixer.params); wp["window"] = 12
    layers[1] = dataclasses.replace(layers[1], mixer=PartSpec("paged_attention", wp))
    spec = dataclasses.replace(spec, layers=tuple(layers))
    for dtype, tol in (("float32", H.FP32_TOL), ("bfloat16", H.BF16_TOL)):
        model = Decoder(spec)
        assert [n.kind for n in model.group_needs] == ["full", "window"] and model.group_slots == [2, 1]
        tensors = dict(random_tensors(model.catalog(), 9))
        model.bind((n, t if dtype == "bfloat16" else t.float()) for n, t in tensors.items())
        eng = Engine(model, None, EngineConfig(dtype=dtype, page_size=4, max_cache_tokens=128, max_requests=4, max_batch_tokens=64,
                                                max_context=128))
        w = {n: t.double().numpy() for n, t in tensors.items()}
        toks = H.tokens_for("A", 90, 77)
        # plain: layer 1 with a window
        T = len(toks)
        x = w["model.embed_tokens.weight"][toks]
        inv = pm.rope_inv_freq(16, 10000.0)
        for l in range(3):
            p = f"model.layers.{l}."
            h = pm.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
            q = pm.apply_rope(pm.linear(h, w[p + "self_attn.q_proj.weight"]).reshape(T, 4, 16), range(T), inv)
            k = pm.apply_rope(pm.linear(h, w[p + "self_attn.k_proj.weight"]).reshape(T, 2, 16), range(T), inv)
            v = pm.linear(h, w[p + "self_attn.v_proj.weight"]).reshape(T, 2, 16)
            o = pm.attention(q, k, v, np.arange(T), 12 if l == 1 else None).reshape(T, 64)
            x = pm.f32(x + pm.linear(o, w[p + "self_attn.o_proj.weight"]))
            h = pm.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
            x = pm.f32(x + pm.linear(pm.swiglu(pm.linear(h, w[p + "mlp.gate_proj.weight"]), pm.linear(h, w[p + "mlp.up_proj.weight"])), w[p + "mlp.down_proj.weight"]))
        want = pm.linear(pm.rms_norm(x, w["model.norm.weight"], 1e-5), w["lm_head.weight"])
        steps = [([(1, toks[:30], range(30))], []), ([(1, toks[30:37], range(7))], [])] + [([(1, [t], [0])], []) for t in toks[37:]]
        got = H.run_steps(eng, steps)
        H.assert_close(np.stack([got[1][p] for p in range(T)]), want, tol, f"windowed model {dtype}")
        st = eng.cache_state()
        assert st["metrics"]["window_releases"] >= 15 and st["free_pages"][1] >= 32 - 5 and st["free_pages"][0] == 32 - 23


# ---------------------------------------------------------------------------- more toy parts: other arrangements, other ends, another cache
def register_more_toy_parts():
    from aien_sovereign_core_mv_b200 import kernels as K
    from aien_sovereign_core_mv_b200 import register_block, register_embedding, register_head, register_mixer
    from aien_sovereign_core_mv_b200.parts import Block, CacheNeed, Embedding, Head, Mixer, add_to_residual, linear

    @register_block("toy_postnorm")
    class PostNorm(Block):
        """x = norm_mixer(x + mixer(x)); x = norm_ff(x + ff(x)): the stream itself is normed."""
        norm_slots = ("norm_mixer", "norm_ff")

        def __init__(self, mixer, feed_forward, norm_mixer, norm_ff):
            self.mixer, self.feed_forward, self.norm_mixer, self.norm_ff = mixer, feed_forward, norm_mixer, norm_ff

        def parts(self):
            return {"norm_mixer": self.norm_mixer, "mixer": self.mixer, "norm_ff": self.norm_ff, "feed_forward": self.feed_forward}

        def forward(self, ctx, x, delta, run):
            add_to_residual(ctx, x, delta)                    # what the block before left pending
            a = self.mixer.forward(ctx, x.to(ctx.dtype), run)
            x.copy_(self.norm_mixer.forward(ctx, x, a))       # the norm adds a to x first
            f = self.feed_forward.forward(ctx, x.to(ctx.dtype))
            x.copy_(self.norm_ff.forward(ctx, x, f))
            return None

    @register_block("toy_mixer_only")
    class MixerOnly(Block):
        """x += mixer(norm(x)); no feed-forward."""
        norm_slots = ("norm",)

        def __init__(self, mixer, feed_forward, norm):
            assert feed_forward is None
            self.mixer, self.norm = mixer, norm

        def parts(self):
            return {"norm": self.norm, "mixer": self.mixer}

        def forward(self, ctx, x, delta, run):
            return self.mixer.forward(ctx, self.norm.forward(ctx, x, delta), run)

    @register_embedding("toy_scaled")
    class Scaled(Embedding):
        def __init__(self, vocab_size, hidden_size, scale):
            self.shape, self.scale = (vocab_size, hidden_size), float(scale)

        def param_shapes(self):
            return {"weight": (self.shape, "embedding")}

        def bind(self, tensors):
            self.weight = tensors["weight"].contiguous()

        def tied_weight(self):
            return self.weight

        def forward(self, ctx, token_ids, x):
            K.embed_gather(self.weight, token_ids, x)
            x.mul_(self.scale)

    @register_head("toy_softcap")
    class SoftCap(Head):
        """logits = cap * tanh((rows . W^T + bias) / cap), W the embedding's table."""
        tied = True

        def __init__(self, vocab_size, hidden_size, cap):
            self.vocab_size, self.cap = vocab_size, float(cap)

        def param_shapes(self):
            return {"bias": ((self.vocab_size,), "norm")}

        def bind(self, tensors):
            self.bias = tensors["bias"].float()

        def tie(self, embedding):
            self.weight = embedding.tied_weight()

        def forward(self, ctx, rows, logits):
            linear(ctx, rows, self.weight, out=logits)
            logits.copy_(self.cap * torch.tanh((logits + self.bias) / self.cap))

    @register_mixer("toy_latent")
    class Latent(Mixer):
        """One latent vector per token in the cache (a single plane, not keys and values): c = Wd h
        is stored; a token attends over the latents up to its own, o = softmax(q . c / sqrt(r)) c
        with q = Wq h, and y = Wu o."""

        def __init__(self, hidden_size, rank, position=None):
            self.hidden_size, self.rank = hidden_size, rank

        def param_shapes(self):
            return {"down": ((self.rank, self.hidden_size), "matrix"), "q": ((self.rank, self.hidden_size), "matrix"),
                    "up": ((self.hidden_size, self.rank), "matrix")}

        def bind(self, tensors):
            self.t = {k: v.float() for k, v in tensors.items()}

        def cache_need(self):
            return CacheNeed("full", planes=(("latent", (self.rank,)),))

        def forward(self, ctx, h, run):
            g = ctx.groups[run.group]
            plane = g.storage["latent"][run.slot]                 # [tokens of the pool, rank]
            T, ps = ctx.num_tokens, g.page_size
            x = h.float()
            c = (x @ self.t["down"].T).to(plane.dtype)
            slots = g.slot_map[:T].long()
            plane[slots.clamp(min=0)] = torch.where((slots >= 0)[:, None], c, plane[slots.clamp(min=0)])
            q = x @ self.t["q"].T
            j = torch.arange(max(ctx.max_ctx_len, 1), device=h.device)
            table = g.block_table[ctx.seq_of_token[:T].long()].long()                    # [T, max_blocks]
            page = table.gather(1, (j // ps).clamp(max=g.max_blocks - 1)[None].expand(T, -1))
            seen = j[None] <= ctx.positions[:T].long()[:, None]
            keys = plane[torch.where(seen, page * ps + j % ps, 0)].float()              # [T, kmax, rank]
            s = ((keys * q[:, None]).sum(-1) / math.sqrt(self.rank)).masked_fill(~seen, float("-inf"))
            o = (torch.softmax(s, -1)[..., None] * keys).sum(1)
            return (o @ self.t["up"].T).to(h.dtype)


def toy_spec_two():
    from aien_sovereign_core_mv_b200 import LayerSpec, ModelSpec, PartSpec, RunEntry
    Hd, V = 40, 61
    swiglu = PartSpec("swiglu", {"hidden_size": Hd, "intermediate_size": 56})
    layers = (
        LayerSpec("toy_postnorm", PartSpec("toy_latent", {"hidden_size": Hd, "rank": 12}), swiglu, None, PartSpec("none", {}), "a.",
                  norms={"norm_mixer": PartSpec("rmsnorm", {"eps": 1e-5}), "norm_ff": PartSpec("rmsnorm", {"eps": 1e-2})}),
        LayerSpec("toy_mixer_only", PartSpec("toy_latent", {"hidden_size": Hd, "rank": 12}), None, PartSpec("rmsnorm", {"eps": 1e-6}),
                  PartSpec("none", {}), "b."),
        LayerSpec("prenorm", PartSpec("paged_attention", {"hidden_size": Hd, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16}), swiglu,
                  PartSpec("rmsnorm", {"eps": 1e-5}), PartSpec("rotary", {"head_dim": 16, "theta": 10000.0}), "c."),
    )
    return ModelSpec("ToyTwo", Hd, V, layers, (RunEntry(0, 0), RunEntry(1, 1), RunEntry(2, 2)),
                     PartSpec("toy_scaled", {"name": "emb", "scale": math.sqrt(Hd)}), PartSpec("rmsnorm", {"eps": 1e-5, "name": "fn"}),
                     PartSpec("toy_softcap", {"cap": 5.0, "names": {"bias": "head.b"}}), 256)


def toy_two_plain(w, ids, round_cache=None):
    Hd, r = 40, 12
    T = len(ids)
    x = pm.f32(w["emb"][ids] * np.float32(math.sqrt(Hd)))

    def latent(prefix, h):
        c = pm.linear(h, w[prefix + "mixer.down"])
        if round_cache is not None:
            c = round_cache(c)
        q = pm.linear(h, w[prefix + "mixer.q"])
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), (q @ c.T) / math.sqrt(r), -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
        return pm.linear(p @ c, w[prefix + "mixer.up"])

    def swiglu_ff(prefix, h):
        return pm.linear(pm.swiglu(pm.linear(h, w[prefix + "feed_forward.gate_proj"]), pm.linear(h, w[prefix + "feed_forward.up_proj"])),
                         w[prefix + "feed_forward.down_proj"])

    rs = round_cache or (lambda v: v)      # the toy post-norm block keeps the stream in the compute dtype: rounded where it is
    x = rs(pm.rms_norm(pm.f32(x + latent("a.", rs(x))), w["a.norm_mixer.weight"], 1e-5))  # post-norm, each norm its own eps
    x = rs(pm.rms_norm(pm.f32(x + swiglu_ff("a.", x)), w["a.norm_ff.weight"], 1e-2))
    x = pm.f32(x + latent("b.", pm.rms_norm(x, w["b.norm.weight"], 1e-6)))               # mixer only
    h = pm.rms_norm(x, w["c.norm_in.weight"], 1e-5)
    inv = pm.rope_inv_freq(16, 10000.0)
    q = pm.apply_rope(pm.linear(h, w["c.mixer.q_proj"]).reshape(T, 2, 16), range(T), inv)
    k = pm.apply_rope(pm.linear(h, w["c.mixer.k_proj"]).reshape(T, 1, 16), range(T), inv)
    v = pm.linear(h, w["c.mixer.v_proj"]).reshape(T, 1, 16)
    x = pm.f32(x + pm.linear(pm.attention(q, k, v, np.arange(T)).reshape(T, 32), w["c.mixer.o_proj"]))
    x = pm.f32(x + swiglu_ff("c.", pm.rms_norm(x, w["c.norm_post.weight"], 1e-5)))
    logits = pm.linear(pm.rms_norm(x, w["fn"], 1e-5), w["emb"]) + w["head.b"]
    return 5.0 * np.tanh(logits / 5.0)


@pytest.mark.parametrize("dtype,tol", [("float32", H.FP32_TOL), ("bfloat16", H.BF16_TOL)])
def test_other_arrangements_ends_and_cache_planes_from_outside_the_package(dtype, tol):
    """A post-norm block with two different norms by slot name, a block with one norm and no
    feed-forward, an embedding that scales, a tied head with a bias and a soft cap, and a mixer
    that caches one latent plane per token: all registered here, built from the spec by the
    generic decoder, their cache allocated by the engine from the declared plane shapes."""
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    from aien_sovereign_core_mv_b200.models import Decoder
    from aien_sovereign_core_mv_b200.weights import random_tensors
    register_more_toy_parts()
    model = Decoder(toy_spec_two())
    assert [(n.kind, n.planes) for n in model.group_needs] == [("full", (("latent", (12,)),)), ("full", (("k", (1, 16)), ("v", (1, 16))))]
    assert model.group_slots == [2, 1] and model.tied
    cat = model.catalog()
    assert {"emb", "fn", "head.b", "a.norm_mixer.weight", "a.norm_ff.weight", "b.norm.weight", "b.mixer.down"} <= set(cat) and "b.feed_forward.gate_proj" not in cat
    tensors = dict(random_tensors(cat, 6))
    model.bind((n, t if dtype == "bfloat16" else t.float()) for n, t in tensors.items())
    eng = Engine(model, None, EngineConfig(dtype=dtype, page_size=4, max_cache_tokens=96, max_requests=4, max_batch_tokens=64, max_context=64))
    assert {n: tuple(t.shape) for n, t in eng.storage[0].items()} == {"latent": (2, 96, 12)}
    assert {n: tuple(t.shape) for n, t in eng.storage[1].items()} == {"k": (1, 96, 1, 16), "v": (1, 96, 1, 16)}
    w = {n: t.double().numpy() for n, t in tensors.items()}
    reqs = {1: [t % 61 for t in H.tokens_for("A", 21, 4)], 2: [t % 61 for t in H.tokens_for("A", 10, 5)]}
    rc = pm.round_bf16 if dtype == "bfloat16" else None
    want = {r: toy_two_plain(w, toks, rc) for r, toks in reqs.items()}
    whole = H.run_steps(eng, [([(r, toks, list(range(len(toks))))], [r]) for r, toks in reqs.items()])
    for r in reqs:
        H.assert_close(np.stack([whole[r][p] for p in range(len(reqs[r]))]), want[r], tol, f"second toy model whole, request {r}")
    steps = [([(1, reqs[1][:7], range(7)), (2, reqs[2][:3], range(3))], []),
             ([(1, reqs[1][7:8], [0]), (2, reqs[2][3:], range(7))], [2])]
    steps += [([(1, [t], [0])], []) for t in reqs[1][8:]]
    cut = H.run_steps(eng, steps)
    for r in reqs:
        H.assert_close(np.stack([cut[r][p] for p in range(len(reqs[r]))]), want[r], tol, f"second toy model in portions, request {r}")
    eng.fork(1, 5, 10)                                        # copy-on-write copies every plane of the page
    a = H.run_steps(eng, [([(5, reqs[1][10:13], range(3))], [1, 5])])
    H.assert_close(np.stack([a[5][p] for p in range(3)]), want[1][10:13], tol, "child forked inside a page")
    assert eng.cache_state()["check"] == "" and eng.cache_state()["requests"] == 0


def test_state_mixer_on_the_device_keeps_cuda_graphs():
    """The first toy model in bfloat16: its running-mean mixer follows the device-side contract of
    fixed-size state, so decode steps are captured and replayed as CUDA graphs (three requests in
    a graph of four rows: the padding row is pointed at the slot that belongs to nobody)."""
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    from aien_sovereign_core_mv_b200.models import Decoder
    from aien_sovereign_core_mv_b200.weights import random_tensors
    register_toy_parts()
    model = Decoder(toy_spec())
    tensors = dict(random_tensors(model.catalog(), 5))
    model.bind(iter(tensors.items()))
    eng = Engine(model, None, EngineConfig(dtype="bfloat16", page_size=4, max_cache_tokens=128, max_requests=4, max_batch_tokens=64,
                                            max_context=64))
    assert eng._graphable and not eng._replayable            # parts from outside the package: graphs yes, recorded launches no
    w = {n: t.double().numpy() for n, t in tensors.items()}
    reqs = {r: [t % 97 for t in H.tokens_for("A", n, r)] for r, n in ((1, 19), (2, 12), (3, 15))}
    want = {r: toy_plain(w, toks) for r, toks in reqs.items()}
    H.run_steps(eng, [([(r, toks[:6], []) for r, toks in reqs.items()], [])])
    steps = [([(r, [toks[6 + s]], [0]) for r, toks in reqs.items()], []) for s in range(6)]
    got = H.run_steps(eng, steps)
    assert len(eng._graphs) >= 1
    for r in reqs:
        H.assert_close(np.stack([got[r][p] for p in range(6)]), want[r][6:12], H.BF16_TOL, f"state mixer under graphs, request {r}")
