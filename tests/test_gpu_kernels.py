"""Each kernel alone against a plain float32 (or float64) restatement in torch/numpy, at sizes
other than the engine's: widths and vocabularies that are no power of two, head sizes in steps
of 16, odd numbers of heads and groups, and inputs made so that a single far key or a window's
edge decides the result."""
import math

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as pm

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from aien_sovereign_core_mv_b200 import kernels
    kernels.lib()
    return kernels


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).cuda() if not isinstance(a, torch.Tensor) else a.to("cuda", dtype)


def tol_for(dtype):
    return 2e-5 if dtype == torch.float32 else 1.5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (3, 130, 77), (65, 64, 16), (130, 333, 200), (2, 1000, 1031)])
def test_gemm_simple(K, dtype, M, N, K_):
    g = torch.Generator().manual_seed(M * 1000 + N)
    a = torch.randn(M, K_, generator=g).to(dtype).cuda()
    w = torch.randn(N, K_, generator=g).to(dtype).cuda()
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    K.gemm_simple(a, w, out)
    want = a.double().cpu() @ w.double().cpu().T
    H.assert_close(out.float().cpu().numpy(), want.numpy(), tol_for(dtype), f"gemm {M}x{N}x{K_}")
    # float32 logits out of bfloat16 operands, strided input rows
    big = torch.randn(M, K_ + 9, generator=g).to(dtype).cuda()
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    K.gemm_simple(big[:, 4:4 + K_], w, out32)
    want = big[:, 4:4 + K_].double().cpu() @ w.double().cpu().T
    H.assert_close(out32.cpu().numpy(), want.numpy(), 2e-5, "gemm strided, f32 out")


def test_gemm_rows_do_not_depend_on_batch(K):
    g = torch.Generator().manual_seed(5)
    a = torch.randn(70, 200, generator=g).cuda()
    w = torch.randn(90, 200, generator=g).cuda()
    full = torch.empty(70, 90, device="cuda")
    K.gemm_simple(a, w, full)
    one = torch.empty(1, 90, device="cuda")
    for r in (0, 37, 69):
        K.gemm_simple(a[r:r + 1], w, one)
        assert torch.equal(one[0], full[r])          # bit-identical


@pytest.mark.parametrize("hdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,Hd", [(1, 72), (5, 96), (3, 4100)])
def test_embed_and_add_rmsnorm(K, hdt, T, Hd):
    g = torch.Generator().manual_seed(T + Hd)
    table = torch.randn(50, Hd, generator=g).to(hdt).cuda()
    ids = torch.tensor([(7 * i + 3) % 50 for i in range(T)], dtype=torch.int32).cuda()
    x = torch.empty(T, Hd, device="cuda")
    K.embed_gather(table, ids, x)
    assert torch.equal(x, table.float()[ids.long()])
    delta = torch.randn(T, Hd, generator=g).to(hdt).cuda()
    w = (torch.rand(Hd, generator=g) * 0.4 + 0.8).to(hdt).cuda()
    x0 = x.clone()
    out = torch.empty(T, Hd, dtype=hdt, device="cuda")
    K.add_rmsnorm(x, delta, w, 1e-5, out)
    xs = (x0 + delta.float()).cpu().numpy()
    assert np.array_equal(x.cpu().numpy(), xs.astype(np.float32))
    want = pm.rms_norm(xs, w.float().cpu().numpy().astype(np.float64), 1e-5)
    H.assert_close(out.float().cpu().numpy(), want, tol_for(hdt), "rmsnorm")
    rows = torch.tensor([T - 1, 0], dtype=torch.int32).cuda()
    got = torch.empty(2, Hd, device="cuda")
    K.gather_add_rows(x0, delta, rows, got)
    assert np.array_equal(got.cpu().numpy(), xs[[T - 1, 0]].astype(np.float32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(K, dtype):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(5, 2 * 77, generator=g) * 3).to(dtype).cuda()
    out = torch.empty(5, 77, dtype=dtype, device="cuda")
    K.swiglu(gu, out)
    want = pm.swiglu(gu[:, :77].double().cpu().numpy(), gu[:, 77:].double().cpu().numpy())
    H.assert_close(out.float().cpu().numpy(), want, tol_for(dtype), "swiglu")


def test_rope_table_far_positions(K):
    inv = torch.tensor(pm.rope_inv_freq(48, 1e6), dtype=torch.float64).cuda()
    pos = torch.tensor([0, 1, 17, 4095, 131071], dtype=torch.int32).cuda()
    cos = torch.empty(5, 24, device="cuda"); sin = torch.empty(5, 24, device="cuda")
    K.rope_table(pos, inv, cos, sin)
    ang = pos.cpu().numpy().astype(np.float64)[:, None] * inv.cpu().numpy()[None]
    assert np.abs(cos.cpu().numpy() - np.cos(ang)).max() <= 1.2e-7
    assert np.abs(sin.cpu().numpy() - np.sin(ang)).max() <= 1.2e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,rot,norm", [(4, 2, 16, 16, False), (6, 3, 48, 48, True), (5, 1, 80, 32, True), (2, 2, 256, 256, True),
                                                 (8, 2, 128, 128, True), (3, 3, 128, 128, False), (6, 2, 128, 64, True)])   # 128: the vectorised kernel (bfloat16, full rotation)
def test_qk_norm_rope_kv_write(K, dtype, nq, nkv, hd, rot, norm):
    T, slots = 7, 40
    g = torch.Generator().manual_seed(nq * hd)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, generator=g).to(dtype).cuda()
    q, k, v = qkv[:, :nq * hd], qkv[:, nq * hd:(nq + nkv) * hd], qkv[:, (nq + nkv) * hd:]
    qw = (torch.rand(hd, generator=g) * 0.4 + 0.8).to(dtype).cuda() if norm else None
    kw = (torch.rand(hd, generator=g) * 0.4 + 0.8).to(dtype).cuda() if norm else None
    pos = [0, 3, 4, 100, 101, 2000, 7]
    inv = pm.rope_inv_freq(rot, 10000.0)
    cos = torch.empty(T, rot // 2, device="cuda"); sin = torch.empty(T, rot // 2, device="cuda")
    K.rope_table(torch.tensor(pos, dtype=torch.int32).cuda(), torch.tensor(inv, dtype=torch.float64).cuda(), cos, sin)
    slot_map = torch.tensor([5, 6, 39, 0, 17, -1, 8], dtype=torch.int32).cuda()
    kc = torch.full((slots, nkv, hd), 7.0, dtype=dtype, device="cuda"); vc = torch.full((slots, nkv, hd), 7.0, dtype=dtype, device="cuda")
    q0, k0, v0 = (t.float().cpu().numpy().astype(np.float64) for t in (q, k, v))
    K.qk_norm_rope_kv_write(q, k, v, hd, qw, kw, 1e-6, cos, sin, rot, slot_map, kc, vc)

    def ref(x, heads, w):
        x = x.reshape(T, heads, hd)
        if w is not None:
            x = pm.rms_norm(x, w.float().cpu().numpy().astype(np.float64), 1e-6)
        r = pm.apply_rope(x[..., :rot], pos, inv)
        return np.concatenate([r, x[..., rot:]], -1)
    H.assert_close(q.float().cpu().numpy().reshape(T, nq, hd), ref(q0, nq, qw), tol_for(dtype), "q")
    kref, kcn, vcn = ref(k0, nkv, kw), kc.float().cpu().numpy(), vc.float().cpu().numpy()
    sm = slot_map.cpu().numpy()
    for t in range(T):
        if sm[t] >= 0:
            H.assert_close(kcn[sm[t]], kref[t], tol_for(dtype), f"k token {t}")
            H.assert_close(vcn[sm[t]], v0.reshape(T, nkv, hd)[t], tol_for(dtype), f"v token {t}")
    untouched = [s for s in range(slots) if s not in set(sm.tolist())]
    assert (kcn[untouched] == 7.0).all() and (vcn[untouched] == 7.0).all()     # a token without a slot writes nothing


@pytest.mark.parametrize("nq,nkv,norm", [(5, 2, True), (8, 1, False), (16, 8, True), (32, 8, False), (6, 2, True)])
def test_qk_kernel_head128_many_tokens(K, nq, nkv, norm):
    """The prompt-portion form of the head-128 q/k kernel (128 tokens and more): a token count that
    is no multiple of its group of four, head counts that are no multiple of its eight warps,
    tokens without a cache slot, q rotated in place."""
    g = torch.Generator().manual_seed(nq)
    T, hd, slots = 131, 128, 200
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, generator=g).to(torch.bfloat16).cuda()
    q, k, v = qkv[:, :nq * hd], qkv[:, nq * hd:(nq + nkv) * hd], qkv[:, (nq + nkv) * hd:]
    qw = (torch.rand(hd, generator=g) * 0.4 + 0.8).to(torch.bfloat16).cuda() if norm else None
    kw = (torch.rand(hd, generator=g) * 0.4 + 0.8).to(torch.bfloat16).cuda() if norm else None
    pos = [(37 * t) % 5000 for t in range(T)]
    inv = pm.rope_inv_freq(hd, 10000.0)
    cos = torch.empty(T, hd // 2, device="cuda"); sin = torch.empty(T, hd // 2, device="cuda")
    K.rope_table(torch.tensor(pos, dtype=torch.int32).cuda(), torch.tensor(inv, dtype=torch.float64).cuda(), cos, sin)
    sm = np.array([-1 if t % 17 == 3 else (t * 7) % slots for t in range(T)], dtype=np.int32)
    assert len(set(sm[sm >= 0].tolist())) == (sm >= 0).sum()
    kc = torch.full((slots, nkv, hd), 7.0, dtype=torch.bfloat16, device="cuda"); vc = torch.full_like(kc, 7.0)
    q0, k0, v0 = (t.float().cpu().numpy().astype(np.float64) for t in (q, k, v))
    K.qk_norm_rope_kv_write(q, k, v, hd, qw, kw, 1e-6, cos, sin, hd, torch.tensor(sm).cuda(), kc, vc)

    def ref(x, heads, w):
        x = x.reshape(T, heads, hd)
        if w is not None:
            x = pm.rms_norm(x, w.float().cpu().numpy().astype(np.float64), 1e-6)
        return pm.apply_rope(x, pos, inv)
    H.assert_close(q.float().cpu().numpy().reshape(T, nq, hd), ref(q0, nq, qw), 1e-2, "q")
    kref, kcn, vcn = ref(k0, nkv, kw), kc.float().cpu().numpy(), vc.float().cpu().numpy()
    live = sm >= 0
    H.assert_close(kcn[sm[live]], kref[live], 1e-2, "k rows")
    H.assert_close(vcn[sm[live]], v0.reshape(T, nkv, hd)[live], 1e-2, "v rows")
    untouched = [s_ for s_ in range(slots) if s_ not in set(sm.tolist())]
    assert (kcn[untouched] == 7.0).all() and (vcn[untouched] == 7.0).all()


def paged_setup(rng, seq_lens, nkv, hd, page, dtype, n_pages):
    """Random K/V for each request scattered over shuffled pages; returns caches, tables, dense copies."""
    perm = rng.permutation(n_pages)
    kc = torch.zeros(n_pages * page, nkv, hd); vc = torch.zeros(n_pages * page, nkv, hd)
    max_blocks = max((n + page - 1) // page for n in seq_lens) + 1
    bt = np.full((len(seq_lens), max_blocks), -1, dtype=np.int32)
    dense, nxt = [], 0
    for s, n in enumerate(seq_lens):
        k = torch.tensor(rng.standard_normal((n, nkv, hd)), dtype=torch.float32).to(dtype).float()
        v = torch.tensor(rng.standard_normal((n, nkv, hd)), dtype=torch.float32).to(dtype).float()
        dense.append((k, v))
        for b in range((n + page - 1) // page):
            pg = int(perm[nxt]); nxt += 1
            bt[s, b] = pg
            lo, hi = b * page, min(n, (b + 1) * page)
            kc[pg * page:pg * page + hi - lo] = k[lo:hi]
            vc[pg * page:pg * page + hi - lo] = v[lo:hi]
    return kc.to(dtype).cuda(), vc.to(dtype).cuda(), torch.tensor(bt).cuda(), max_blocks, dense


def attention_reference(q, dense, seq_of, positions, nq, nkv, hd, window, scale):
    out = np.zeros((len(seq_of), nq, hd))
    for t, (s, p) in enumerate(zip(seq_of, positions)):
        k, v = dense[s]
        lo = max(0, p - window + 1) if window > 0 else 0
        kk, vv = k[lo:p + 1].double().numpy(), v[lo:p + 1].double().numpy()
        for h in range(nq):
            sc = (kk[:, h // (nq // nkv)] @ q[t, h]) * scale
            e = np.exp(sc - sc.max()); e /= e.sum()
            out[t, h] = e @ vv[:, h // (nq // nkv)]
    return out.reshape(len(seq_of), nq * hd)


ATT_CASES = [(4, 2, 16, 16, 0), (6, 3, 48, 8, 0), (5, 1, 80, 16, 0), (8, 2, 128, 16, 0), (3, 3, 32, 4, 21), (2, 1, 256, 32, 0), (8, 4, 64, 16, 40)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,page,window", ATT_CASES)
def test_paged_attention_generic(K, dtype, nq, nkv, hd, page, window):
    rng = np.random.default_rng(nq * 100 + hd)
    seq_lens = [1, 37, 300, 129]
    kc, vc, bt, mb, dense = paged_setup(rng, seq_lens, nkv, hd, page, dtype, 64 * 16 // page + 8)
    # tokens: decode rows (last position), a portion in the middle of request 2, the first tokens of request 1
    seq_of = [0, 1, 2, 3] + [2] * 9 + [1, 1, 1]
    positions = [0, 36, 299, 128] + list(range(250, 259)) + [0, 1, 2]
    q = torch.tensor(rng.standard_normal((len(seq_of), nq * hd)), dtype=torch.float32).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty(len(seq_of), nq * hd, dtype=dtype, device="cuda")
    K.paged_attention_generic(q.cuda(), kc, vc, bt, mb, torch.tensor(seq_of, dtype=torch.int32).cuda(),
                              torch.tensor(positions, dtype=torch.int32).cuda(), out, nq, nkv, hd, page, window, scale)
    want = attention_reference(q.float().double().numpy().reshape(-1, nq, hd), dense, seq_of, positions, nq, nkv, hd, window, scale)
    H.assert_close(out.float().cpu().numpy(), want, tol_for(dtype), "attention")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_one_far_key_decides(K, dtype):
    """Among 600 keys one far key matches the query; the output must be that key's value.  A kernel
    that drops a page, misreads a table entry or stops early cannot pass."""
    nq, nkv, hd, page = 2, 1, 64, 16
    n = 600
    for far in (0, 15, 16, 303, 599):
        kc = torch.zeros(48 * page, nkv, hd); vc = torch.zeros(48 * page, nkv, hd)
        perm = np.random.default_rng(far).permutation(48)
        bt = np.full((1, 40), -1, dtype=np.int32)
        for b in range((n + page - 1) // page):
            bt[0, b] = perm[b]
        slot = lambda j: int(bt[0, j // page]) * page + j % page
        for j in range(n):
            vc[slot(j), 0, :] = j
        kc[slot(far), 0, 0] = 40.0
        q = torch.zeros(1, nq * hd); q[0, 0] = 8.0; q[0, hd] = 8.0
        out = torch.empty(1, nq * hd, dtype=dtype, device="cuda")
        K.paged_attention_generic(q.to(dtype).cuda(), kc.to(dtype).cuda(), vc.to(dtype).cuda(), torch.tensor(bt).cuda(), 40,
                                  torch.zeros(1, dtype=torch.int32).cuda(), torch.tensor([n - 1], dtype=torch.int32).cuda(),
                                  out, nq, nkv, hd, page, 0, 1.0 / math.sqrt(hd))
        got = out.float().cpu().numpy()
        assert np.abs(got - far).max() <= max(1e-3, 0.01 * far), (far, got[0, :4])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_window_edge(K, dtype):
    """The key just outside the window carries a huge score: it must not be seen; the one just
    inside must."""
    nq, nkv, hd, page, window, n = 1, 1, 32, 8, 24, 100
    bt = np.arange(16, dtype=np.int32)[None]
    for outside in (True, False):
        kc = torch.zeros(16 * page, nkv, hd); vc = torch.zeros(16 * page, nkv, hd)
        for j in range(n):
            vc[j, 0, :] = 1.0
        edge = (n - 1) - window + (0 if outside else 1)
        kc[edge, 0, 0] = 50.0
        vc[edge, 0, :] = -5.0
        q = torch.zeros(1, hd); q[0, 0] = 8.0
        out = torch.empty(1, hd, dtype=dtype, device="cuda")
        K.paged_attention_generic(q.to(dtype).cuda(), kc.to(dtype).cuda(), vc.to(dtype).cuda(), torch.tensor(bt).cuda(), 16,
                                  torch.zeros(1, dtype=torch.int32).cuda(), torch.tensor([n - 1], dtype=torch.int32).cuda(),
                                  out, nq, nkv, hd, page, window, 1.0 / math.sqrt(hd))
        got = out.float().cpu().numpy()
        assert np.allclose(got, 1.0 if outside else -5.0, atol=2e-2), (outside, got[0, :3])


def test_argmax_and_sampling(K):
    from aien_sovereign_core_mv_b200.sampling import philox_uniform
    rng = np.random.default_rng(0)
    R, V = 6, 1537
    logits = rng.standard_normal((R, V)).astype(np.float32) * 3
    logits[0, 700] = logits[0, 30] = logits[0].max() + 1      # tie: the lower id wins
    lg = torch.tensor(logits).cuda()
    ids = torch.empty(R, dtype=torch.int32, device="cuda")
    K.argmax_rows(lg, ids)
    assert ids.cpu().tolist() == [pm.argmax_token(r) for r in logits]
    temp = [0.0, 0.7, 1.0, 1.3, 0.7, 0.0005]
    top_p = [1.0, 0.95, 1.0, 0.5, 0.9, 0.3]
    top_k = [0, 0, 40, 0, 5, 3]
    seeds = [11, 12, 13, 14, 15, 16]
    rids = [1, 2, 3, 4, 2 ** 40 + 5, 6]
    scratch = torch.empty(R * V, device="cuda")
    for position in (0, 1, 77, 100000):
        K.sample_rows(lg, torch.tensor(temp).cuda(), torch.tensor(top_p).cuda(), torch.tensor(top_k, dtype=torch.int32).cuda(),
                      torch.tensor(seeds, dtype=torch.int64).cuda(), torch.tensor(rids, dtype=torch.int64).cuda(),
                      torch.full((R,), position, dtype=torch.int32).cuda(), scratch, ids)
        got = ids.cpu().tolist()
        for r in range(R):
            u = philox_uniform(seeds[r], rids[r], position)
            assert got[r] == pm.sample_token(logits[r], temp[r], top_p[r], top_k[r], u), (position, r)
    # the draws follow the distribution: many positions, one row
    counts = np.zeros(V)
    row = torch.tensor(logits[2:3]).cuda()
    one = torch.empty(1, dtype=torch.int32, device="cuda")
    for position in range(300):
        K.sample_rows(row, torch.tensor([1.0]).cuda(), torch.tensor([1.0]).cuda(), torch.tensor([8], dtype=torch.int32).cuda(),
                      torch.tensor([5], dtype=torch.int64).cuda(), torch.tensor([9], dtype=torch.int64).cuda(),
                      torch.tensor([position], dtype=torch.int32).cuda(), scratch, one)
        counts[one.item()] += 1
    kept, probs = pm.kept_set(logits[2], 1.0, 1.0, 8)
    assert counts.sum() == counts[kept].sum()
    assert counts[int(np.argmax(logits[2]))] == counts.max()


def test_sampling_at_a_large_vocabulary(K):
    """A vocabulary of 40,013 with a language-model-like row (a few tokens far above the rest) and
    a flat one: the one-pass cases of the sampler (nucleus alone, top-k with and without nucleus)
    and the general path (flat distribution, large k, pure temperature) against the plain sampler."""
    from aien_sovereign_core_mv_b200.sampling import philox_uniform
    rng = np.random.default_rng(7)
    V = 40013
    peaked = (rng.standard_normal(V) * 2).astype(np.float32)
    hot = rng.choice(V, 60, replace=False)
    peaked[hot] = (rng.random(60) * 9 + 9).astype(np.float32)
    flat = (rng.standard_normal(V) * 0.5).astype(np.float32)
    rows = [peaked, peaked, peaked, peaked, peaked, flat, flat]
    temp = [0.7, 0.6, 1.0, 0.7, 1.2, 0.7, 1.0]
    top_p = [0.95, 0.8, 1.0, 0.9, 1.0, 0.95, 0.5]
    top_k = [0, 20, 50, 2000, 0, 0, 40]
    R = len(rows)
    lg = torch.tensor(np.stack(rows)).cuda()
    ids = torch.empty(R, dtype=torch.int32, device="cuda")
    scratch = torch.empty(R * V, device="cuda")
    seeds = list(range(21, 21 + R)); rids = list(range(1, R + 1))
    for position in (0, 5, 9, 123, 4000, 77777):
        K.sample_rows(lg, torch.tensor(temp).cuda(), torch.tensor(top_p).cuda(), torch.tensor(top_k, dtype=torch.int32).cuda(),
                      torch.tensor(seeds, dtype=torch.int64).cuda(), torch.tensor(rids, dtype=torch.int64).cuda(),
                      torch.full((R,), position, dtype=torch.int32).cuda(), scratch, ids)
        got = ids.cpu().tolist()
        for r in range(R):
            kept, _ = pm.kept_set(rows[r], temp[r], top_p[r], top_k[r])
            assert got[r] in kept, (position, r)
            u = philox_uniform(seeds[r], rids[r], position)
            # float32 exponentials against float64: only a draw on an edge may differ
            assert got[r] == pm.sample_token(rows[r], temp[r], top_p[r], top_k[r], u) or H.knife_edge(rows[r], temp[r], top_p[r], top_k[r], u), (position, r)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K_", [(1, 16, 32), (1, 333, 72), (3, 100, 200), (8, 4096, 512), (9, 77, 1032), (16, 130, 4096), (5, 48, 8)])
def test_gemv_against_simple(K, out_dtype, M, N, K_):
    g = torch.Generator().manual_seed(M * 7 + N)
    a_full = torch.randn(M, K_ + 16, generator=g).to(torch.bfloat16).cuda()
    a = a_full[:, 8:8 + K_]                                  # row stride differs from K, still 16-byte aligned
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).cuda()
    assert K.gemv_supports(a, w, torch.empty(M, N, dtype=out_dtype, device="cuda"))
    out = torch.empty(M, N, dtype=out_dtype, device="cuda")
    K.gemv(a, w, out)
    want = a.double().cpu() @ w.double().cpu().T
    H.assert_close(out.float().cpu().numpy(), want.numpy(), 2e-5 if out_dtype == torch.float32 else 1e-2, f"gemv {M}x{N}x{K_}")
    # a row's result does not depend on the other rows
    if M > 1:
        one = torch.empty(1, N, dtype=out_dtype, device="cuda")
        K.gemv(a[M - 1:M], w, one)
        assert torch.equal(one[0], out[M - 1])


def test_gemv_swiglu_epilogue(K):
    g = torch.Generator().manual_seed(1)
    M, I, Hd = 5, 88, 136
    a = torch.randn(M, Hd, generator=g).to(torch.bfloat16).cuda()
    gate = torch.randn(I, Hd, generator=g).to(torch.bfloat16)
    up = torch.randn(I, Hd, generator=g).to(torch.bfloat16)
    inter = torch.stack([gate.view(I // 8, 8, Hd), up.view(I // 8, 8, Hd)], dim=1).reshape(2 * I, Hd).contiguous().cuda()
    out = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    K.gemv(a, inter, out, epilogue=1)
    ad = a.double().cpu()
    want = pm.swiglu((ad @ gate.double().T).numpy(), (ad @ up.double().T).numpy())
    H.assert_close(out.float().cpu().numpy(), want, 1e-2, "gemv+swiglu")


@pytest.mark.parametrize("nq,nkv,hd,page,window", ATT_CASES + [(16, 1, 64, 16, 0), (12, 1, 96, 16, 300)])
def test_paged_attention_decode(K, nq, nkv, hd, page, window):
    dtype = torch.bfloat16
    rng = np.random.default_rng(nq * 10 + hd)
    seq_lens = [1, 37, 700, 256, 257, 513]
    kc, vc, bt, mb, dense = paged_setup(rng, seq_lens, nkv, hd, page, dtype, sum((n + page - 1) // page for n in seq_lens) + 8)
    seq_of = list(range(len(seq_lens)))
    positions = [n - 1 for n in seq_lens]
    T = len(seq_of)
    big = torch.tensor(rng.standard_normal((T, nq * hd + 64)), dtype=torch.float32).to(dtype).cuda()
    q = big[:, 32:32 + nq * hd]
    scale = 1.0 / math.sqrt(hd)
    splits = (max(seq_lens) + 127) // 128
    part_out = torch.empty(T * nq * splits * hd, device="cuda"); part_ml = torch.empty(T * nq * splits * 2, device="cuda")
    out = torch.empty(T, nq * hd, dtype=dtype, device="cuda")
    K.paged_attention_decode(q, kc, vc, bt, mb, torch.tensor(seq_of, dtype=torch.int32).cuda(),
                             torch.tensor(positions, dtype=torch.int32).cuda(), out, part_out, part_ml,
                             nq, nkv, hd, page, window, scale, splits)
    want = attention_reference(q.float().double().cpu().numpy().reshape(-1, nq, hd), dense, seq_of, positions, nq, nkv, hd, window, scale)
    H.assert_close(out.float().cpu().numpy(), want, 1.5e-2, "decode attention")
    ref = torch.empty_like(out)
    K.paged_attention_generic(q, kc, vc, bt, mb, torch.tensor(seq_of, dtype=torch.int32).cuda(),
                              torch.tensor(positions, dtype=torch.int32).cuda(), ref, nq, nkv, hd, page, window, scale)
    H.assert_close(out.float().cpu().numpy(), ref.float().cpu().numpy(), 1e-2, "decode vs generic kernel")
    # a subset of the tokens, named by a list (the single-token entries of a mixed step)
    some = [4, 0, 2]
    sub = torch.full_like(out, 3.0)
    K.paged_attention_decode(q, kc, vc, bt, mb, torch.tensor(seq_of, dtype=torch.int32).cuda(),
                             torch.tensor(positions, dtype=torch.int32).cuda(), sub, part_out, part_ml,
                             nq, nkv, hd, page, window, scale, splits,
                             token_list=torch.tensor(some, dtype=torch.int32).cuda(), num_tokens=len(some))
    assert torch.equal(sub[some], out[some]) and (sub[[1, 3, 5]] == 3.0).all()


# query heads, kv heads, head size, page, window, requests
DECODE_STREAM_CASES = [(8, 2, 128, 16, 0, 6), (32, 8, 128, 16, 0, 40), (16, 1, 64, 8, 0, 5), (12, 4, 64, 32, 300, 7),
                       (5, 5, 128, 128, 0, 9), (9, 1, 128, 64, 150, 3), (32, 8, 128, 16, 200, 70), (4, 2, 64, 16, 0, 200)]


@pytest.mark.parametrize("nq,nkv,hd,page,window,n_req", DECODE_STREAM_CASES)
def test_paged_attention_decode_stream_gives_the_same_bits(K, nq, nkv, hd, page, window, n_req):
    """The streamed kernel (TMA ring, CTAs that take many chunks, tickets per segment) against the
    one-CTA-per-chunk kernel: equal bits, for few and for many requests of mixed lengths, with
    segments of one, two and four chunks, and for a subset of the tokens.  With more (token, kv
    head) pairs than CTAs (the cases of 40, 70 and 200 requests) the chunks of all pairs are cut into
    equal ranges, so pairs are shared between CTAs at arbitrary chunks."""
    dtype = torch.bfloat16
    rng = np.random.default_rng(nq + hd + n_req)
    seq_lens = [1, 37, 700, 256, 257, 513, 128, 129, 1025][:n_req] + [int(x) for x in rng.integers(1, 1100, size=max(0, n_req - 9))]
    kc, vc, bt, mb, dense = paged_setup(rng, seq_lens, nkv, hd, page, dtype, sum((n + page - 1) // page for n in seq_lens) + 8)
    T = len(seq_lens)
    positions = torch.tensor([n - 1 for n in seq_lens], dtype=torch.int32).cuda()
    seq_of = torch.arange(T, dtype=torch.int32).cuda()
    q = torch.tensor(rng.standard_normal((T, nq * hd)), dtype=torch.float32).to(dtype).cuda()
    scale = 1.0 / math.sqrt(hd)
    splits = (max(seq_lens) + 127) // 128
    assert K.decode_stream_supports(nq, nkv, hd, page, splits)
    outs = {}
    for impl in ("direct", "stream"):
        part_out = torch.empty(T * nq * splits * hd, device="cuda"); part_ml = torch.empty(T * nq * splits * 2, device="cuda")
        out = torch.full((T, nq * hd), 5.0, dtype=dtype, device="cuda")
        for _ in range(2):                                    # twice: the ticket counters must come back to zero
            K.paged_attention_decode(q, kc, vc, bt, mb, seq_of, positions, out, part_out, part_ml,
                                     nq, nkv, hd, page, window, scale, splits, impl=impl)
        torch.cuda.synchronize()
        assert K.attention_decode_stream_error() == 0
        outs[impl] = out
    assert torch.equal(outs["stream"], outs["direct"])
    want = attention_reference(q.float().double().cpu().numpy().reshape(-1, nq, hd), dense, list(range(T)), [n - 1 for n in seq_lens],
                               nq, nkv, hd, window, scale)
    H.assert_close(outs["stream"].float().cpu().numpy(), want, 1.5e-2, "streamed decode attention")
    some = [T - 1, 0, 2]
    sub = torch.full_like(out, 3.0)
    K.paged_attention_decode(q, kc, vc, bt, mb, seq_of, positions, sub, part_out, part_ml, nq, nkv, hd, page, window, scale, splits,
                             token_list=torch.tensor(some, dtype=torch.int32).cuda(), num_tokens=len(some), impl="stream")
    rest = [i for i in range(T) if i not in some]
    assert torch.equal(sub[some], outs["direct"][some]) and (sub[rest] == 3.0).all()
    assert K.attention_decode_stream_error() == 0


@pytest.mark.parametrize("nq,nkv,hd,page,window,lens", [(8, 2, 128, 16, 0, [20001, 9000, 130]), (4, 1, 64, 64, 12000, [16500, 1]),
                                                          (6, 2, 96, 16, 0, [8300, 700])])
def test_decode_attention_over_long_contexts(K, nq, nkv, hd, page, window, lens):
    """Up to 157 chunks of 128 keys per token: the merge adds them in eight interleaved series with
    several chunks of a series in flight, beyond one round of every loop; three keys spread over the
    context decide head 0 of every token.  Both kernels (the same bits where both take the shape), with a
    window that starts inside the context.  From 128 chunks on the streamed kernel leaves the merge to a
    kernel of its own (the first two cases), which must add in the same order as the merge inside."""
    dtype = torch.bfloat16
    rng = np.random.default_rng(hd + len(lens))
    kc, vc, bt, mb, dense = paged_setup(rng, lens, nkv, hd, page, dtype, sum((n + page - 1) // page for n in lens) + 8)
    T = len(lens)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    seq_of = torch.arange(T, dtype=torch.int32).cuda()
    q = torch.tensor(rng.standard_normal((T, nq * hd)), dtype=torch.float32).to(dtype).cuda()
    scale = 1.0 / math.sqrt(hd)
    splits = (max(lens) + 127) // 128
    # for head 0 of every token three keys stand out, in chunks that fall into different series and rounds of
    # the merge; a chunk lost or weighed wrongly moves that head's result by a third
    btc = bt.cpu().numpy()
    for s_, n in enumerate(lens):
        lo = max(0, n - window) if window > 0 else 0
        for p_ in sorted({lo + (n - 1 - lo) * f // 100 for f in (3, 47, 96)}):
            kv = (q[s_, :hd].float().cpu() * 1.5).to(dtype)
            dense[s_][0][p_, 0] = kv.float()
            kc[int(btc[s_, p_ // page]) * page + p_ % page, 0] = kv.cuda()
    want = attention_reference(q.float().double().cpu().numpy().reshape(-1, nq, hd), dense, list(range(T)), [n - 1 for n in lens],
                               nq, nkv, hd, window, scale)
    impls = ["direct"] + (["stream"] if K.decode_stream_supports(nq, nkv, hd, page, splits) else [])
    outs = []
    for impl in impls:
        part_out = torch.empty(T * nq * splits * hd, device="cuda"); part_ml = torch.empty(T * nq * splits * 2, device="cuda")
        out = torch.full((T, nq * hd), 5.0, dtype=dtype, device="cuda")
        K.paged_attention_decode(q, kc, vc, bt, mb, seq_of, positions, out, part_out, part_ml, nq, nkv, hd, page, window, scale, splits, impl=impl)
        torch.cuda.synchronize()
        assert K.attention_decode_stream_error() == 0
        H.assert_close(out.float().cpu().numpy(), want, 1.5e-2, f"decode attention over {max(lens)} keys ({impl})")
        outs.append(out)
    if len(outs) == 2:
        assert torch.equal(outs[0], outs[1])


def test_decode_attention_one_far_key_decides(K):
    nq, nkv, hd, page, n = 4, 1, 64, 16, 1500
    for far in (0, 255, 256, 1023, 1499):
        pages = (n + page - 1) // page
        perm = np.random.default_rng(far).permutation(pages + 4)
        bt = np.full((1, pages + 2), -1, dtype=np.int32)
        bt[0, :pages] = perm[:pages]
        slots = (bt[0, np.arange(n) // page] * page + np.arange(n) % page)
        kc = torch.zeros((pages + 4) * page, nkv, hd); vc = torch.zeros((pages + 4) * page, nkv, hd)
        vc[slots, 0, :] = torch.arange(n, dtype=torch.float32)[:, None] / 8.0
        kc[slots[far], 0, 0] = 40.0
        q = torch.zeros(1, nq * hd)
        q[0, ::hd] = 8.0
        splits = (n + 127) // 128
        out = torch.empty(1, nq * hd, dtype=torch.bfloat16, device="cuda")
        K.paged_attention_decode(q.to(torch.bfloat16).cuda(), kc.to(torch.bfloat16).cuda(), vc.to(torch.bfloat16).cuda(),
                                 torch.tensor(bt).cuda(), pages + 2, torch.zeros(1, dtype=torch.int32).cuda(),
                                 torch.tensor([n - 1], dtype=torch.int32).cuda(), out,
                                 torch.empty(nq * splits * hd, device="cuda"), torch.empty(nq * splits * 2, device="cuda"),
                                 nq, nkv, hd, page, 0, 1.0 / math.sqrt(hd), splits)
        got = out.float().cpu().numpy()
        assert np.abs(got - far / 8.0).max() <= max(1e-2, 0.01 * far / 8.0), (far, got[0, :4])


def test_gemv_partial_products_and_their_consumers(K):
    """K cut across CTAs: the partial products add up to the plain product, and the kernels that
    consume them (norm, row gather, q/k kernel) add them on the way in."""
    g = torch.Generator().manual_seed(11)
    M, N, K_ = 3, 96, 2048
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).cuda()
    parts = torch.empty(4, M, N, device="cuda")
    K.gemv(a, w, parts)
    want = (a.double().cpu() @ w.double().cpu().T).numpy()
    H.assert_close(parts.sum(0).cpu().numpy(), want, 2e-5, "sum of partials")
    assert K.gemv_splits(24576, 4096) == 1 and K.gemv_splits(151936, 4096) == 1
    # norm consumes partials
    x = torch.randn(M, N, generator=g).cuda()
    x0 = x.clone()
    wn = torch.ones(N, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    K.add_rmsnorm(x, parts, wn, 1e-6, out)
    xs = x0.double().cpu().numpy() + want
    H.assert_close(x.cpu().numpy(), xs, 2e-5, "residual + partials")
    H.assert_close(out.float().cpu().numpy(), pm.rms_norm(xs, np.ones(N), 1e-6), 1e-2, "norm of residual + partials")
    rows = torch.tensor([2, 0], dtype=torch.int32).cuda()
    got = torch.empty(2, N, device="cuda")
    K.gather_add_rows(x0, parts, rows, got)
    H.assert_close(got.cpu().numpy(), xs[[2, 0]], 2e-5, "gather of residual + partials")
    # q/k kernel consumes partials: heads of 32, 1 q head + 1 kv head
    hd = 32
    q_out = torch.empty(M, hd, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(8, 1, hd, dtype=torch.bfloat16, device="cuda"); vc = torch.zeros(8, 1, hd, dtype=torch.bfloat16, device="cuda")
    slot = torch.tensor([1, 5, 2], dtype=torch.int32).cuda()
    K.qk_norm_rope_kv_write(parts[..., :hd], parts[..., hd:2 * hd], parts[..., 2 * hd:3 * hd], hd, None, None, 1e-6,
                            None, None, 0, slot, kc, vc, q_out=q_out)
    H.assert_close(q_out.float().cpu().numpy(), want[:, :hd], 1e-2, "q from partials")
    H.assert_close(kc[[1, 5, 2], 0].float().cpu().numpy(), want[:, hd:2 * hd], 1e-2, "k from partials")
    H.assert_close(vc[[1, 5, 2], 0].float().cpu().numpy(), want[:, 2 * hd:3 * hd], 1e-2, "v from partials")


def test_qk_kernel_head128_takes_partial_products(K):
    """The vectorised q/k kernel on float32 partial products (what a product cut over K leaves):
    sum, per-head norm, rotation, cache write, against the same values given whole in bfloat16."""
    g = torch.Generator().manual_seed(3)
    T, nq, nkv, hd, P = 7, 4, 2, 128, 3
    width = (nq + 2 * nkv) * hd
    parts = torch.randn(P, T, width, generator=g).cuda()
    whole = parts.sum(0)
    qw = (torch.rand(hd, generator=g) * 0.4 + 0.8).to(torch.bfloat16).cuda()
    kw = (torch.rand(hd, generator=g) * 0.4 + 0.8).to(torch.bfloat16).cuda()
    pos = [0, 3, 4, 100, 101, 2000, 7]
    inv = pm.rope_inv_freq(hd, 10000.0)
    cos = torch.empty(T, hd // 2, device="cuda"); sin = torch.empty(T, hd // 2, device="cuda")
    K.rope_table(torch.tensor(pos, dtype=torch.int32).cuda(), torch.tensor(inv, dtype=torch.float64).cuda(), cos, sin)
    slot_map = torch.tensor([5, 6, 39, 0, 17, -1, 8], dtype=torch.int32).cuda()
    kc = torch.full((40, nkv, hd), 7.0, dtype=torch.bfloat16, device="cuda"); vc = torch.full_like(kc, 7.0)
    q_out = torch.empty(T, nq * hd, dtype=torch.bfloat16, device="cuda")
    K.qk_norm_rope_kv_write(parts[..., :nq * hd], parts[..., nq * hd:(nq + nkv) * hd], parts[..., (nq + nkv) * hd:], hd, qw, kw, 1e-6,
                            cos, sin, hd, slot_map, kc, vc, q_out=q_out)
    w64 = whole.double().cpu().numpy()

    def ref(x, heads, w):
        x = pm.rms_norm(x.reshape(T, heads, hd), w.float().cpu().numpy().astype(np.float64), 1e-6)
        return pm.apply_rope(x, pos, inv)
    H.assert_close(q_out.float().cpu().numpy().reshape(T, nq, hd), ref(w64[:, :nq * hd], nq, qw), 1e-2, "q from partials, head 128")
    kref = ref(w64[:, nq * hd:(nq + nkv) * hd], nkv, kw)
    vref = w64[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
    sm = slot_map.cpu().numpy()
    for t in range(T):
        if sm[t] >= 0:
            H.assert_close(kc[sm[t]].float().cpu().numpy(), kref[t], 1e-2, f"k token {t}")
            H.assert_close(vc[sm[t]].float().cpu().numpy(), vref[t], 1e-2, f"v token {t}")
    untouched = [s_ for s_ in range(40) if s_ not in set(sm.tolist())]
    assert (kc[untouched] == 7.0).all() and (vc[untouched] == 7.0).all()


def test_swiglu_interleaved_layout(K):
    g = torch.Generator().manual_seed(4)
    T, I = 3, 40
    gate = torch.randn(T, I, generator=g); up = torch.randn(T, I, generator=g)
    inter = torch.stack([gate.view(T, I // 8, 8), up.view(T, I // 8, 8)], dim=2).reshape(T, 2 * I).contiguous().cuda()
    out = torch.empty(T, I, device="cuda")
    K.swiglu(inter, out, 8)
    H.assert_close(out.cpu().numpy(), pm.swiglu(gate.double().numpy(), up.double().numpy()), 2e-5, "interleaved swiglu")


# the last three have at least 148 tiles of 128 x 256 and take the persistent kernel (ragged edges in M, N and K)
TC_SHAPES = [(128, 128, 64), (1, 16, 8), (17, 100, 200), (130, 333, 72), (256, 384, 4096), (300, 130, 1032), (2048, 512, 256), (64, 1000, 512),
             (2053, 2584, 136), (300, 37900, 72), (4096, 1280, 1024),
             (600, 5130, 264)]          # the last: persistent tiles of 192 columns (100 units of 256 columns, 135 of 192)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K_", TC_SHAPES)
def test_gemm_tensor_core(K, out_dtype, M, N, K_):
    g = torch.Generator().manual_seed(M + 3 * N + K_)
    a_full = torch.randn(M, K_ + 24, generator=g).to(torch.bfloat16).cuda()
    a = a_full[:, 8:8 + K_]
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).cuda()
    out_full = torch.full((M, N + 5), 9.0, dtype=out_dtype, device="cuda")
    out = out_full[:, :N]
    assert K.gemm_tc_supports(a, w, out)
    K.gemm_tc(a, w, out)
    torch.cuda.synchronize()
    assert K.gemm_tc_error() == 0
    want = a.double().cpu() @ w.double().cpu().T
    H.assert_close(out.float().cpu().numpy(), want.numpy(), 2e-5 if out_dtype == torch.float32 else 1e-2, f"tc gemm {M}x{N}x{K_}")
    assert (out_full[:, N:] == 9.0).all()                    # nothing written beyond N


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K_", [(512, 18944, 2048), (4096, 4112, 1032), (2900, 5000, 1032)])      # tiles 256, 240 and 224 wide
def test_gemm_tensor_core_tiles_of_256_rows(K, M, N, K_, out_dtype):
    """Products that the persistent kernel takes with tiles of 256 x 256 (two accumulators side by side,
    eight epilogue warps), 256, 240 or 224 columns wide as makes the shortest waves: a last row tile of 84
    rows, widths that are no multiple of the tile or of a chunk of 32 columns, a K that is no multiple of
    the k-block, two tiles per CTA (the accumulators handed back and forth)."""
    assert K.gemm_tc_takes_256_rows(M, N, K_) and not K.gemm_tc_takes_256_rows(2048, 6144, 4096) and not K.gemm_tc_takes_256_rows(128, 24576, 4096)
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16).cuda()
    out_full = torch.full((M, N + 8), 9.0, dtype=out_dtype, device="cuda")
    out = out_full[:, :N]
    K.gemm_tc(a, w, out)
    torch.cuda.synchronize()
    assert K.gemm_tc_error() == 0
    want = a.double().cpu() @ w.double().cpu().T
    H.assert_close(out.float().cpu().numpy(), want.numpy(), 2e-5 if out_dtype == torch.float32 else 1e-2, f"tc gemm, 256-row tiles, {M}x{N}x{K_}")
    assert (out_full[:, N:] == 9.0).all()


def test_gemm_tensor_core_tiles_of_256_rows_with_swiglu(K):
    M, I, Hd = 2900, 2504, 1032                     # tiles of 224 columns over 5,008: the last one 80 wide
    assert K.gemm_tc_takes_256_rows(M, 2 * I, Hd)
    g = torch.Generator().manual_seed(3)
    a = torch.randn(M, Hd, generator=g).to(torch.bfloat16).cuda()
    gate = (torch.randn(I, Hd, generator=g) / math.sqrt(Hd)).to(torch.bfloat16)
    up = (torch.randn(I, Hd, generator=g) / math.sqrt(Hd)).to(torch.bfloat16)
    inter = torch.stack([gate.view(I // 8, 8, Hd), up.view(I // 8, 8, Hd)], dim=1).reshape(2 * I, Hd).contiguous().cuda()
    out = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    K.gemm_tc(a, inter, out, epilogue=1)
    torch.cuda.synchronize()
    assert K.gemm_tc_error() == 0
    ad = a.double().cpu()
    want = pm.swiglu((ad @ gate.double().T).numpy(), (ad @ up.double().T).numpy())
    H.assert_close(out.float().cpu().numpy(), want, 1e-2, "tc gemm with 256-row tiles + swiglu")


@pytest.mark.parametrize("M,I,Hd", [(150, 264, 136), (1100, 2152, 200)])     # the second: the persistent kernel
def test_gemm_tensor_core_swiglu_epilogue(K, M, I, Hd):
    g = torch.Generator().manual_seed(2)
    a = torch.randn(M, Hd, generator=g).to(torch.bfloat16).cuda()
    gate = torch.randn(I, Hd, generator=g).to(torch.bfloat16)
    up = torch.randn(I, Hd, generator=g).to(torch.bfloat16)
    inter = torch.stack([gate.view(I // 8, 8, Hd), up.view(I // 8, 8, Hd)], dim=1).reshape(2 * I, Hd).contiguous().cuda()
    out = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    K.gemm_tc(a, inter, out, epilogue=1)
    torch.cuda.synchronize()
    assert K.gemm_tc_error() == 0
    ad = a.double().cpu()
    want = pm.swiglu((ad @ gate.double().T).numpy(), (ad @ up.double().T).numpy())
    H.assert_close(out.float().cpu().numpy(), want, 1e-2, "tc gemm + swiglu")


PREFILL_CASES = [(4, 2, 16, 16, 0), (6, 3, 48, 8, 0), (5, 1, 80, 16, 0), (8, 2, 128, 16, 0), (3, 3, 32, 4, 21), (8, 4, 64, 16, 40), (2, 1, 112, 32, 100)]


def _prefill_case(K, nq, nkv, hd, page, window, seq_lens, q_lens, impl, splits=0):
    dtype = torch.bfloat16
    rng = np.random.default_rng(nq * 31 + hd + len(seq_lens))
    kc, vc, bt, mb, dense = paged_setup(rng, seq_lens, nkv, hd, page, dtype, sum((n + page - 1) // page for n in seq_lens) + 8)
    seq_of, positions, q_start, tile_seq, tile_q0 = [], [], [0], [], []
    for s, (n, ql) in enumerate(zip(seq_lens, q_lens)):
        seq_of += [s] * ql
        positions += list(range(n - ql, n))
        q_start.append(q_start[-1] + ql)
        for t in range((ql + K.PREFILL_TILE - 1) // K.PREFILL_TILE):
            tile_seq.append(s); tile_q0.append(t * K.PREFILL_TILE)
    T = len(seq_of)
    big = torch.tensor(rng.standard_normal((T, nq * hd + 64)), dtype=torch.float32).to(dtype).cuda()
    q = big[:, 32:32 + nq * hd]
    scale = 1.0 / math.sqrt(hd)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    out = torch.full((T, nq * hd), 7.0, dtype=dtype, device="cuda")
    scratch = None
    if splits:
        # NaN everywhere: a range that holds nothing leaves its sums unwritten, and the merge must not read them
        scratch = torch.full((len(tile_seq) * K.PREFILL_TILE * nq * splits * (hd + 2),), float("nan"), device="cuda")
    K.paged_attention_prefill(q, kc, vc, bt, mb, i32(q_start), i32(seq_lens), i32(tile_seq), i32(tile_q0), len(tile_seq),
                              out, nq, nkv, hd, page, window, scale, impl=impl, scratch=scratch, max_ctx=max(seq_lens), splits=splits)
    torch.cuda.synchronize()
    assert K.attention_prefill_tc_error() == 0
    want = attention_reference(q.float().double().cpu().numpy().reshape(-1, nq, hd), dense, seq_of, positions, nq, nkv, hd, window, scale)
    H.assert_close(out.float().cpu().numpy(), want, 1.5e-2, f"prefill attention ({impl}, {splits} ranges)")


@pytest.mark.parametrize("nq,nkv,hd,page,window", PREFILL_CASES)
def test_paged_attention_prefill(K, nq, nkv, hd, page, window):
    # context after the step / tokens the step brings: whole, decode, offset portion, 2, one full tile
    _prefill_case(K, nq, nkv, hd, page, window, [130, 64, 300, 5, 200], [130, 1, 77, 2, 128], "mma")


# query heads, kv heads, head size, page, window: groups of 4, 2, 3 (a pair with one head) and 1; every page size
PREFILL_TC_CASES = [(8, 2, 128, 16, 0), (8, 4, 64, 16, 40), (3, 1, 128, 8, 0), (2, 2, 64, 32, 0), (4, 1, 128, 64, 300),
                    (6, 3, 64, 128, 0), (5, 5, 128, 16, 130)]


@pytest.mark.parametrize("nq,nkv,hd,page,window", PREFILL_TC_CASES)
def test_paged_attention_prefill_tensor_memory(K, nq, nkv, hd, page, window):
    """The tcgen05 kernel: portions that start and end anywhere against key blocks of 128, more key
    blocks than the shared-memory ring has slots, a single token, a portion of several tiles."""
    assert K.prefill_tc_supports(torch.empty(1, nq * hd, dtype=torch.bfloat16, device="cuda"),
                                 torch.empty(1, nq * hd, dtype=torch.bfloat16, device="cuda"), hd, page)
    _prefill_case(K, nq, nkv, hd, page, window, [130, 64, 300, 5, 200, 1000, 700], [130, 1, 77, 2, 128, 333, 700], "tc")


@pytest.mark.parametrize("splits", [2, 3, 8])
@pytest.mark.parametrize("nq,nkv,hd,page,window", [(8, 2, 128, 16, 0), (8, 4, 64, 16, 40), (3, 1, 128, 8, 0), (4, 1, 128, 64, 300), (5, 5, 128, 16, 130)])
def test_paged_attention_prefill_keys_cut_into_ranges(K, nq, nkv, hd, page, window, splits):
    """The same cases with every tile's key blocks cut into 2, 3 or 8 ranges on separate CTAs whose
    partial results a second kernel adds up: tiles with fewer blocks than ranges (empty ranges), a
    window that leaves early ranges empty for late rows, one head alone in a pair's place."""
    _prefill_case(K, nq, nkv, hd, page, window, [130, 64, 300, 5, 200, 1000, 700], [130, 1, 77, 2, 128, 333, 700], "tc", splits=splits)


def test_paged_attention_prefill_chooses_ranges_for_few_tiles_over_a_long_context(K):
    """The launch's own choice: 256 tokens at the end of 4,200 are two tiles of 16 pairs each, which it
    cuts into ranges when it is given the room; the result is the same as without."""
    nq, nkv, hd, page, n = 32, 8, 128, 16, 4200
    scratch_bytes = K.prefill_split_scratch_bytes(2, nq, hd, n)
    assert scratch_bytes > 0 and K.prefill_split_scratch_bytes(2, nq, hd, 500) == 0 and K.prefill_split_scratch_bytes(40, nq, hd, n) == 0
    rng = np.random.default_rng(11)
    kc, vc, bt, mb, dense = paged_setup(rng, [n], nkv, hd, page, torch.bfloat16, n // page + 9)
    q = torch.tensor(rng.standard_normal((256, nq * hd)), dtype=torch.float32).to(torch.bfloat16).cuda()
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    outs = []
    for scratch in (None, torch.full((scratch_bytes // 4,), float("nan"), device="cuda")):
        out = torch.empty_like(q)
        K.paged_attention_prefill(q, kc, vc, bt, mb, i32([0, 256]), i32([n]), i32([0, 0]), i32([0, 128]), 2, out, nq, nkv, hd, page, 0,
                                  1.0 / math.sqrt(hd), impl="tc", scratch=scratch, max_ctx=n)
        torch.cuda.synchronize()
        assert K.attention_prefill_tc_error() == 0
        outs.append(out.float().cpu().numpy())
    assert scratch.isnan().sum().item() < scratch.numel()                    # the room was used
    want = attention_reference(q.float().double().cpu().numpy().reshape(-1, nq, hd), dense, [0] * 256, list(range(n - 256, n)), nq, nkv, hd, 0,
                               1.0 / math.sqrt(hd))
    H.assert_close(outs[0], want, 1.5e-2, "one range")
    H.assert_close(outs[1], want, 1.5e-2, "chosen ranges")


@pytest.mark.parametrize("splits", [0, 1, 5])
def test_prefill_attention_of_a_portion_at_the_end_of_a_long_context(K, splits):
    """256 tokens at offset 20,000: 159 key blocks per tile, the ring and every barrier go round many
    times; three keys far apart decide head 0 of every row.  With every tile's keys in one range, in
    five, and as the launch chooses."""
    nq, nkv, hd, page, n, ql = 8, 2, 128, 16, 20256, 256
    rng = np.random.default_rng(3)
    kc, vc, bt, mb, dense = paged_setup(rng, [n], nkv, hd, page, torch.bfloat16, n // page + 9)
    q = torch.tensor(rng.standard_normal((ql, nq * hd)), dtype=torch.float32)
    q[:, :hd] = q[0, :hd]                                                      # head 0 asks the same of every row
    q = q.to(torch.bfloat16).cuda()
    btc = bt.cpu().numpy()
    for p_ in (611, 9500, 19990):
        kv = (q[0, :hd].float().cpu() * 1.5).to(torch.bfloat16)
        dense[0][0][p_, 0] = kv.float()
        kc[int(btc[0, p_ // page]) * page + p_ % page, 0] = kv.cuda()
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    scale = 1.0 / math.sqrt(hd)
    room = 2 * K.PREFILL_TILE * nq * 8 * (hd + 2)
    scratch = torch.full((room,), float("nan"), device="cuda") if splits != 1 else None
    out = torch.empty(ql, nq * hd, dtype=torch.bfloat16, device="cuda")
    K.paged_attention_prefill(q, kc, vc, bt, mb, i32([0, ql]), i32([n]), i32([0, 0]), i32([0, 128]), 2, out, nq, nkv, hd, page, 0, scale,
                              impl="tc", scratch=scratch, max_ctx=n, splits=splits if splits > 1 else 0)
    torch.cuda.synchronize()
    assert K.attention_prefill_tc_error() == 0
    rows = [0, 1, 63, 127, 128, 129, 200, 255]                               # the reference for some rows of both tiles
    want = attention_reference(q[rows].float().double().cpu().numpy().reshape(-1, nq, hd), dense, [0] * len(rows), [n - ql + r for r in rows],
                               nq, nkv, hd, 0, scale)
    H.assert_close(out[rows].float().cpu().numpy(), want, 1.5e-2, f"prefill attention at offset 20,000 ({splits} ranges)")
    assert torch.isfinite(out.float()).all()


def test_prefill_attention_growing_maximum(K):
    """Scores that keep growing with the key position: every row's maximum rises block after
    block, so the tensor-memory kernel must rescale its output again and again."""
    nq, nkv, hd, page, n = 4, 2, 128, 16, 900
    rng = np.random.default_rng(5)
    pages = (n + page - 1) // page
    perm = rng.permutation(pages + 3)
    bt = np.full((1, pages + 1), -1, dtype=np.int32)
    bt[0, :pages] = perm[:pages]
    slots = bt[0, np.arange(n) // page] * page + np.arange(n) % page
    k = torch.tensor(rng.standard_normal((n, nkv, hd)), dtype=torch.float32)
    v = torch.tensor(rng.standard_normal((n, nkv, hd)), dtype=torch.float32)
    k[:, :, 0] += torch.arange(n, dtype=torch.float32)[:, None] / 16.0
    k, v = k.to(torch.bfloat16).float(), v.to(torch.bfloat16).float()
    kc = torch.zeros((pages + 3) * page, nkv, hd); vc = torch.zeros_like(kc)
    kc[slots] = k; vc[slots] = v
    q = torch.tensor(rng.standard_normal((n, nq, hd)), dtype=torch.float32)
    q[:, :, 0] = 6.0
    q = q.to(torch.bfloat16).reshape(n, nq * hd)
    tiles = (n + K.PREFILL_TILE - 1) // K.PREFILL_TILE
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    scale = 1.0 / math.sqrt(hd)
    want = attention_reference(q.float().double().numpy().reshape(n, nq, hd), [(k, v)], [0] * n, list(range(n)), nq, nkv, hd, 0, scale)
    for impl in ("tc", "mma"):
        out = torch.empty(n, nq * hd, dtype=torch.bfloat16, device="cuda")
        K.paged_attention_prefill(q.cuda(), kc.to(torch.bfloat16).cuda(), vc.to(torch.bfloat16).cuda(), torch.tensor(bt).cuda(), pages + 1,
                                  i32([0, n]), i32([n]), i32([0] * tiles), i32([t * K.PREFILL_TILE for t in range(tiles)]), tiles,
                                  out, nq, nkv, hd, page, 0, scale, impl=impl)
        torch.cuda.synchronize()
        assert K.attention_prefill_tc_error() == 0
        H.assert_close(out.float().cpu().numpy(), want, 1.5e-2, f"prefill attention, growing maximum ({impl})")


@pytest.mark.parametrize("impl", ["mma", "tc"])
def test_prefill_attention_one_far_key_decides(K, impl):
    nq, nkv, hd, page, n = 2, 1, 64, 16, 700
    for far in (0, 63, 64, 303, 636):
        pages = (n + page - 1) // page
        perm = np.random.default_rng(far).permutation(pages + 4)
        bt = np.full((1, pages + 2), -1, dtype=np.int32)
        bt[0, :pages] = perm[:pages]
        slots = (bt[0, np.arange(n) // page] * page + np.arange(n) % page)
        kc = torch.zeros((pages + 4) * page, nkv, hd); vc = torch.zeros((pages + 4) * page, nkv, hd)
        vc[slots, 0, :] = torch.arange(n, dtype=torch.float32)[:, None] / 8.0
        kc[slots[far], 0, 0] = 40.0
        ql = 64                                                    # the last 64 tokens are the step's portion
        q = torch.zeros(ql, nq * hd); q[:, ::hd] = 8.0
        i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
        out = torch.empty(ql, nq * hd, dtype=torch.bfloat16, device="cuda")
        K.paged_attention_prefill(q.to(torch.bfloat16).cuda(), kc.to(torch.bfloat16).cuda(), vc.to(torch.bfloat16).cuda(),
                                  torch.tensor(bt).cuda(), pages + 2, i32([0, ql]), i32([n]), i32([0]), i32([0]), 1,
                                  out, nq, nkv, hd, page, 0, 1.0 / math.sqrt(hd), impl=impl)
        got = out.float().cpu().numpy()
        assert np.abs(got - far / 8.0).max() <= max(1e-2, 0.01 * far / 8.0), (far, got[0, :4], got[-1, :4])


@pytest.mark.parametrize("M,N,K_,N2", [(1, 256, 128, 96), (8, 4096, 512, 1024), (5, 1000, 192, 264), (16, 2560, 1088, 512), (11, 136, 64, 48)])
def test_gemv_fused_with_the_norm_between_two_products(K, M, N, K_, N2):
    """The product that ends a residual branch adds into the residual and prepares the next norm;
    the product after it finishes the norm on its result rows.  Together: x += a W^T;
    y = rmsnorm(x) W2^T (and silu(gate)*up of it)."""
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16).cuda()
    x0 = torch.randn(M, N, generator=g)
    nw = (1.0 + 0.3 * torch.randn(N, generator=g)).to(torch.bfloat16).cuda()
    eps = 1e-5
    x = x0.clone().cuda()
    xw = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    parts = K.gemv_stream_grid(N)
    ssq = torch.full((parts, 16), 7.0, device="cuda")
    assert K.gemv_stream_fusable(a, w)
    assert K.gemv_residual(a, w, x, nw, xw, ssq) == parts
    torch.cuda.synchronize()
    assert K.gemv_stream_error() == 0
    x_want = x0.double() + a.double().cpu() @ w.double().cpu().T
    H.assert_close(x.cpu().numpy(), x_want.numpy(), 2e-5, "residual sum")
    H.assert_close(xw.float().cpu().numpy(), (x_want * nw.double().cpu()).numpy(), 1e-2, "weighted copy")
    got_ss = ssq.double().cpu().sum(0)
    np.testing.assert_allclose(got_ss[:M].numpy(), (x_want ** 2).sum(1).numpy(), rtol=1e-5)
    assert (got_ss[M:] == 0).all()
    # the following product: plain, and with the swiglu epilogue over interleaved rows
    if N % 64 == 0:
        r = 1.0 / torch.sqrt((x.double().cpu() ** 2).mean(1) + eps)
        w2 = (torch.randn(N2, N, generator=g) / math.sqrt(N)).to(torch.bfloat16).cuda()
        out = torch.empty(M, N2, dtype=torch.bfloat16, device="cuda")
        K.gemv_scaled(xw, w2, out, ssq, parts, eps)
        y = (xw.double().cpu() @ w2.double().cpu().T) * r[:, None]
        H.assert_close(out.float().cpu().numpy(), y.numpy(), 1e-2, "scaled product")
        I = N2 // 2
        if I % 8 == 0:
            gate, up = w2[:I].cpu(), w2[I:].cpu()
            inter = torch.stack([gate.view(I // 8, 8, N), up.view(I // 8, 8, N)], dim=1).reshape(2 * I, N).contiguous().cuda()
            act = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
            K.gemv_scaled(xw, inter, act, ssq, parts, eps, epilogue=1)
            want = pm.swiglu(y[:, :I].numpy(), y[:, I:].numpy())
            H.assert_close(act.float().cpu().numpy(), want, 1e-2, "scaled product + swiglu")
        hn = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        K.scale_rows_ssq(xw, ssq, parts, eps, hn)
        H.assert_close(hn.float().cpu().numpy(), (xw.double().cpu() * r[:, None]).numpy(), 1e-2, "materialised norm")
        torch.cuda.synchronize()
        assert K.gemv_stream_error() == 0


@pytest.mark.parametrize("M,N,K_", [(1, 16, 64), (1, 333, 192), (3, 100, 320), (8, 4096, 512), (9, 77, 1088), (16, 130, 4096), (5, 48, 64), (2, 64, 1600)])
def test_gemv_stream_against_direct(K, M, N, K_, monkeypatch):
    g = torch.Generator().manual_seed(M * 7 + N)
    a_full = torch.randn(M, K_ + 16, generator=g).to(torch.bfloat16).cuda()
    a = a_full[:, 8:8 + K_]
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).cuda()
    want = (a.double().cpu() @ w.double().cpu().T).numpy()
    monkeypatch.setattr(K, "GEMV_IMPL", "stream")
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.empty(M, N, dtype=out_dtype, device="cuda")
        K.gemv(a, w, out)
        torch.cuda.synchronize()
        assert K.gemv_stream_error() == 0
        H.assert_close(out.float().cpu().numpy(), want, 2e-5 if out_dtype == torch.float32 else 1e-2, f"stream gemv {M}x{N}x{K_}")
    for splits in (2, 3, 5):
        parts = torch.full((splits, M, N), 7.0, device="cuda")
        K.gemv(a, w, parts)
        torch.cuda.synchronize()
        assert K.gemv_stream_error() == 0
        H.assert_close(parts.sum(0).cpu().numpy(), want, 2e-5, f"stream gemv partials {splits}")
    if N % 16 == 0:
        I = N // 2
        out = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
        K.gemv(a, w, out, epilogue=1)
        wd = w.double().cpu().view(I // 8, 2, 8, K_)
        ad = a.double().cpu()
        ref = pm.swiglu((ad @ wd[:, 0].reshape(I, K_).T).numpy(), (ad @ wd[:, 1].reshape(I, K_).T).numpy())
        H.assert_close(out.float().cpu().numpy(), ref, 1e-2, "stream gemv + swiglu")


# the last four take the persistent kernel with 128 x 256 tiles, one unit per (range of K, tile): a narrow product with long K
# (40 tiles x 3 ranges), ragged edges in M, N and K, more units than SMs, and a last range shorter than the others
@pytest.mark.parametrize("M,N,K_,splits", [(64, 4096, 4096, 4), (17, 130, 1032, 8), (100, 256, 576, 4), (128, 384, 12288, 8),
                                           (512, 2560, 4096, 3), (536, 2570, 9736, 3), (1100, 2584, 1160, 4), (300, 2000, 1992, 3),
                                           (536, 2570, 4104, 2)])       # the last: tiles of 192 columns (110 units of 256, 140 of 192)
def test_gemm_tensor_core_split_k(K, M, N, K_, splits):
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).cuda()
    ranges = K.gemm_tc_ranges(K_, splits)
    assert 1 <= ranges <= splits
    parts = torch.full((ranges, M, N), 5.0, device="cuda")
    K.gemm_tc(a, w, parts)
    torch.cuda.synchronize()
    assert K.gemm_tc_error() == 0
    want = (a.double().cpu() @ w.double().cpu().T).numpy()
    H.assert_close(parts.sum(0).cpu().numpy(), want, 2e-5, f"tc gemm split-K {M}x{N}x{K_}/{ranges}")
    assert K.gemm_tc_splits(2048, 4096, 4096) == 1 and K.gemm_tc_splits(64, 4096, 4096) > 1
    assert K.gemm_tc_splits(512, 2560, 4096) == 3 and K.gemm_tc_splits(512, 6144, 2560) == 1
    # 80 tiles over a long K: three ranges in two waves of units; 96 tiles: left alone
    assert K.gemm_tc_splits(536, 4096, 12288) == 3 and K.gemm_tc_splits(724, 4096, 12288) == 1


@pytest.mark.parametrize("nq,nkv,hd,page,window,norm", [(8, 2, 128, 16, 0, True), (6, 3, 48, 8, 0, True), (5, 1, 80, 16, 0, False),
                                                        (4, 4, 64, 16, 40, True), (16, 1, 32, 4, 0, True)])
def test_decode_attention_with_qk_work_folded_in(K, nq, nkv, hd, page, window, norm):
    """The fused launch against q/k kernel + attention kernel: the same cache rows and outputs to one
    bfloat16 step (the two do the norm and the rotation in another order of float32 operations, so
    about one input in forty lands one step apart somewhere; every input here comes from a seed)."""
    from types import SimpleNamespace
    from aien_sovereign_core_mv_b200.parts import GroupView, Workspace
    dtype = torch.bfloat16
    rng = np.random.default_rng(nq + hd)
    seq_lens = [1, 37, 700, 128, 129, 513]
    kc, vc, bt, mb, dense = paged_setup(rng, seq_lens, nkv, hd, page, dtype, sum((n + page - 1) // page for n in seq_lens) + 8)
    T = len(seq_lens)
    positions = [n - 1 for n in seq_lens]
    slot_map = torch.tensor([int(bt[s, p // page]) * page + p % page for s, p in enumerate(positions)], dtype=torch.int32).cuda()
    qkv = torch.tensor(rng.standard_normal((T, (nq + 2 * nkv) * hd)), dtype=torch.float32).to(dtype).cuda()
    q, k, v = qkv[:, :nq * hd], qkv[:, nq * hd:(nq + nkv) * hd], qkv[:, (nq + nkv) * hd:]
    qw = torch.tensor(rng.random(hd) * 0.4 + 0.8, dtype=torch.float32).to(dtype).cuda() if norm else None
    kw = torch.tensor(rng.random(hd) * 0.4 + 0.8, dtype=torch.float32).to(dtype).cuda() if norm else None
    pos_t = torch.tensor(positions, dtype=torch.int32).cuda()
    cos = torch.empty(T, hd // 2, device="cuda"); sin = torch.empty(T, hd // 2, device="cuda")
    K.rope_table(pos_t, torch.tensor(pm.rope_inv_freq(hd, 10000.0), dtype=torch.float64).cuda(), cos, sin)
    scale = 1.0 / math.sqrt(hd)
    splits = (max(seq_lens) + K.DECODE_CHUNK - 1) // K.DECODE_CHUNK
    # the two-kernel path
    kc1, vc1, q1 = kc.clone(), vc.clone(), q.clone()
    K.qk_norm_rope_kv_write(q1, k, v, hd, qw, kw, 1e-6, cos, sin, hd, slot_map, kc1, vc1)
    want = torch.empty(T, nq * hd, dtype=dtype, device="cuda")
    K.paged_attention_decode(q1, kc1, vc1, bt, mb, None, pos_t, want, torch.empty(T * nq * splits * hd, device="cuda"),
                             torch.empty(T * nq * splits * 2, device="cuda"), nq, nkv, hd, page, window, scale, splits)
    # the fused path
    kc2, vc2 = kc.clone(), vc.clone()
    ws = Workspace(1 << 24, 1 << 24, torch.device("cuda")); ws.begin_layer()
    ctx = SimpleNamespace(max_ctx_len=max(seq_lens), workspace=ws, positions=pos_t)
    group = GroupView("full", page, window, mb, bt, slot_map, None)
    got = torch.empty(T, nq * hd, dtype=dtype, device="cuda")
    K.paged_attention_decode_fused(ctx, q, k, v, qw, kw, 1e-6, cos, sin, hd, group, kc2, vc2, got, nq, nkv, hd, window, scale)
    torch.cuda.synchronize()
    step = lambda a, b: ((a.float() - b.float()).abs() <= 2.0 ** -7 * torch.maximum(a.float().abs(), b.float().abs())).all().item()
    assert step(kc1, kc2) and torch.equal(vc1, vc2)
    assert step(got, want) and (got.float() - want.float()).abs().max().item() <= 1e-2


# ------------------------------------------------------------------ the output head of a real vocabulary
def test_the_kernels_of_the_head_at_151936_rows(K):
    """N = 151,936 is what the logits product, the argmax and the sampler meet in serving (the
    vocabulary of Qwen3); K = 256 keeps the float64 reference cheap.  The streamed product with
    float32 output at 1 and 8 rows, the tensor-core tiles at 64 rows, argmax and a nucleus draw."""
    from aien_sovereign_core_mv_b200.sampling import philox_uniform
    V, Kd = 151936, 256
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(V, Kd, generator=g) * 0.05).to(torch.bfloat16).cuda()
    a = torch.randn(64, Kd, generator=g).to(torch.bfloat16).cuda()
    want = (a.double().cpu() @ w.double().cpu().T).numpy()
    for M in (1, 8):
        out = torch.empty(M, V, dtype=torch.float32, device="cuda")
        K.gemv(a[:M], w, out)
        H.assert_close(out.cpu().numpy(), want[:M], 2e-5, f"streamed product, {M} rows, float32 logits")
    out = torch.empty(64, V, dtype=torch.float32, device="cuda")
    K.gemm_tc(a, w, out)
    H.assert_close(out.cpu().numpy(), want, 2e-5, "tensor-core product, 64 rows, float32 logits")
    assert K.read_wait_errors() == (0, 0, 0, 0)
    # argmax: the maximum in the last 16-byte group and, on another row, twice (the lower id wins)
    lg = out[:8].clone()
    lg[0, V - 1] = lg[0].max() + 1
    lg[1, 151000] = lg[1, 77] = lg[1].max() + 2
    ids = torch.empty(8, dtype=torch.int32, device="cuda")
    K.argmax_rows(lg, ids)
    host = lg.cpu().numpy()
    assert ids.cpu().tolist() == [pm.argmax_token(r) for r in host] and ids[0].item() == V - 1 and ids[1].item() == 77
    # sampling: scaled so that a few dozen tokens carry the nucleus; every row against the plain sampler
    sharp = (lg * 6).contiguous()
    temp, top_p, top_k = [0.7, 1.0, 0.9, 0.7, 1.3, 0.8, 0.7, 1.0], [0.95, 0.9, 1.0, 0.5, 0.95, 1.0, 0.99, 0.3], [0, 0, 50, 0, 200, 1000, 0, 7]
    scratch = torch.empty(8 * V, device="cuda")
    sharp_host = sharp.cpu().numpy()
    for position in (0, 3, 1000):
        K.sample_rows(sharp, torch.tensor(temp).cuda(), torch.tensor(top_p).cuda(), torch.tensor(top_k, dtype=torch.int32).cuda(),
                      torch.arange(8, dtype=torch.int64).cuda() + 40, torch.arange(8, dtype=torch.int64).cuda() + 1,
                      torch.full((8,), position, dtype=torch.int32).cuda(), scratch, ids)
        got = ids.cpu().tolist()
        for r in range(8):
            kept, _ = pm.kept_set(sharp_host[r], temp[r], top_p[r], top_k[r])
            assert got[r] in kept, (position, r)
            u = philox_uniform(40 + r, 1 + r, position)
            assert got[r] == pm.sample_token(sharp_host[r], temp[r], top_p[r], top_k[r], u) or \
                H.knife_edge(sharp_host[r], temp[r], top_p[r], top_k[r], u), (position, r)


def test_philox_known_answers_on_the_device(K):
    """The uniform number of a draw, read back from a two-token distribution: with probabilities
    (p, 1 - p) the draw is token 0 iff u < p.  At (seed, request, position) = (0, 0, 0) the counter
    and the key are all zero, the first known-answer vector of Philox4x32-10 (6627e8d5 e169c58d ...);
    elsewhere the host function, which tests/test_sampling_host.py holds to all three vectors."""
    from aien_sovereign_core_mv_b200.sampling import philox_uniform
    u0 = float(((0x6627e8d5 << 32) | 0xe169c58d) >> 11) / 9007199254740992.0
    assert philox_uniform(0, 0, 0) == u0
    cases = [(0, 0, 0), (1, 0, 0), (0, 1, 0), (0, 0, 1), (2 ** 63 - 1, 2 ** 40 + 3, 2 ** 31 - 1), (12345, 678, 90)]
    for seed, rid, pos in cases:
        u = philox_uniform(seed, rid, pos)
        for p, want in ((u + 1e-6, 0), (u - 1e-6, 1)):
            if not 0.0 < p < 1.0:
                continue
            lg = torch.tensor([[math.log(p), math.log1p(-p)]], dtype=torch.float32).cuda()
            out = torch.empty(1, dtype=torch.int32, device="cuda")
            K.sample_rows(lg, torch.tensor([1.0]).cuda(), torch.tensor([1.0]).cuda(), torch.tensor([0], dtype=torch.int32).cuda(),
                          torch.tensor([seed], dtype=torch.int64).cuda(), torch.tensor([rid], dtype=torch.int64).cuda(),
                          torch.tensor([pos], dtype=torch.int32).cuda(), torch.empty(2, device="cuda"), out)
            assert out.item() == want, (seed, rid, pos, p)


# ------------------------------------------------------------------ a window's edge in the kernels that serve
# (context, window): the first visible key of the last token lands on a 128-key chunk boundary (256),
# on a page boundary only (272), and inside a page (269)
WINDOW_EDGES = [(400, 144), (400, 128), (400, 131)]


def _edge_cache(n, page, hd, spike_at, released_before):
    """One request of n tokens on shuffled pages: every value 1, but the key at `spike_at` carries a
    huge score and the value -5.  Pages wholly before `released_before` are given back (-1 in the table),
    and what they held is overwritten with poison that a kernel must never let through."""
    pages = (n + page - 1) // page
    perm = np.random.default_rng(n + spike_at).permutation(pages + 4)
    bt = np.full((1, pages + 2), -1, dtype=np.int32)
    bt[0, :pages] = perm[:pages]
    slots = bt[0, np.arange(n) // page] * page + np.arange(n) % page
    kc = torch.zeros((pages + 4) * page, 1, hd); vc = torch.zeros((pages + 4) * page, 1, hd)
    vc[slots, 0, :] = 1.0
    kc[slots[spike_at], 0, 0] = 50.0
    vc[slots[spike_at], 0, :] = -5.0
    for lp in range(released_before // page):
        if lp * page <= spike_at < (lp + 1) * page:
            continue                                           # (never: the spike sits at the edge)
        lo = bt[0, lp] * page
        kc[lo:lo + page, 0, 0] = 60.0                          # poison: would win every softmax
        vc[lo:lo + page] = 99.0
        bt[0, lp] = -1
    return kc.to(torch.bfloat16).cuda(), vc.to(torch.bfloat16).cuda(), torch.tensor(bt).cuda(), pages + 2


@pytest.mark.parametrize("released", [False, True])
@pytest.mark.parametrize("impl", ["direct", "stream"])
@pytest.mark.parametrize("n,window", WINDOW_EDGES)
def test_decode_attention_window_edge(K, n, window, impl, released):
    """The key just outside the window carries a huge score and must not be seen; the one just
    inside must; pages the window has passed may be gone from the block table."""
    nq, hd, page = 2, 64, 16
    first = n - window                                         # first visible key of the token at position n - 1
    for spike, want in ((first - 1, 1.0), (first, -5.0)):
        kc, vc, bt, mb = _edge_cache(n, page, hd, spike, ((first - 1) // page) * page if released else 0)
        q = torch.zeros(1, nq * hd); q[:, ::hd] = 8.0
        splits = (n + 127) // 128
        part_out = torch.empty(nq * splits * hd, device="cuda"); part_ml = torch.empty(nq * splits * 2, device="cuda")
        out = torch.empty(1, nq * hd, dtype=torch.bfloat16, device="cuda")
        K.paged_attention_decode(q.to(torch.bfloat16).cuda(), kc, vc, bt, mb, torch.zeros(1, dtype=torch.int32).cuda(),
                                 torch.tensor([n - 1], dtype=torch.int32).cuda(), out, part_out, part_ml,
                                 nq, 1, hd, page, window, 1.0 / math.sqrt(hd), splits, impl=impl)
        got = out.float().cpu().numpy()
        assert np.allclose(got, want, atol=2e-2), (impl, spike, got[0, :3])
    assert K.attention_decode_stream_error() == 0


@pytest.mark.parametrize("released", [False, True])
@pytest.mark.parametrize("impl", ["mma", "tc"])
@pytest.mark.parametrize("n,window", WINDOW_EDGES)
def test_prefill_attention_window_edge(K, n, window, impl, released):
    """A portion of 40 tokens whose rows straddle the edge: the spiked key is inside the window of
    the first 21 rows and outside that of the other 19."""
    nq, hd, page, ql = 2, 64, 16, 40
    p0 = n - ql
    spike = (p0 + 20) - window + 1                              # row at position p sees it iff p <= p0 + 20
    kc, vc, bt, mb = _edge_cache(n, page, hd, spike, ((p0 - window + 1) // page) * page if released else 0)
    q = torch.zeros(ql, nq * hd); q[:, ::hd] = 8.0
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    out = torch.empty(ql, nq * hd, dtype=torch.bfloat16, device="cuda")
    K.paged_attention_prefill(q.to(torch.bfloat16).cuda(), kc, vc, bt, mb, i32([0, ql]), i32([n]), i32([0]), i32([0]), 1,
                              out, nq, 1, hd, page, window, 1.0 / math.sqrt(hd), impl=impl)
    got = out.float().cpu().numpy()
    assert np.allclose(got[:21], -5.0, atol=2e-2), (impl, got[:21, 0])
    assert np.allclose(got[21:], 1.0, atol=2e-2), (impl, got[21:, 0])
    assert K.attention_prefill_tc_error() == 0


@pytest.mark.parametrize("V", [8, 40000])
def test_sampling_edges_of_the_nucleus_and_of_top_k(K, V):
    """Probabilities that are exact ratios, (16, 8, 4, 4, 1, 1, 1, 1) / 36, with ties at both kinds of
    threshold: the kept set must be exactly the reference's (smallest prefix in order of falling
    probability whose mass reaches top_p, ties to the lower id; the k largest, ties to the lower id),
    no token more and none fewer.  Over 400 positions every kept token is drawn and nothing else is.
    The logprob that comes back is ln(p / kept mass).  In the large vocabulary the other tokens
    carry no mass at all."""
    ln2 = math.log(2.0)
    row = np.full(V, -1e4, dtype=np.float32)
    where = [3, 0, 5, 6, 1, 2, 4, 7] if V == 8 else [977, 12, 30011, 30012, 5, 17, 20000, 39999]
    for at, k in zip(where, [0, 1, 2, 2, 4, 4, 4, 4]):
        row[at] = -k * ln2
    order = sorted(where, key=lambda i: (-row[i], i))
    # cumulative mass in that order: .444 .667 .778 .889 .917 .944 .972 1
    cases = [(0.66, 0, 2), (0.67, 0, 3), (0.78, 0, 4), (0.80, 0, 4), (0.89, 0, 5), (0.93, 0, 6), (1.0, 3, 3), (1.0, 5, 5), (1.0, 1, 1),
             (0.5, 6, 2), (0.99, 4, 4)]
    R = len(cases)
    lg = torch.tensor(np.tile(row, (R, 1))).cuda()
    f = lambda v, dt: torch.tensor(v, dtype=dt).cuda()
    ids = torch.empty(R, dtype=torch.int32, device="cuda"); lps = torch.empty(R, dtype=torch.float32, device="cuda")
    scratch = torch.empty(R * V, device="cuda")
    seen = [set() for _ in cases]
    p = np.exp(row.astype(np.float64) - row.max())
    for position in range(400):
        K.sample_rows(lg, f([1.0] * R, torch.float32), f([c[0] for c in cases], torch.float32), f([c[1] for c in cases], torch.int32),
                      f([7] * R, torch.int64), f(list(range(R)), torch.int64), f([position] * R, torch.int32), scratch, ids, lps)
        got, glp = ids.cpu().tolist(), lps.cpu().tolist()
        for r, (tp, tk, nkeep) in enumerate(cases):
            kept = order[:nkeep]
            assert got[r] in kept, (cases[r], position, got[r])
            seen[r].add(got[r])
            assert abs(glp[r] - math.log(p[got[r]] / p[kept].sum())) < 1e-4, (cases[r], position)
    for r, (tp, tk, nkeep) in enumerate(cases):
        assert seen[r] == set(order[:nkeep]), (cases[r], seen[r])
    # greedy rows give the log softmax at the maximum
    K.sample_rows(lg, f([0.0] * R, torch.float32), f([1.0] * R, torch.float32), f([0] * R, torch.int32),
                  f([7] * R, torch.int64), f(list(range(R)), torch.int64), f([0] * R, torch.int32), scratch, ids, lps)
    assert ids.cpu().tolist() == [order[0]] * R and abs(lps[0].item() - math.log(16.0 / 36.0)) < 1e-5


def test_cache_housekeeping_kernels(K):
    """The copy of a page in every run of a group (16-byte and odd row sizes, spans that touch) and zero fill
    from an odd address."""
    for shape, dtype in (((3, 64, 2, 16), torch.bfloat16), ((2, 40, 5), torch.float32), ((4, 17, 3), torch.int8)):
        st = torch.arange(int(np.prod(shape)), dtype=torch.float32).reshape(shape).to(dtype).cuda()
        want = st.clone()
        want[:, 8:16] = want[:, 0:8]
        K.copy_rows(st, 0, 8, 8)
        assert torch.equal(st, want)
        want[:, 1] = want[:, 7]
        K.copy_rows(st, 7, 1)
        assert torch.equal(st, want)
        with pytest.raises(K.KernelError):
            K.copy_rows(st, 0, 4, 8)                              # the spans overlap
    buf = torch.full((1000,), 7, dtype=torch.uint8, device="cuda")
    K.zero_fill(buf[3:990])
    assert (buf[3:990] == 0).all() and (buf[:3] == 7).all() and (buf[990:] == 7).all()
    big = torch.full((1 << 20,), 3.0, device="cuda")
    assert (K.zero_fill(big) == 0).all()
