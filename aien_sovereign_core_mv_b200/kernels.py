"""Python face of the CUDA kernel library (``csrc/kernels``), loaded with ctypes.

Every function here takes torch tensors that already live on the device, checks what the
kernel cannot check for itself, and launches on the current CUDA stream.  Nothing falls back
to another implementation: a missing library, a refused size or a failed launch raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_long, c_size_t, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {
    -2: "unsupported dtype combination",
    -3: "a size this kernel refuses",
    -4: "pointer or stride not aligned as the kernel requires",
    -5: "library state error (tensor map / attribute)",
    -6: "a bounded wait inside the kernel ran out",
}


class KernelError(RuntimeError):
    pass


_lib: Optional[ctypes.CDLL] = None
_proxy = None
_RECORD: Optional[list] = None
_QUERIES = ("_supports", "_ranges", "_grid", "_error")     # answer a question, launch nothing


class _Entry:
    """One launching entry point.  Calls go to the ctypes function and, while a recording is on,
    into the list; every attribute (argtypes, restype, ...) is the ctypes function's own, so code
    that declares a signature on what :func:`lib` hands out declares it on the real thing."""
    __slots__ = ("_fn",)

    def __init__(self, fn):
        object.__setattr__(self, "_fn", fn)

    def __call__(self, *args):
        rc = self._fn(*args)
        if _RECORD is not None:
            _RECORD.append((self._fn, args))
        return rc

    def __getattr__(self, key):
        return getattr(self._fn, key)

    def __setattr__(self, key, value):
        setattr(self._fn, key, value)


class _Library:
    """The loaded library with its launching entry points wrapped, so that what a forward pass
    launches can be written down as (function, arguments) and issued again by
    :func:`replay_launches` without the Python that chose the arguments."""

    def __init__(self, cdll: ctypes.CDLL):
        self._cdll = cdll

    def __getattr__(self, name: str):
        fn = getattr(self._cdll, name)
        wrapped = fn if name.endswith(_QUERIES) else _Entry(fn)
        self.__dict__[name] = wrapped
        return wrapped


def lib() -> "_Library":
    global _lib, _proxy
    if _proxy is None:
        _lib = _build.load_kernels()
        _declare(_lib)
        _proxy = _Library(_lib)
    return _proxy


def begin_recording() -> None:
    """From here every launch made through this module is also written down."""
    global _RECORD
    _RECORD = []


def end_recording() -> list:
    global _RECORD
    plan, _RECORD = _RECORD or [], None
    return plan


def replay_launches(plan: list) -> None:
    """Issue a recorded list again.  Valid only while every argument still means the same: the
    same buffers at the same addresses, the same sizes, the same stream."""
    global _launches
    for fn, args in plan:
        rc = fn(*args)
        if rc != 0:
            _check(rc, getattr(fn, "__name__", "a recorded launch"))
    _launches += len(plan)


def _declare(l: ctypes.CDLL) -> None:
    P, I, L, F = c_void_p, c_int, c_long, c_float
    sigs = {
        "aien_embed_gather": [P, I, P, P, I, I, I, P],
        "aien_add_rmsnorm": [P, P, I, I, c_size_t, P, I, F, P, I, I, I, P],
        "aien_gather_add_rows": [P, P, I, I, c_size_t, P, P, I, I, P],
        "aien_swiglu": [P, P, I, I, I, I, P],
        "aien_add_residual": [P, P, I, I, c_size_t, I, I, P],
        "aien_rope_table": [P, P, P, P, I, I, P],
        "aien_qk_norm_rope_kv_write": [P, L, I, P, L, P, L, I, I, I, c_size_t, P, L, I, P, P, I, F, P, P, I, P, P, P, I, I, I, P],
        "aien_convert": [P, I, P, I, c_size_t, P],
        "aien_gemm_simple": [P, I, L, P, I, L, P, I, L, I, I, I, P],
        "aien_paged_attention_generic": [P, L, P, P, P, I, P, P, P, L, I, I, I, I, I, F, I, I, I, P],
        "aien_argmax_rows": [P, I, I, P, P],
        "aien_sample_rows": [P, I, I, P, P, P, P, P, P, P, P, P],
        "aien_sample_rows_logprob": [P, I, I, P, P, P, P, P, P, P, P, P, P],
        "aien_gemv_bf16": [P, L, P, L, P, I, L, I, I, I, I, I, c_size_t, P],
        "aien_gemv_stream_bf16": [P, L, P, L, P, I, L, I, I, I, I, I, c_size_t, P],
        "aien_gemv_stream_error": [],
        "aien_gemm_tc": [P, L, P, L, P, I, L, I, I, I, I, I, c_size_t, P],
        "aien_gemm_tc_ranges": [I, I],
        "aien_gemm_tc_m256_supports": [I, I, I, I],
        "aien_gemv_stream_scaled": [P, L, P, L, P, I, L, I, I, I, I, P, I, F, P],
        "aien_gemv_stream_residual": [P, L, P, L, P, L, P, I, P, L, P, I, I, I, P],
        "aien_gemv_stream_grid": [I],
        "aien_feed_token_ids": [P, P, P, I, P],
        "aien_copy_spans": [P, c_size_t, I, c_size_t, c_size_t, c_size_t, P],
        "aien_zero_fill": [P, c_size_t, P],
        "aien_scale_rows_ssq": [P, L, P, I, F, P, L, I, I, P],
        "aien_gemm_tc_error": [],
        "aien_attention_prefill_tc_error": [],
        "aien_paged_attention_prefill": [P, L, P, P, P, I, P, P, P, P, I, P, L, I, I, I, I, I, F, P],
        "aien_paged_attention_prefill_tc": [P, L, I, P, P, I, P, I, P, P, P, P, I, P, L, I, I, I, I, I, F, P],
        "aien_paged_attention_prefill_tc_split": [P, L, I, P, P, I, P, I, P, P, P, P, I, P, L, I, I, I, I, I, F, P, L, I, I, P],
        "aien_paged_attention_prefill_tc_supports": [I, I],
        "aien_paged_attention_decode": [P, L, P, P, P, I, P, P, P, P, L, P, P, P, I, I, I, I, I, F, I, I, P],
        "aien_paged_attention_decode_stream": [P, L, P, P, I, P, I, P, P, P, P, L, P, P, P, I, I, I, I, I, F, I, I, P],
        "aien_paged_attention_decode_stream_supports": [I, I, I, I, I],
        "aien_attention_decode_stream_error": [],
        "aien_collect_wait_errors": [P, P],
        "aien_paged_attention_decode_fused": [P, L, P, L, P, L, P, P, I, F, P, P, I, P, P, P, P, I, P, P, L, P, P, P,
                                              I, I, I, I, I, F, I, I, P],
    }
    for name, args in sigs.items():
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = c_int


def declare_optional(name: str, args) -> bool:
    """Declare a symbol that later kernel files add; returns False when the library lacks it."""
    lib()
    try:
        fn = getattr(_lib, name)
    except AttributeError:
        return False
    fn.argtypes = args
    fn.restype = c_int
    return True


_launches = 0


def launch_count() -> int:
    """Kernel launches issued through this module so far (replayed graph nodes included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(rc: int, name: str) -> None:
    global _launches
    if rc == 0:
        _launches += 1
        return
    if rc < 0:
        raise KernelError(f"{name}: {_ERRORS.get(rc, 'refused')} (code {rc})")
    raise KernelError(f"{name}: CUDA error {rc} at launch")


_STREAM: Optional[int] = None


class stream_scope:
    """Looks the current CUDA stream up once for every launch made inside the block (a step
    makes hundreds; the lookup costs more than the launch)."""

    def __enter__(self):
        global _STREAM
        self._prev = _STREAM
        _STREAM = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _STREAM
        _STREAM = self._prev
        return False


def _stream() -> int:
    return _STREAM if _STREAM is not None else torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels") from None


def _dev(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on the CUDA device (there is no CPU path)")


# ---------------------------------------------------------------------------- row-wise ops
def embed_gather(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor) -> None:
    """x[t] = table[ids[t]] as float32.  table [V,H], ids int32 [T], x float32 [T,H]."""
    _dev(table, ids, x)
    T, H = x.shape
    assert table.is_contiguous() and x.is_contiguous() and ids.dtype == torch.int32 and x.dtype == torch.float32
    assert table.shape[1] == H and ids.numel() >= T
    _check(lib().aien_embed_gather(_p(table), dt(table), _p(ids), _p(x), T, H, table.shape[0], _stream()), "embed_gather")


def _parts_of(delta: Optional[torch.Tensor], shape) -> tuple:
    """(nparts, stride in elements) of a pending sum: [T,H], or float32 partials [P,T,H]."""
    if delta is None:
        return 1, 0
    assert delta.is_contiguous()
    if delta.dim() == 3:
        assert tuple(delta.shape[1:]) == tuple(shape) and delta.dtype == torch.float32
        return delta.shape[0], delta.shape[1] * delta.shape[2]
    assert tuple(delta.shape) == tuple(shape)
    return 1, 0


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """x += delta (when given); out = rmsnorm(x) * weight.  x float32 [T,H] updated in place."""
    _dev(x, delta, weight, out)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == x.shape
    assert weight.numel() == H and weight.is_contiguous()
    nparts, stride = _parts_of(delta, x.shape)
    _check(lib().aien_add_rmsnorm(_p(x), _p(delta), dt(delta) if delta is not None else F32, nparts, stride,
                                  _p(weight), dt(weight), float(eps), _p(out), dt(out), T, H, _stream()), "add_rmsnorm")


def gather_add_rows(x: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = x[rows[r]] + delta[rows[r]] in float32."""
    _dev(x, delta, rows, out)
    R, H = out.shape
    assert x.dtype == torch.float32 and out.dtype == torch.float32 and rows.dtype == torch.int32
    assert x.is_contiguous() and out.is_contiguous() and x.shape[1] == H and rows.numel() >= R
    nparts, stride = _parts_of(delta, x.shape)
    _check(lib().aien_gather_add_rows(_p(x), _p(delta), dt(delta) if delta is not None else F32, nparts, stride,
                                      _p(rows), _p(out), R, H, _stream()), "gather_add_rows")


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    """x += delta in float32; delta [T,H] in any kernel dtype, or float32 partial products [P,T,H]."""
    _dev(x, delta)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    nparts, stride = _parts_of(delta, x.shape)
    _check(lib().aien_add_residual(_p(x), _p(delta), dt(delta), nparts, stride, T, H, _stream()), "add_residual")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, group: int = 0) -> None:
    """out = silu(gate) * up for gate_up = [T, 2I]: gate columns first (group 0), or gate and up
    columns interleaved in runs of ``group``."""
    _dev(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype
    _check(lib().aien_swiglu(_p(gate_up), _p(out), dt(out), T, I, int(group), _stream()), "swiglu")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    """cos/sin [T, half] float32 of positions[t] * inv_freq[i], the angle taken in float64."""
    _dev(positions, inv_freq, cos, sin)
    T, half = cos.shape
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float64 and inv_freq.numel() == half
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    _check(lib().aien_rope_table(_p(positions), _p(inv_freq), _p(cos), _p(sin), T, half, _stream()), "rope_table")


def qk_norm_rope_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], head_dim: int,
                          q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                          cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                          slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], q_out: Optional[torch.Tensor] = None) -> None:
    """Per-head RMSNorm of q and k (when weights are given), rotation of the first
    ``rotary_dim`` values, q written to ``q_out`` (default: in place), k and v written to their
    cache slots.  q [T, nq*hd], k/v [T, nkv*hd] may be column slices of one projection output, or
    of float32 partial products [P, T, ...] that are summed on the way in (then q_out is needed)."""
    _dev(q, k, v, q_norm_w, k_norm_w, cos, sin, slot_map, k_cache, v_cache, q_out)
    nparts, part_stride = 1, 0
    if q.dim() == 3:
        assert q.dtype == torch.float32 and q_out is not None
        nparts, part_stride = q.shape[0], q.stride(0)
        if k is not None:
            assert k.dim() == 3 and v.dim() == 3 and k.stride(0) == part_stride and v.stride(0) == part_stride
    if q_out is None:
        q_out = q
    T = q.shape[-2]
    assert q.stride(-1) == 1 and q.shape[-1] % head_dim == 0 and q_out.stride(1) == 1 and q_out.shape == (T, q.shape[-1])
    nq = q.shape[-1] // head_dim
    nkv = 0
    if k is not None:
        assert v is not None and slot_map is not None and k_cache is not None and v_cache is not None
        assert k.stride(-1) == 1 and v.stride(-1) == 1 and k.dtype == q.dtype and v.dtype == q.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == v_cache.dtype
        assert slot_map.dtype == torch.int32 and slot_map.numel() >= T
        nkv = k.shape[-1] // head_dim
    wdt = F32
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            assert w.numel() == head_dim and w.is_contiguous()
            wdt = dt(w)
    if q_norm_w is not None and k_norm_w is not None:
        assert q_norm_w.dtype == k_norm_w.dtype
    if cos is not None:
        assert sin is not None and cos.shape == (T, rotary_dim // 2) and cos.is_contiguous() and sin.is_contiguous()
    _check(lib().aien_qk_norm_rope_kv_write(
        _p(q), q.stride(-2), nq, _p(k), k.stride(-2) if k is not None else 0, _p(v), v.stride(-2) if v is not None else 0,
        nkv, dt(q), nparts, part_stride, _p(q_out), q_out.stride(0), head_dim, _p(q_norm_w), _p(k_norm_w), wdt, float(eps),
        _p(cos), _p(sin), rotary_dim if cos is not None else 0, _p(slot_map), _p(k_cache), _p(v_cache),
        dt(q_out), dt(k_cache) if k_cache is not None else dt(q_out), T, _stream()), "qk_norm_rope_kv_write")


def convert(src: torch.Tensor, dst: torch.Tensor) -> None:
    _dev(src, dst)
    assert src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel()
    _check(lib().aien_convert(_p(src), dt(src), _p(dst), dt(dst), src.numel(), _stream()), "convert")


# ---------------------------------------------------------------------------- matrix products
def gemm_simple(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] . w[N,K]^T, float32 accumulation on the CUDA cores, any sizes."""
    _dev(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib().aien_gemm_simple(_p(a), dt(a), a.stride(0), _p(w), dt(w), w.stride(0), _p(out), dt(out), out.stride(0),
                                  M, N, K, _stream()), "gemm_simple")


# ---------------------------------------------------------------------------- attention
def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            max_blocks: int, seq_of_token: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                            num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                            scale: float) -> None:
    """Causal attention of T query tokens over their requests' pages.  q [T, nq*hd] (row stride
    free), caches [slots, nkv, hd], block_table int32 [S, max_blocks], out [T, nq*hd]."""
    _dev(q, k_cache, v_cache, block_table, seq_of_token, positions, out)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == v_cache.dtype
    assert block_table.dtype == torch.int32 and seq_of_token.dtype == torch.int32 and positions.dtype == torch.int32
    _check(lib().aien_paged_attention_generic(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), max_blocks, _p(seq_of_token), _p(positions),
        _p(out), out.stride(0), num_q_heads, num_kv_heads, head_dim, page_size, window, float(scale),
        dt(q), dt(k_cache), T, _stream()), "paged_attention_generic")


# ---------------------------------------------------------------------------- sampling
def argmax_rows(logits: torch.Tensor, out_ids: torch.Tensor) -> None:
    _dev(logits, out_ids)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and out_ids.dtype == torch.int32 and out_ids.numel() >= R
    _check(lib().aien_argmax_rows(_p(logits), R, V, _p(out_ids), _stream()), "argmax_rows")


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, top_k: torch.Tensor,
                seeds: torch.Tensor, request_ids: torch.Tensor, positions: torch.Tensor, scratch: torch.Tensor,
                out_ids: torch.Tensor, out_logprob: Optional[torch.Tensor] = None) -> None:
    """One token per row; see csrc/kernels/sampling.cu for the rules.  scratch: R*V float32.
    ``out_logprob`` (float32 [R]) also receives the log-probability of each chosen token."""
    _dev(logits, temperature, top_p, top_k, seeds, request_ids, positions, scratch, out_ids, out_logprob)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and top_k.dtype == torch.int32
    assert seeds.dtype == torch.int64 and request_ids.dtype == torch.int64 and positions.dtype == torch.int32
    assert scratch.dtype == torch.float32 and scratch.numel() >= R * V and out_ids.dtype == torch.int32
    if out_logprob is not None:
        assert out_logprob.dtype == torch.float32 and out_logprob.numel() >= R and out_logprob.is_contiguous()
        _check(lib().aien_sample_rows_logprob(_p(logits), R, V, _p(temperature), _p(top_p), _p(top_k), _p(seeds), _p(request_ids),
                                              _p(positions), _p(scratch), _p(out_ids), _p(out_logprob), _stream()), "sample_rows_logprob")
        return
    _check(lib().aien_sample_rows(_p(logits), R, V, _p(temperature), _p(top_p), _p(top_k), _p(seeds), _p(request_ids),
                                  _p(positions), _p(scratch), _p(out_ids), _stream()), "sample_rows")


# ---------------------------------------------------------------------------- decode product
GEMV_MAX_ROWS = 16          # what the decode products take
# Up to how many rows a step's products go to them: beyond 8 rows (their second token tile) the
# tensor-core tile kernel with 32 rows of A per stage is faster (Qwen3-8B shape, batch 9 / 12 / 16:
# 4.15 / 4.19 / 4.21 ms a step against 3.59 / 3.68 / 3.75 ms).
GEMV_ROUTE_ROWS = 8
# "stream": persistent TMA-fed kernel; "direct": loads straight from global memory into fragments
GEMV_IMPL = __import__("os").environ.get("AIEN_B200_GEMV", "stream").strip().lower()


def gemv_supports(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    K_ = a.shape[1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] <= GEMV_MAX_ROWS and K_ % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(-1) == 1)


def gemv_splits(N: int, K_: int) -> int:
    """How many ranges K is cut into across CTAs, from the weight's shape alone (never from the
    batch): enough CTAs to fill the GPU when the matrix has few rows."""
    if GEMV_IMPL == "stream" and K_ % 64 == 0:
        return 1                     # the persistent kernel balances itself; no partial products needed
    tiles = (N + 15) // 16
    return max(1, min(8, 1184 // tiles, K_ // 512))


def gemv(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0) -> None:
    """out = a . w^T for up to 16 rows of a (bfloat16, float32 accumulation).  ``epilogue=1``:
    w holds gate|up rows interleaved in groups of 8 and out = silu(gate)*up with N/2 columns.
    ``out`` of shape [P, M, N] float32 receives P partial products over P ranges of K."""
    _dev(a, w, out)
    M, K_ = a.shape
    N = w.shape[0]
    splits, part_stride = 1, 0
    if out.dim() == 3:
        assert epilogue == 0 and out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape[1:]) == (M, N)
        splits, part_stride = out.shape[0], M * N
    else:
        assert w.shape[1] == K_ and out.shape == (M, N if epilogue == 0 else N // 2)
    fn = lib().aien_gemv_stream_bf16 if (GEMV_IMPL == "stream" and K_ % 64 == 0) else lib().aien_gemv_bf16
    _check(fn(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), dt(out), out.stride(-2), M, N, K_,
              epilogue, splits, part_stride, _stream()), "gemv_bf16")


def gemv_stream_error() -> int:
    """Error code left by a bounded wait inside the streamed decode product (0: none); clears it."""
    return int(lib().aien_gemv_stream_error())


def gemm_tc_supports(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    K_ = a.shape[1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K_ % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0) -> None:
    """out = a . w^T on the tcgen05 tensor cores (bfloat16 operands, float32 accumulation in
    tensor memory).  ``epilogue=1``: w holds gate|up rows interleaved in runs of 8 and
    out = silu(gate)*up with N/2 columns."""
    _dev(a, w, out)
    M, K_ = a.shape
    N = w.shape[0]
    splits, part_stride = 1, 0
    if out.dim() == 3:                      # float32 partial products over ranges of K, for the consumer to add
        assert epilogue == 0 and out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape[1:]) == (M, N)
        assert out.shape[0] == gemm_tc_ranges(K_, out.shape[0])
        splits, part_stride = out.shape[0], M * N
    else:
        assert w.shape[1] == K_ and out.shape == (M, N if epilogue == 0 else N // 2)
    _check(lib().aien_gemm_tc(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), dt(out), out.stride(-2), M, N, K_,
                              epilogue, splits, part_stride, _stream()), "gemm_tc")


# Upper bound of the float32 partial products one deferred product may leave in the workspace:
# ranges x M x N <= (296 / tiles) x (tiles x 128 x 128) elements within one wave of units; ranges over
# several waves (gemm_tc_splits) are taken only while they fit.
PARTIALS_MAX_BYTES = 40 * 1024 * 1024 + (1 << 16)


def gemm_tc_ranges(K_: int, splits: int) -> int:
    """How many ranges of K the tensor-core kernel makes when asked for ``splits``."""
    return int(lib().aien_gemm_tc_ranges(int(K_), int(splits)))


def gemm_tc_takes_256_rows(M: int, N: int, K_: int, splits: int = 1) -> bool:
    """Whether gemm_tc runs this product on the persistent kernel with tiles of 256 x 256."""
    return bool(lib().aien_gemm_tc_m256_supports(int(M), int(N), int(K_), int(splits)))


def gemm_tc_splits(M: int, N: int, K_: int) -> int:
    """Ranges of K for a product with few rows: enough CTAs to occupy the GPU (148 SMs, two CTAs
    each) when the tile grid alone is small.  Depends on the shapes only."""
    if M > 64 and N >= 256:
        # the persistent kernel with 128 x 256 tiles: as many ranges (eight at most) as still give every range
        # 8 k-blocks and every SM at most one unit (128 rows x 4,096 x 12,288: 16 tiles, 4 -> 8 ranges, 29.9 -> 25.9 us)
        tiles = ((M + 127) // 128) * ((N + 255) // 256)
        if tiles >= 148:
            return 1
        one_wave = gemm_tc_ranges(K_, max(1, min(8, 148 // tiles, K_ // 512)))
        # Three sevenths of the SMs or more idle over a long K: ranges over two or three waves of units can still be
        # faster, the float32 partial products they write and their consumer reads counted in (536 rows x 4,096
        # x 12,288: 80 tiles; one range 80.1 us, three 60.0 us + 3.5 us for the consumer; x 14,336: 89.9 -> 68.4 us).
        # Costs in cycles: a k-block of a tile 768, a tile's fixed part 1,500, a partly filled GPU clocks higher,
        # partial products at 3,800 bytes a cycle both ways.  Taken when a tenth faster by this count.
        kb = (K_ + 63) // 64

        def cost(r: int) -> float:
            units = tiles * r
            waves = (units + 147) // 148
            c = waves * (-(-kb // r) * 768 + 1500)
            if units < 148:
                c *= 0.75 + 0.25 * units / 148
            return c + ((r * M * N * 8) / 3800 + 2000 if r > 1 else 0)

        best, best_cost = one_wave, cost(one_wave)
        if tiles * 7 > 148 * 4:         # with more than four sevenths of the SMs busy it measured no faster (724 rows: 96 tiles)
            return best
        for r in range(one_wave + 1, 9):
            if K_ // 512 < r or r * M * N * 4 > PARTIALS_MAX_BYTES - (1 << 16) or gemm_tc_ranges(K_, r) != r:
                continue
            if cost(r) < 0.9 * best_cost:
                best, best_cost = r, cost(r)
        return best
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    if tiles >= 148:
        return 1
    return gemm_tc_ranges(K_, max(1, min(8, 296 // tiles, K_ // 512)))


def small_step_products_fuse(dtype: torch.dtype, num_tokens: int) -> bool:
    """Whether the products of this step are the streamed decode kernel, whose epilogues can do a
    norm's work (residual add and preparation before it, the row factor after it).  The one place
    that knows the routing; norms of any kind ask here."""
    return dtype == torch.bfloat16 and num_tokens <= GEMV_ROUTE_ROWS and GEMV_IMPL == "stream"


def FUSED_NORM_SCRATCH_BYTES(hidden: int) -> int:
    """What a product that ends a residual branch takes for the next norm: bfloat16 rows and partial sums, with slack."""
    return GEMV_MAX_ROWS * hidden * 2 + 1024 * 16 * 4 + 1024


def gemv_stream_fusable(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the streamed decode product, and so its fusions with the norm around it, takes a . w^T."""
    return (GEMV_IMPL == "stream" and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2
            and a.shape[0] <= GEMV_MAX_ROWS and a.shape[1] % 64 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemv_stream_grid(n_rows: int) -> int:
    """Number of CTAs (and so of partial sums of squares) of a streamed product over ``n_rows`` rows of W."""
    return int(lib().aien_gemv_stream_grid(int(n_rows)))


def gemv_scaled(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ssq: torch.Tensor, parts: int, eps: float, epilogue: int = 0) -> None:
    """out = (a . w^T) with row t multiplied by 1/sqrt(sum_p ssq[p, t] / K + eps) first; epilogue 1
    then applies silu(gate)*up over rows of w interleaved in runs of 8."""
    _dev(a, w, out, ssq)
    M, Kd = a.shape
    N = w.shape[0]
    assert gemv_stream_fusable(a, w) and ssq.dtype == torch.float32 and ssq.is_contiguous() and ssq.numel() >= parts * 16
    assert out.shape == (M, N // 2 if epilogue else N) and out.stride(1) == 1
    _check(lib().aien_gemv_stream_scaled(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), dt(out), out.stride(0), M, N, Kd,
                                         int(epilogue), _p(ssq), int(parts), float(eps), _stream()), "gemv_stream_scaled")


def gemv_residual(a: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, norm_w: torch.Tensor, xw: torch.Tensor, ssq_out: torch.Tensor) -> int:
    """resid += a . w^T in place (float32); xw = bfloat16(resid * norm_w); ssq_out[p, t] = partial
    sums of resid[t]^2.  Returns the number of parts written."""
    _dev(a, w, resid, norm_w, xw, ssq_out)
    M, Kd = a.shape
    N = w.shape[0]
    parts = gemv_stream_grid(N)
    assert gemv_stream_fusable(a, w) and resid.dtype == torch.float32 and resid.shape == (M, N) and resid.stride(1) == 1
    assert xw.dtype == torch.bfloat16 and xw.shape == (M, N) and xw.stride(1) == 1 and norm_w.numel() == N and norm_w.is_contiguous()
    assert ssq_out.dtype == torch.float32 and ssq_out.is_contiguous() and ssq_out.numel() >= parts * 16
    _check(lib().aien_gemv_stream_residual(_p(a), a.stride(0), _p(w), w.stride(0), _p(resid), resid.stride(0), _p(norm_w), dt(norm_w),
                                           _p(xw), xw.stride(0), _p(ssq_out), M, N, Kd, _stream()), "gemv_stream_residual")
    return parts


def feed_token_ids(token_ids: torch.Tensor, src: torch.Tensor, prev: torch.Tensor) -> None:
    """token_ids[i] = prev[src[i]] where src[i] >= 0 (int32 device tensors)."""
    _dev(token_ids, src, prev)
    assert token_ids.dtype == torch.int32 and src.dtype == torch.int32 and prev.dtype == torch.int32 and src.numel() >= token_ids.numel()
    _check(lib().aien_feed_token_ids(_p(token_ids), _p(src), _p(prev), token_ids.numel(), _stream()), "feed_token_ids")


def copy_rows(storage: torch.Tensor, src: int, dst: int, count: int = 1) -> None:
    """storage[:, dst:dst+count] = storage[:, src:src+count] for a contiguous [runs, rows, ...] tensor: the copy
    of a cache page (count = tokens a page) or of a state slot in every run of a cache group."""
    _dev(storage)
    assert storage.is_contiguous() and storage.dim() >= 2
    row = storage[0, 0].numel() * storage.element_size()
    _check(lib().aien_copy_spans(_p(storage), storage.shape[1] * row, storage.shape[0], src * row, dst * row, count * row, _stream()),
           "copy_spans")


def zero_fill(t: torch.Tensor) -> torch.Tensor:
    """Zeroes a contiguous device tensor in place (the cache pools at start: the paged kernels load whole pages)."""
    _dev(t)
    assert t.is_contiguous()
    _check(lib().aien_zero_fill(_p(t), t.numel() * t.element_size(), _stream()), "zero_fill")
    return t


def scale_rows_ssq(xw: torch.Tensor, ssq: torch.Tensor, parts: int, eps: float, out: torch.Tensor) -> None:
    """out[t] = bfloat16(xw[t] / sqrt(sum_p ssq[p, t] / H + eps)): the rest of a norm whose weight is inside xw."""
    _dev(xw, ssq, out)
    T, H = xw.shape
    assert xw.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape == (T, H) and xw.stride(1) == 1 and out.stride(1) == 1
    _check(lib().aien_scale_rows_ssq(_p(xw), xw.stride(0), _p(ssq), int(parts), float(eps), _p(out), out.stride(0), T, H, _stream()),
           "scale_rows_ssq")


def gemm_tc_error() -> int:
    """Error code left by a bounded wait inside the tensor-core kernel (0: none); clears it."""
    return int(lib().aien_gemm_tc_error())


# ---------------------------------------------------------------------------- attention choice
DECODE_CHUNK = 128
PREFILL_TILE = 128         # query tokens per CTA of the prefill attention kernel


def attention_workspace_bytes(lim, num_heads: int, head_dim: int) -> int:
    """Scratch of the split-key decode kernel for the largest decode-only step."""
    splits = (lim.max_context + DECODE_CHUNK - 1) // DECODE_CHUNK
    return lim.max_seqs * num_heads * splits * (head_dim + 2) * 4 + 1024 \
        + prefill_split_scratch_bytes(PREFILL_SPLIT_MAX_TILES, num_heads, head_dim, lim.max_context) + 256


_ticket_counters: Optional[torch.Tensor] = None


_DECODE_ATTN_IMPL = __import__("os").environ.get("AIEN_B200_DECODE_ATTENTION", "stream").strip().lower()     # "stream" | "direct"


def decode_stream_supports(num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, max_splits: int) -> bool:
    """Whether the streamed decode attention kernel takes this case (head size 64 or 128, pages that divide 128)."""
    return bool(lib().aien_paged_attention_decode_stream_supports(num_q_heads, num_kv_heads, head_dim, page_size, max_splits))


def paged_attention_decode(q, k_cache, v_cache, block_table, max_blocks, seq_of_token, positions, out,
                           part_out, part_ml, num_q_heads, num_kv_heads, head_dim, page_size, window, scale,
                           max_splits, token_list=None, num_tokens=None, impl: Optional[str] = None) -> None:
    """Split-key decode attention; the CTA that finishes last merges the chunks.  The ticket
    counters are one small device buffer that every launch finds zero and leaves zero.
    ``impl``: "stream" (TMA ring, persistent CTAs; where the sizes allow) or "direct" (one CTA per
    chunk); both give the same bits.  Default from ``AIEN_B200_DECODE_ATTENTION``, else "stream"."""
    global _ticket_counters
    _dev(q, k_cache, v_cache, block_table, seq_of_token, positions, out, part_out, part_ml)
    # seq_of_token None: token t belongs to row t of the block table.  token_list: serve only these tokens.
    T = q.shape[0] if token_list is None else int(num_tokens)
    if _ticket_counters is None:
        _ticket_counters = torch.zeros(1 << 16, dtype=torch.int32, device=q.device)
    assert T * num_kv_heads <= _ticket_counters.numel()
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert part_out.dtype == torch.float32 and part_out.numel() >= T * num_q_heads * max_splits * head_dim
    assert part_ml.dtype == torch.float32 and part_ml.numel() >= T * num_q_heads * max_splits * 2
    impl = impl or _DECODE_ATTN_IMPL
    if impl == "stream" and decode_stream_supports(num_q_heads, num_kv_heads, head_dim, page_size, max_splits):
        _check(lib().aien_paged_attention_decode_stream(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), k_cache.shape[0], _p(block_table), max_blocks, _p(seq_of_token),
            _p(positions), _p(token_list), _p(out), out.stride(0), _p(part_out), _p(part_ml), _p(_ticket_counters), num_q_heads,
            num_kv_heads, head_dim, page_size, window, float(scale), max_splits, T, _stream()), "paged_attention_decode_stream")
        return
    _check(lib().aien_paged_attention_decode(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), max_blocks, _p(seq_of_token), _p(positions),
        _p(token_list), _p(out), out.stride(0), _p(part_out), _p(part_ml), _p(_ticket_counters), num_q_heads, num_kv_heads, head_dim,
        page_size, window, float(scale), max_splits, T, _stream()), "paged_attention_decode")


def attention_decode_stream_error() -> int:
    """Code left by a wait that ran out in the streamed decode attention kernel (0: none)."""
    return int(lib().aien_attention_decode_stream_error())


def paged_attention_decode_fused(ctx, q, k, v, q_norm_w, k_norm_w, eps, cos, sin, rotary_dim, group, k_cache, v_cache, out,
                                 num_q_heads, num_kv_heads, head_dim, window, scale) -> None:
    """Decode-only steps: per-head q/k norm, rotation, the write of k and v into the cache and the
    split-key attention in one launch.  q, k, v are the raw projections [T, heads*head_dim]."""
    global _ticket_counters
    _dev(q, k, v, q_norm_w, k_norm_w, cos, sin, k_cache, v_cache, out)
    T = q.shape[0]
    if _ticket_counters is None:
        _ticket_counters = torch.zeros(1 << 16, dtype=torch.int32, device=q.device)
    assert T * num_kv_heads <= _ticket_counters.numel()
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and out.stride(1) == 1
    wdt = F32
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            assert w.numel() == head_dim and w.is_contiguous()
            wdt = dt(w)
    if cos is not None:
        assert cos.shape == (T, rotary_dim // 2) and cos.is_contiguous() and sin.is_contiguous()
    splits = max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
    part_out = ctx.workspace.take((T * num_q_heads * splits * head_dim,), torch.float32)
    part_ml = ctx.workspace.take((T * num_q_heads * splits * 2,), torch.float32)
    k2 = k_cache.view(-1, num_kv_heads, head_dim)
    v2 = v_cache.view(-1, num_kv_heads, head_dim)
    _check(lib().aien_paged_attention_decode_fused(
        _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(q_norm_w), _p(k_norm_w), wdt, float(eps),
        _p(cos), _p(sin), rotary_dim if cos is not None else 0, _p(group.slot_map), _p(k2), _p(v2), _p(group.block_table),
        group.max_blocks, _p(ctx.positions), _p(out), out.stride(0), _p(part_out), _p(part_ml), _p(_ticket_counters),
        num_q_heads, num_kv_heads, head_dim, group.page_size, window, float(scale), splits, T, _stream()),
        "paged_attention_decode_fused")


def decode_attention_supports(q: torch.Tensor, k_cache: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
            and num_q_heads // num_kv_heads <= 16 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


_FORCE_ATTN = __import__("os").environ.get("AIEN_B200_ATTENTION", "").strip().lower()


def paged_attention(ctx, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, group, out: torch.Tensor,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float) -> None:
    """Attention of the step's tokens over one cache group; picks the kernel for the step:
    the split-key kernel when every request brings one token (bfloat16), else the generic one.
    ``AIEN_B200_ATTENTION=generic`` pins the generic kernel for debugging; ``fused`` folds the q/k
    kernel into the decode attention launch (see parts/attention.py)."""
    k2 = k_cache.view(-1, num_kv_heads, head_dim)
    v2 = v_cache.view(-1, num_kv_heads, head_dim)
    if (ctx.decode_only and _FORCE_ATTN != "generic"
            and decode_attention_supports(q, k2, num_q_heads, num_kv_heads, head_dim)):
        T = q.shape[0]
        splits = max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
        part_out = ctx.workspace.take((T * num_q_heads * splits * head_dim,), torch.float32)
        part_ml = ctx.workspace.take((T * num_q_heads * splits * 2,), torch.float32)
        paged_attention_decode(q, k2, v2, group.block_table, group.max_blocks, None, ctx.positions, out,
                               part_out, part_ml, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale, splits)
        return
    if (not ctx.decode_only and _FORCE_ATTN != "generic" and ctx.prefill_tiles is not None
            and prefill_attention_supports(q, k2, out, head_dim)
            and decode_attention_supports(q, k2, num_q_heads, num_kv_heads, head_dim)):
        # a mixed step: portions go through the tiled kernel, single tokens through the split-key kernel
        tile_seq, tile_q0, n = ctx.prefill_tiles
        if n > 0:
            room = prefill_split_scratch_bytes(n, num_q_heads, head_dim, ctx.max_ctx_len)
            scratch = ctx.workspace.take((room // 4,), torch.float32) if room else None
            paged_attention_prefill(q, k2, v2, group.block_table, group.max_blocks, ctx.q_start, ctx.ctx_len, tile_seq, tile_q0, n,
                                    out, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                                    scratch=scratch, max_ctx=ctx.max_ctx_len)
        tokens, nd = ctx.single_tokens if ctx.single_tokens is not None else (None, 0)
        if nd > 0:
            splits = max(1, (ctx.max_ctx_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
            part_out = ctx.workspace.take((nd * num_q_heads * splits * head_dim,), torch.float32)
            part_ml = ctx.workspace.take((nd * num_q_heads * splits * 2,), torch.float32)
            paged_attention_decode(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out,
                                   part_out, part_ml, num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale,
                                   splits, token_list=tokens, num_tokens=nd)
        return
    paged_attention_generic(q, k2, v2, group.block_table, group.max_blocks, ctx.seq_of_token, ctx.positions, out,
                            num_q_heads, num_kv_heads, head_dim, group.page_size, window, scale)


def prefill_attention_supports(q: torch.Tensor, k_cache: torch.Tensor, out: torch.Tensor, head_dim: int) -> bool:
    return (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 128
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0)


_PREFILL_IMPL = __import__("os").environ.get("AIEN_B200_PREFILL", "tc").strip().lower()     # "tc" | "mma"


def prefill_tc_supports(q, out, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this case (head size 64 or 128, pages that divide 128)."""
    return (bool(lib().aien_paged_attention_prefill_tc_supports(head_dim, page_size)) and q.stride(0) % 8 == 0
            and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


PREFILL_SPLIT_MAX_TILES = 8          # steps with more tiles fill the GPU without cutting the keys


def prefill_split_scratch_bytes(num_tiles: int, num_q_heads: int, head_dim: int, max_ctx: int) -> int:
    """Room the tcgen05 prefill kernel can use to cut the keys of `num_tiles` tiles into ranges
    (float32 partial results); 0 where it would not cut."""
    if num_tiles <= 0 or num_tiles > PREFILL_SPLIT_MAX_TILES or max_ctx < 8 * PREFILL_TILE:
        return 0
    return num_tiles * PREFILL_TILE * num_q_heads * 8 * (head_dim + 2) * 4


def paged_attention_prefill(q, k_cache, v_cache, block_table, max_blocks, q_start, ctx_len, tile_seq, tile_q0, num_tiles,
                            out, num_q_heads, num_kv_heads, head_dim, page_size, window, scale, impl: Optional[str] = None,
                            scratch: Optional[torch.Tensor] = None, max_ctx: int = 0, splits: int = 0) -> None:
    """Causal attention of portions of prompts over their requests' pages (bfloat16, tensor
    cores).  ``tile_seq``/``tile_q0``: for every 128-token query tile, the index of its request in
    the step and the tile's offset inside that request's portion.  ``impl``: "tc" (tcgen05, where
    the sizes allow) or "mma" (mma.sync); default from ``AIEN_B200_PREFILL``, else "tc".
    ``scratch`` (float32, optional) with ``max_ctx`` (an upper bound of the contexts) lets the
    tcgen05 kernel cut the keys of a step with few tiles into ranges that run on separate SMs;
    ``splits`` > 0 asks for that many ranges (tests)."""
    _dev(q, k_cache, v_cache, block_table, q_start, ctx_len, tile_seq, tile_q0, out)
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    for t in (block_table, q_start, ctx_len, tile_seq, tile_q0):
        assert t.dtype == torch.int32
    impl = impl or _PREFILL_IMPL
    if impl == "tc" and prefill_tc_supports(q, out, head_dim, page_size):
        if scratch is not None:
            _dev(scratch)
            assert scratch.dtype == torch.float32 and scratch.is_contiguous()
        _check(lib().aien_paged_attention_prefill_tc_split(
            _p(q), q.stride(0), q.shape[0], _p(k_cache), _p(v_cache), k_cache.shape[0], _p(block_table), max_blocks, _p(q_start),
            _p(ctx_len), _p(tile_seq), _p(tile_q0), num_tiles, _p(out), out.stride(0), num_q_heads, num_kv_heads, head_dim,
            page_size, window, float(scale), _p(scratch) if scratch is not None else None,
            scratch.numel() * 4 if scratch is not None else 0, int(max_ctx), int(splits), _stream()), "paged_attention_prefill_tc")
        return
    _check(lib().aien_paged_attention_prefill(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), max_blocks, _p(q_start), _p(ctx_len), _p(tile_seq),
        _p(tile_q0), num_tiles, _p(out), out.stride(0), num_q_heads, num_kv_heads, head_dim, page_size, window,
        float(scale), _stream()), "paged_attention_prefill")


def attention_prefill_tc_error() -> int:
    """Code left by a wait that ran out in the tcgen05 prefill attention kernel (0: none)."""
    return int(lib().aien_attention_prefill_tc_error())


# ---------------------------------------------------------------------------- bounded waits
# The kernels whose mbarrier waits are bounded, in the order of the words collect_wait_errors writes.
WAIT_KERNELS = ("gemm_tc", "gemv_stream", "attention_prefill_tc", "attention_decode_stream")


def collect_wait_errors(out: torch.Tensor) -> None:
    """out[0:4] (int32, device) = the error words of WAIT_KERNELS, read in the stream behind
    whatever was launched before.  The words stay set until read_wait_errors() clears them."""
    _dev(out)
    assert out.dtype == torch.int32 and out.numel() >= 4 and out.is_contiguous()
    _check(lib().aien_collect_wait_errors(_p(out), _stream()), "collect_wait_errors")


def read_wait_errors() -> tuple:
    """The four error words, read with synchronous copies (the device is idle afterwards) and
    cleared.  All zero: every bounded wait so far was met."""
    return (gemm_tc_error(), gemv_stream_error(), attention_prefill_tc_error(), attention_decode_stream_error())


def wait_error_message(words) -> str:
    """'' when all words are zero, else which kernels gave up and with which code."""
    bad = [f"{name} (code {int(w)})" for name, w in zip(WAIT_KERNELS, words) if int(w) != 0]
    if not bad:
        return ""
    return ("a bounded wait ran out inside " + ", ".join(bad) +
            ": the results of the step are not valid (a broken TMA / tensor-core pipeline, not a property of the inputs)")
