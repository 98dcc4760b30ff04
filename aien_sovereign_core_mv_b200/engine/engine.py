"""The engine: one model, its cache, and the step function.

``Engine.step(entries)`` is the single way tokens reach the model.  An entry is
``(request id, its next tokens, want)``: a portion of a prompt or one decoded token; all
entries of a call run as one batch from the cache earlier steps left, and float32 logits come
back for the wanted places only.  The engine keeps no token history: positions follow from how
many tokens of a request the cache already holds.

Differences from the reference's ``execute_step`` (crates/aien-inference-abi/src/
transformer_backend.rs:2519-2613), by design: prefill portions and decode tokens run as one
batch instead of one request after the other; positions are explicit; capacity for the whole
batch is checked before anything changes; a token id outside the vocabulary is refused rather
than reduced modulo the vocabulary (transformer_backend.rs:1179).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import os

import numpy as np
import torch

from .. import kernels as K
from ..config.engine_config import EngineConfig
from ..csrc import build as _build
from ..models.decoder import Decoder
from ..models.loading import build_model_from_config, build_model_from_folder
from ..parts.base import FeedForward, GroupView, Mixer, Norm, Position, StepContext, StepLimits, Workspace


@dataclass
class StepEntry:
    request_id: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _align4(n: int) -> int:
    return (n + 3) & ~3


def _own_parts_only(model) -> bool:
    """Whether every part of the model is one of this package's (whose forward passes only launch
    kernels of this library)."""
    root = __name__.split(".")[0] + "."
    return all(type(o).__module__.startswith(root) for o in model.parts())


class Engine:
    """Model + cache + step.  Build with :meth:`from_folder` or :meth:`from_config`."""

    def __init__(self, model: Decoder, model_config, engine_config: EngineConfig):
        if not torch.cuda.is_available():
            raise RuntimeError("this engine runs on a CUDA device (sm_100a) only; no CPU path exists")
        K.lib()                                   # compile/load the kernels now, loudly
        self.host = _build.load_host()
        self.model = model
        self.model_config = model_config
        self.cfg = engine_config
        self.dtype_name = engine_config.resolved_dtype()
        self.dtype = torch.bfloat16 if self.dtype_name == "bfloat16" else torch.float32
        self.device = torch.device("cuda")
        self.vocab_size = model.vocab_size
        spec = model.spec
        self.page_size = int(engine_config.page_size)
        self.max_context = int(engine_config.max_context or spec.max_position)
        self.max_requests = int(engine_config.max_requests)
        self.max_tokens_per_step = int(engine_config.max_batch_tokens)

        # ---- cache groups
        pages = int(engine_config.num_pages)
        if pages <= 0:
            tokens = int(engine_config.max_cache_tokens or self.max_context)
            pages = (tokens + self.page_size - 1) // self.page_size
        self.num_pages = pages
        # what block tables, scratch and key-chunk counts are sized for: a request that keeps every
        # key can never be longer than the whole pool, whatever the context limit says
        self.table_context = self.max_context
        if any(need.kind == "full" for need in model.group_needs):
            self.table_context = min(self.max_context, pages * self.page_size)
        # Device storage per group, from what the mixers declare (CacheNeed): for every plane of a
        # paged group [runs, tokens of the pool, *per-token shape]; for a state group one plane
        # "state" [runs, slots + 1, *shape], the extra slot being nobody's (padding rows use it).
        # Zero-filled: kernels that load whole pages need finite values everywhere.
        gspecs, self.storage = [], []
        kinds = {"full": self.host.GroupKind.Full, "window": self.host.GroupKind.Window, "state": self.host.GroupKind.State}
        for need, slots in zip(model.group_needs, model.group_slots):
            if need.kind == "state":
                gspecs.append(self.host.GroupSpec(kinds["state"], 0, self.max_requests))
                sdt = getattr(torch, need.state_dtype)
                self.storage.append({"state": K.zero_fill(torch.empty((slots, self.max_requests + 1) + tuple(need.state_shape), dtype=sdt, device=self.device))})
            else:
                if not need.planes:
                    raise ValueError(f"a mixer asks for a {need.kind!r} cache and names no planes to keep in it")
                gspecs.append(self.host.GroupSpec(kinds[need.kind], need.window, pages))
                pdt = getattr(torch, need.dtype) if need.dtype else self.dtype
                self.storage.append({name: K.zero_fill(torch.empty((slots, pages * self.page_size) + tuple(int(d) for d in shape), dtype=pdt, device=self.device))
                                     for name, shape in need.planes})
        self.cache = self.host.CacheManager(self.page_size, gspecs, self.max_requests)
        self.max_blocks = (self.table_context + self.page_size - 1) // self.page_size

        # ---- workspace and metadata buffers
        itemsize = 2 if self.dtype == torch.bfloat16 else 4
        T = self.max_tokens_per_step
        self.limits = StepLimits(max_tokens=T, max_seqs=self.max_requests, max_context=self.table_context, itemsize=itemsize)
        self.workspace = Workspace(model.step_workspace_bytes(self.limits), model.layer_workspace_bytes(self.limits), self.device)
        meta_len = self._meta_len(T, self.max_requests, T)
        # pinned staging buffers in a ring: a buffer is rewritten only after its copy has run
        self._meta_ring = []
        for _ in range(4):
            h = torch.empty(meta_len, dtype=torch.int32, pin_memory=True)
            self._meta_ring.append([h, h.numpy(), None])
        self._meta_turn = 0
        self.meta_dev = torch.empty(meta_len, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self._graphs = {}
        # a part that reads device data on the host cannot be captured
        self._graphable = not any(getattr(p, "host_reads", False) for p in model.parts())
        # A step that is not captured still repeats: the launches of a forward pass are fixed by a
        # few host numbers (tokens, requests, wanted rows, attention tiles, key chunks) because every
        # buffer comes from the step workspace or the metadata block at addresses that follow from
        # them.  Such a step is written down once and re-issued for every later step with the same
        # numbers, without the Python in between.  Only for models made of this package's parts
        # alone: a part defined elsewhere may do work that is not a launch of this library.
        self._replayable = bool(engine_config.replay_steps) and self._graphable and _own_parts_only(model) \
            and os.environ.get("AIEN_B200_STEP_REPLAY", "1") != "0"
        self._plans: Dict[tuple, list] = {}
        self._plan_logits: Optional[torch.Tensor] = None
        self.steps_replayed = 0
        # the error words of the kernels with bounded waits, collected behind every step()
        self._wait_dev = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._wait_host = torch.zeros(4, dtype=torch.int32, pin_memory=True)
        self._wait_event: Optional[torch.cuda.Event] = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir: str, engine_config: Optional[EngineConfig] = None, strict: bool = False) -> "Engine":
        ec = engine_config or EngineConfig()
        cfg, model = build_model_from_folder(model_dir, ec.resolved_dtype(), strict)
        return cls(model, cfg, ec)

    @classmethod
    def from_config(cls, raw_config: Mapping, seed: int = 0, engine_config: Optional[EngineConfig] = None,
                    init_std: Optional[float] = None, device_init: bool = False) -> "Engine":
        ec = engine_config or EngineConfig()
        cfg, model = build_model_from_config(raw_config, seed, ec.resolved_dtype(), init_std, device_init)
        return cls(model, cfg, ec)

    # ------------------------------------------------------------------ metadata layout
    def _meta_len(self, T: int, S: int, R: int) -> int:
        return self._layout(T, S, R)[1]

    def _layout(self, T: int, S: int, R: int):
        off, o = {}, 0
        for name, n in (("token_ids", T), ("positions", T), ("seq_of_token", T), ("q_start", S + 1), ("ctx_len", S), ("want_rows", R)):
            off[name] = o
            o += _align4(max(n, 1))
        groups = []
        for need in self.model.group_needs:
            if need.kind == "state":
                groups.append((-1, o, 0))
                o += _align4(max(S, 1))
            else:
                bt = o
                o += _align4(S * self.max_blocks)
                groups.append((bt, o, self.max_blocks))
                o += _align4(max(T, 1))
        off["groups"] = groups
        n_tiles = T // K.PREFILL_TILE + S + 1         # query tiles of the prefill attention kernel
        off["tile_seq"] = o
        o += _align4(n_tiles)
        off["tile_q0"] = o
        o += _align4(n_tiles)
        off["single_tokens"] = o                      # token indices of single-token entries in a mixed step
        o += _align4(max(S, 1))
        off["feed_src"] = o                           # per token: row of the previous step's sampled ids to take, or -1
        o += _align4(max(T, 1))
        return off, o

    # ------------------------------------------------------------------ requests
    def has_request(self, request_id: int) -> bool:
        return self.cache.has(int(request_id))

    def num_tokens(self, request_id: int) -> int:
        return self.cache.num_tokens(int(request_id))

    def end_request(self, request_id: int) -> None:
        """Give back everything the request holds."""
        if self.cache.has(int(request_id)):
            self.cache.free_request(int(request_id))

    def fork(self, parent: int, child: int, at_token: int = -1) -> None:
        """``child`` shares the cache of the first ``at_token`` tokens of ``parent`` (all by
        default); pages are copied only when one of the two writes into a shared one."""
        self._do_copies(self.cache.fork(int(parent), int(child), int(at_token)))

    def _do_copies(self, copies) -> None:
        ps = self.page_size
        for g, src, dst in copies:
            state = self.model.group_needs[g].kind == "state"
            for st in self.storage[g].values():
                if state:
                    K.copy_rows(st, src, dst)
                else:
                    K.copy_rows(st, src * ps, dst * ps, ps)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence, logits_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one batch.  ``entries``: StepEntry or (request_id, tokens, want) tuples.  Returns
        float32 logits [number of wanted places, vocab] on the device, in the order of the
        entries and of each entry's ``want``.  Takes the cache pages the tokens need first; if
        they cannot all be had, raises with nothing changed."""
        self.check_waits(block=False)              # a wait that ran out in the step before is reported now at the latest
        ids, counts, flat, want_rows = self._validate(entries)
        if not ids:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        added = []
        try:
            for rid in ids:
                if not self.cache.has(rid):
                    self.cache.add_request(rid)
                    added.append(rid)
            before = [self.cache.num_tokens(rid) for rid in ids]
            copies = self.cache.append(list(zip(ids, counts)))
        except Exception:
            for rid in added:
                self.cache.free_request(rid)
            raise
        try:
            self._do_copies(copies)
            logits = self.run_reserved(ids, counts, flat, want_rows, logits_out)
            self._post_waits()
        except Exception:
            self.rollback(ids, before, added)
            raise
        self._last_step = (ids, before, added)
        return logits

    # ------------------------------------------------------------------ failed steps
    def rollback(self, ids, before, added=()) -> None:
        """Undo what a failed step took from the cache: every request goes back to the length it
        had (``before``), requests the step created are removed.  The reference snapshots and
        rolls back the same way (crates/aien-kv-cache/src/lib.rs:815-858, 1646-1695).  A request
        of a group that cannot be rewound (fixed-size state, a window that has moved on) is
        removed instead: what it holds can no longer be trusted."""
        for rid, n in zip(ids, before):
            if not self.cache.has(rid):
                continue
            if rid in added:
                self.cache.free_request(rid)
                continue
            try:
                self.cache.truncate(rid, n)
            except ValueError:
                self.cache.free_request(rid)

    def collect_waits(self, out: torch.Tensor) -> None:
        """Writes the four error words of the kernels with bounded waits to out[0:4] (int32 on the
        device), in the stream, behind the launches made so far."""
        K.collect_wait_errors(out)

    def _post_waits(self) -> None:
        K.collect_wait_errors(self._wait_dev)
        self._wait_host.copy_(self._wait_dev, non_blocking=True)
        if self._wait_event is None:
            self._wait_event = torch.cuda.Event()
        self._wait_event.record()

    def check_waits(self, block: bool = True) -> None:
        """Raises KernelError if a bounded wait of a kernel ran out in a step() made so far: its
        logits are not valid.  The requests of that step are put back to the lengths they had.
        ``block=False`` looks only if the step's words have already arrived on the host.  step()
        looks this way on entry; a caller that reads the logits on the host calls it after its
        synchronisation, before it uses them."""
        ev = self._wait_event
        if ev is None or (not block and not ev.query()):
            return
        ev.synchronize()
        self._wait_event = None
        self.raise_on_waits(self._wait_host.tolist())

    def raise_on_waits(self, words) -> None:
        msg = K.wait_error_message(words)
        if not msg:
            return
        torch.cuda.synchronize()
        K.read_wait_errors()                       # clears the words
        last, self._last_step = getattr(self, "_last_step", None), None
        if last is not None:
            self.rollback(*last)
        raise K.KernelError(msg)

    def _validate(self, entries: Sequence):
        ids, counts, want_rows, chunks = [], [], [], []
        seen = set()
        t0 = 0
        for e in entries:
            rid, toks, want = (e.request_id, e.tokens, e.want) if isinstance(e, StepEntry) else (e[0], e[1], e[2] if len(e) > 2 else ())
            rid = int(rid)
            arr = np.asarray(toks, dtype=np.int64).reshape(-1)
            n = int(arr.shape[0])
            if rid in seen:
                raise ValueError(f"request {rid} appears twice in one step")
            seen.add(rid)
            if n == 0:
                raise ValueError(f"request {rid}: an entry must bring at least one token")
            if int(arr.min()) < 0 or int(arr.max()) >= self.vocab_size:
                bad = int(arr[(arr < 0) | (arr >= self.vocab_size)][0])
                raise ValueError(f"request {rid}: token id {bad} is outside the vocabulary of {self.vocab_size}")
            for w in want:
                if not (0 <= int(w) < n):
                    raise ValueError(f"request {rid}: wanted place {w} is outside its {n} tokens")
                want_rows.append(t0 + int(w))
            have = self.cache.num_tokens(rid) if self.cache.has(rid) else 0
            if have + n > self.max_context:
                raise ValueError(f"request {rid}: {have + n} tokens exceed the context limit {self.max_context}")
            ids.append(rid)
            counts.append(n)
            chunks.append(arr)
            t0 += n
        if t0 > self.max_tokens_per_step:
            raise ValueError(f"step of {t0} tokens exceeds max_batch_tokens {self.max_tokens_per_step}")
        if len(ids) > self.max_requests:
            raise ValueError(f"step of {len(ids)} requests exceeds max_requests {self.max_requests}")
        flat = np.concatenate(chunks).astype(np.int32) if chunks else np.zeros(0, dtype=np.int32)
        return ids, counts, flat, want_rows

    def run_reserved(self, ids, counts, flat, want_rows, logits_out: Optional[torch.Tensor] = None, feed=None) -> torch.Tensor:
        """The part of a step after its pages were taken (the scheduler takes them itself):
        metadata to the device in one copy, then the model.  Decode-only steps that want every
        row replay a captured CUDA graph.  ``feed`` = (ids on the device, rows): tokens given as -1
        in ``flat`` are taken on the device from ``ids[rows[i]]`` (what the step before sampled,
        not yet seen by the host)."""
        T, S, R = int(sum(counts)), len(ids), len(want_rows)
        for rid in ids:
            if self.cache.num_tokens(rid) > self.max_context:
                raise ValueError(f"request {rid}: {self.cache.num_tokens(rid)} tokens exceed the context limit {self.max_context}")
        graph_step = (T == S and R == T and self.cfg.use_cuda_graphs and self.dtype == torch.bfloat16
                      and self._graphable and want_rows == list(range(T)))
        Tp = self._bucket(T) if graph_step else T          # captured steps run at a few batch sizes; the rest is padding
        off, total = self._layout(Tp, Tp if graph_step else S, Tp if graph_step else R)
        slot = self._meta_ring[self._meta_turn % len(self._meta_ring)]
        self._meta_turn += 1
        if slot[2] is not None:
            slot[2].synchronize()
        meta_host, m = slot[0], slot[1]
        m[off["token_ids"]:off["token_ids"] + T] = flat
        if feed is not None:
            m[off["token_ids"]:off["token_ids"] + T][flat < 0] = 0
            m[off["feed_src"]:off["feed_src"] + T] = feed[1]
        elif T and int(flat.min()) < 0:
            raise ValueError("a step brought a token id of -1 without a device feed")
        if R:
            m[off["want_rows"]:off["want_rows"] + R] = want_rows
        max_ctx = self.cache.fill_meta(ids, counts, m, off["positions"], off["seq_of_token"], off["q_start"], off["ctx_len"], off["groups"])
        decode_only = T == S
        n_tiles, n_single = 0, 0
        if not decode_only:
            t_at = 0
            for i, c in enumerate(counts):
                if c == 1:
                    m[off["single_tokens"] + n_single] = t_at
                    n_single += 1
                    t_at += 1
                    continue
                t_at += c
                k = (c + K.PREFILL_TILE - 1) // K.PREFILL_TILE
                m[off["tile_seq"] + n_tiles:off["tile_seq"] + n_tiles + k] = i
                m[off["tile_q0"] + n_tiles:off["tile_q0"] + n_tiles + k] = np.arange(k, dtype=np.int32) * K.PREFILL_TILE
                n_tiles += k
        if Tp > T:
            self._pad_meta(m, off, T, Tp)
        if graph_step:
            self._warm_decode(off, Tp, max_ctx, total)
        self.meta_dev[:total].copy_(meta_host[:total], non_blocking=True)
        if slot[2] is None:
            slot[2] = torch.cuda.Event()
        slot[2].record()
        if feed is not None:
            d = self.meta_dev
            K.feed_token_ids(d[off["token_ids"]:off["token_ids"] + T], d[off["feed_src"]:off["feed_src"] + T], feed[0])
        self.steps_run += 1
        if graph_step:
            return self._replay_decode(off, Tp, max_ctx, logits_out, T)
        own = logits_out is None
        key = None
        if self._replayable and R <= self.max_requests:
            max_ctx = self._ctx_bucket(max_ctx)
            if own:
                if self._plan_logits is None:
                    self._plan_logits = torch.empty((self.max_requests, self.vocab_size), dtype=torch.float32, device=self.device)
                logits_out = self._plan_logits[:R]
            key = (T, S, R, max_ctx, n_tiles, n_single, logits_out.data_ptr(), torch.cuda.current_stream().cuda_stream)
            plan = self._plans.get(key)
            if plan is not None:
                K.replay_launches(plan)
                self.steps_replayed += 1
                return logits_out.clone() if own else logits_out     # the engine's own buffer is rewritten by the next such step
        elif own:
            logits_out = torch.empty((R, self.vocab_size), dtype=torch.float32, device=self.device)
        ctx = self._context(off, T, S, max(counts), max_ctx, decode_only)
        d = self.meta_dev
        ctx.prefill_tiles = (d[off["tile_seq"]:off["tile_seq"] + max(n_tiles, 1)], d[off["tile_q0"]:off["tile_q0"] + max(n_tiles, 1)], n_tiles)
        ctx.single_tokens = (d[off["single_tokens"]:off["single_tokens"] + max(n_single, 1)], n_single)
        want = d[off["want_rows"]:off["want_rows"] + max(R, 1)]
        with K.stream_scope():
            if key is None:
                self.model.forward(ctx, want, R, logits_out)
                return logits_out
            K.begin_recording()
            try:
                self.model.forward(ctx, want, R, logits_out)
            finally:
                plan = K.end_recording()
        if len(self._plans) >= 512:
            self._plans.pop(next(iter(self._plans)))
        self._plans[key] = plan
        return logits_out.clone() if own else logits_out

    # ------------------------------------------------------------------ captured decode steps
    _BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)

    def _bucket(self, T: int) -> int:
        cap = min(self.max_requests, self.max_tokens_per_step)      # what the workspace and the metadata are sized for
        for b in self._BUCKETS:
            if b >= T:
                return min(b, cap) if cap >= T else T
        return T

    def _ctx_bucket(self, max_ctx: int) -> int:
        """The longest context of a step, rounded up to a power-of-two count of key chunks (what
        sizes the decode attention's partial results), but not beyond the engine's limit."""
        from ..kernels import DECODE_CHUNK
        splits = 1
        while splits * DECODE_CHUNK < max_ctx:
            splits *= 2
        limit = (self.table_context + DECODE_CHUNK - 1) // DECODE_CHUNK
        return max(1, min(splits, limit)) * DECODE_CHUNK

    def _pad_meta(self, m, off, T: int, Tp: int) -> None:
        """Rows T..Tp of a captured step: a token at position 0 of a request with no pages; it
        writes no cache slot and attends over nothing."""
        m[off["token_ids"] + T:off["token_ids"] + Tp] = 0
        m[off["positions"] + T:off["positions"] + Tp] = 0
        m[off["seq_of_token"] + T:off["seq_of_token"] + Tp] = np.arange(T, Tp, dtype=np.int32)
        m[off["q_start"] + T:off["q_start"] + Tp + 1] = np.arange(T, Tp + 1, dtype=np.int32)
        m[off["ctx_len"] + T:off["ctx_len"] + Tp] = 0
        m[off["want_rows"]:off["want_rows"] + Tp] = np.arange(Tp, dtype=np.int32)
        for (bt, sm, mb), need in zip(off["groups"], self.model.group_needs):
            if need.kind == "state":
                m[sm + T:sm + Tp] = self.max_requests      # the slot that belongs to nobody
            else:
                m[bt + T * mb:bt + Tp * mb] = -1
                m[sm + T:sm + Tp] = -1

    def _decode_forward(self, off, T: int, splits: int, logits: torch.Tensor) -> None:
        from ..kernels import DECODE_CHUNK
        d = self.meta_dev
        ctx = self._context(off, T, T, 1, splits * DECODE_CHUNK, True)
        with K.stream_scope():
            self.model.forward(ctx, d[off["want_rows"]:off["want_rows"] + T], T, logits)

    def _warm_decode(self, off, T: int, max_ctx: int, total: int) -> None:
        """Before a decode step of a new shape is captured, the same launches run once outside the
        capture (tables and buffers that parts make at first use).  That run sees padding rows
        only: it writes no cache slot and no request's state, so the step itself runs exactly
        once, whatever its mixers keep between steps."""
        from ..kernels import DECODE_CHUNK
        splits = self._ctx_bucket(max_ctx) // DECODE_CHUNK
        if (T, splits) in self._graphs:
            return
        pad = torch.zeros(total, dtype=torch.int32)
        self._pad_meta(pad.numpy(), off, 0, T)
        self.meta_dev[:total].copy_(pad)
        self._decode_forward(off, T, splits, torch.empty((T, self.vocab_size), dtype=torch.float32, device=self.device))
        torch.cuda.synchronize()

    def _replay_decode(self, off, T: int, max_ctx: int, logits_out: Optional[torch.Tensor], real: Optional[int] = None) -> torch.Tensor:
        """Decode steps are short chains of small kernels; launching them one by one costs more
        than running them.  One CUDA graph per (batch size, key-chunk count) is captured at first
        use and replayed afterwards; its inputs are the metadata buffer, its output a logits
        buffer of its own."""
        from ..kernels import DECODE_CHUNK
        splits = self._ctx_bucket(max_ctx) // DECODE_CHUNK
        key = (T, splits)
        entry = self._graphs.get(key)
        if entry is None:
            logits = torch.empty((T, self.vocab_size), dtype=torch.float32, device=self.device)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = K.launch_count()
            with torch.cuda.graph(graph):
                self._decode_forward(off, T, splits, logits)
            entry = (graph, logits, K.launch_count() - before)
            if len(self._graphs) >= 48:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = entry
        graph, logits, nodes = entry
        graph.replay()
        K.add_launches(nodes)
        real = T if real is None else real
        if logits_out is not None:
            logits_out.copy_(logits[:real])
            return logits_out
        return logits[:real]

    def _context(self, off, T: int, S: int, max_q: int, max_ctx: int, decode_only: bool) -> StepContext:
        d = self.meta_dev
        groups = []
        for g, need in enumerate(self.model.group_needs):
            bt, sm, mb = off["groups"][g]
            if need.kind == "state":
                groups.append(GroupView("state", self.page_size, 0, 0, None, d[sm:sm + S], self.storage[g]))
            else:
                groups.append(GroupView(need.kind, self.page_size, need.window, mb,
                                        d[bt:bt + S * mb].view(S, mb), d[sm:sm + T], self.storage[g]))
        self.workspace.reset()
        return StepContext(
            dtype=self.dtype, num_tokens=T, num_seqs=S,
            token_ids=d[off["token_ids"]:off["token_ids"] + T], positions=d[off["positions"]:off["positions"] + T],
            seq_of_token=d[off["seq_of_token"]:off["seq_of_token"] + T], q_start=d[off["q_start"]:off["q_start"] + S + 1],
            ctx_len=d[off["ctx_len"]:off["ctx_len"] + S], groups=groups, workspace=self.workspace,
            max_q_len=max_q, max_ctx_len=max_ctx, decode_only=decode_only,
        )

    # ------------------------------------------------------------------ information
    def cache_state(self) -> dict:
        return {
            "free_pages": [self.cache.free_count(g) for g in range(self.cache.num_groups)],
            "requests": self.cache.num_requests, "metrics": self.cache.metrics(), "check": self.cache.check(),
        }
