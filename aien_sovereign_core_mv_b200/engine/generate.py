"""Generation: the scheduler above the step function, and sampling above the logits.

``Generator.generate`` is the Python entry point: token ids in, token ids out, any number of
requests batched continuously.  ``generate_tokens`` is the single-request form with the
reference's argument names (crates/aien-inference-abi/src/transformer_backend.rs:643-664:
``generate_tokens(seq_id, prompt_tokens, max_tokens, temperature, stop_tokens)``).

One loop turn = one step: the scheduler plans (and takes the cache pages), the engine runs the
batch and returns logits at the last place of every request that reached the end of its input,
one token per such request is chosen on the device, the ids come back to the host, the
scheduler commits them and finishes what is done.  A stop id ends a request and is not
emitted.

``Generator.run`` keeps the device busy between steps (``EngineConfig.async_scheduling``): step
n+1 is planned and launched while step n still runs; the tokens step n sampled are handed to
step n+1 on the device, and reach the host, for the stop check and the result, one step later.
A request that meets a stop id has then computed one token too many, which is dropped; the
tokens that come out are those of the step-by-step loop.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Union

import os
import sys

import numpy as np
import torch

from .. import kernels as K
from ..sampling.sampler import SamplingParams
from .engine import Engine


_STEP_LOG = os.environ.get("AIEN_STEP_LOG", "") not in ("", "0")


@dataclass
class GenerationResult:
    request_id: int
    tokens: List[int]
    finish_reason: str            # "stop", "length", "cancelled", "aborted"
    message: str = ""
    preemptions: int = 0
    logprobs: Optional[List[float]] = None     # one per token, when SamplingParams.logprobs asked for them


_REASONS = {"StopToken": "stop", "LengthLimit": "length", "Cancelled": "cancelled", "Aborted": "aborted", "NONE": "none"}


class Generator:
    def __init__(self, engine: Engine):
        self.engine = engine
        host = engine.host
        sc = host.SchedulerConfig()
        cfg = engine.cfg
        sc.max_batch_size = min(cfg.max_batch_size, engine.max_requests)
        sc.max_batch_tokens = min(cfg.max_batch_tokens, engine.max_tokens_per_step)
        sc.max_prefill_tokens = min(cfg.max_prefill_tokens, sc.max_batch_tokens)
        sc.prefill_chunk_size = cfg.prefill_chunk_size
        sc.chunk_prefill = cfg.chunk_prefill
        sc.watermark_blocks = cfg.watermark_blocks
        sc.align_step_tokens = cfg.align_step_tokens
        sc.max_context = engine.max_context
        self.scheduler = host.Scheduler(sc, engine.cache)
        self.params: Dict[int, SamplingParams] = {}
        R = engine.max_requests
        dev = engine.device
        # two of each staging buffer: a step is prepared while the one before it is still in flight
        # sampled ids, then the four error words of the kernels with bounded waits, then (when a request
        # asks for them) the log-probabilities of the chosen tokens as float32 bits: one copy brings all
        self._ids_dev2 = [torch.zeros(2 * R + 4, dtype=torch.int32, device=dev) for _ in range(2)]
        self._ids_host2 = [torch.zeros(2 * R + 4, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._logprobs: Dict[int, List[float]] = {}
        # sampling parameters of a step's rows, one block of 8 R words so that one copy brings them:
        # temperature, top_p (float32), top_k, position (int32), seed, request id (int64)
        self._params_host2 = [torch.zeros(8 * R, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._params_np = [(h.numpy()[:2 * R].view(np.float32).reshape(2, R), h.numpy()[2 * R:4 * R].reshape(2, R),
                            h.numpy()[4 * R:].view(np.int64).reshape(2, R)) for h in self._params_host2]
        self._turn = 0
        self._events = [torch.cuda.Event() for _ in range(2)]
        self._inflight = None        # (rows, host ids, count, event) of the step whose tokens the host has not seen
        self._params_dev = torch.zeros(8 * R, dtype=torch.int32, device=dev)
        self._fparams = self._params_dev[:2 * R].view(torch.float32).view(2, R)
        self._iparams = self._params_dev[2 * R:4 * R].view(2, R)
        self._lparams = self._params_dev[4 * R:].view(torch.int64).view(2, R)
        self._scratch: Optional[torch.Tensor] = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps = 0
        self.last_plan = (0, 0, 0)   # (prompt tokens, all tokens, requests) of the step launched last

    # ------------------------------------------------------------------ requests
    def submit(self, request_id: int, prompt: Sequence[int], params: Optional[SamplingParams] = None, priority: int = 0) -> None:
        p = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError(f"request {request_id}: the prompt is empty")
        for t in prompt:
            if not (0 <= t < self.engine.vocab_size):
                raise ValueError(f"request {request_id}: token id {t} is outside the vocabulary of {self.engine.vocab_size}")
        stops = list(self.engine.model.spec.stop_token_ids) if p.stop_token_ids is None else [int(t) for t in p.stop_token_ids]
        if self._inflight is not None and any(e.id == int(request_id) for e in self._inflight[0]):
            self._drain()                     # a token of an earlier request with this id is still on its way
        self.scheduler.submit(int(request_id), prompt, int(p.max_tokens), stops, int(priority))
        self.params[int(request_id)] = p
        self._logprobs.pop(int(request_id), None)

    def fork(self, parent_id: int, child_id: int, params: Optional[SamplingParams] = None, priority: int = 0) -> None:
        """A running request branches: the child continues from the parent's tokens so far on shared
        cache pages (copied only where one of the two writes), with its own sampling parameters."""
        self._drain()
        p = params or self.params.get(int(parent_id)) or SamplingParams()
        stops = list(self.engine.model.spec.stop_token_ids) if p.stop_token_ids is None else [int(t) for t in p.stop_token_ids]
        self.engine._do_copies(self.scheduler.fork(int(parent_id), int(child_id), int(p.max_tokens), stops, int(priority)))
        self.params[int(child_id)] = p

    # ------------------------------------------------------------------ one step
    def step(self) -> List[GenerationResult]:
        """Plan, run, sample, commit.  Returns the requests that finished in this step."""
        self._drain()
        plan = self.scheduler.plan()
        if plan.entries:
            rows, ids_dev = self._launch_or_rollback(plan, None)
            n = len(rows)
            m = self._copy_len(rows)
            host = self._ids_host2[self._turn & 1]
            host[:m].copy_(self._ids_dev2[self._turn & 1][:m], non_blocking=False)
            self.d2h_bytes += 4 * m
            vals = host[:n + 4].tolist()
            msg = K.wait_error_message(vals[n:])
            if msg:
                # the step's results are not valid: the requests go back to where they were
                K.read_wait_errors()
                self.scheduler.rollback()
                raise K.KernelError(msg)
            self._keep_logprobs(rows, host, m)
            self.scheduler.commit(vals[:n])
            self._log(plan, n)
        return self._finished()

    def _copy_len(self, rows) -> int:
        """How many words of the ids buffer a step brings to the host: ids, wait words and, if any
        of its requests wants them, log-probabilities."""
        n = len(rows)
        return 2 * n + 4 if any(e.id in self.params and self.params[e.id].logprobs for e in rows) else n + 4

    def _keep_logprobs(self, rows, host, m) -> None:
        n = len(rows)
        if m <= n + 4:
            return
        lp = host[n + 4:m].view(torch.float32).tolist()
        for e, v in zip(rows, lp):
            p = self.params.get(e.id)              # gone: the request ended on an earlier token (a stop id)
            if p is not None and p.logprobs:
                self._logprobs.setdefault(e.id, []).append(float(v))

    def _launch_or_rollback(self, plan, prev):
        """A launch that is refused (or any other failure before the step is committed) leaves the
        scheduler and the cache as they were before the plan."""
        try:
            return self._launch(plan, prev)
        except Exception:
            self.scheduler.rollback()
            raise

    def _launch(self, plan, prev):
        """Runs the planned step and chooses one token per finished input on the device.
        ``prev``: the step before, whose ids are still on the device: (request id -> row, ids)."""
        eng = self.engine
        entries = plan.entries
        eng._do_copies(plan.copies)
        self._turn += 1
        ids = [e.id for e in entries]
        counts = [len(e.tokens) for e in entries]
        flat = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int32, count=sum(counts))
        feed = None
        if flat.size and int(flat.min()) < 0:
            if prev is None:
                raise RuntimeError("a planned token has no value yet and there is no step to take it from")
            src = np.full(flat.size, -1, dtype=np.int32)
            t0 = 0
            for e, n in zip(entries, counts):
                if e.tokens[n - 1] < 0:
                    src[t0 + n - 1] = prev[0][e.id]
                t0 += n
            feed = (prev[1], src)
        want_rows, rows = [], []
        t0 = 0
        for e, n in zip(entries, counts):
            if e.wants_logits:
                want_rows.append(t0 + n - 1)
                rows.append(e)
            t0 += n
        logits = eng.run_reserved(ids, counts, flat, want_rows, feed=feed)
        self.h2d_bytes += 4 * eng._layout(t0, len(ids), len(want_rows))[1]
        self.steps += 1
        self.last_plan = (int(plan.prefill_tokens), int(plan.num_tokens), len(entries))
        ids_dev = self._sample(logits, rows) if rows else self._ids_dev2[self._turn & 1][:0]
        eng.collect_waits(self._ids_dev2[self._turn & 1][len(rows):len(rows) + 4])
        return rows, ids_dev

    def _log(self, plan, emitted: int) -> None:
        if _STEP_LOG:
            # one line per step, like the reference's AIEN_STEP_LOG (crates/aien-runtime/src/server.rs:273-293)
            print(f"step {plan.step_id}: prefill_tokens={plan.prefill_tokens} decode_tokens={plan.num_tokens - plan.prefill_tokens} "
                  f"requests={len(plan.entries)} emitted={emitted} preempted={len(plan.preempted)}", file=sys.stderr, flush=True)

    def _finished(self) -> List[GenerationResult]:
        out = []
        for ev in self.scheduler.take_finished():
            rec_pre = self.scheduler.record(ev.id).preemptions
            toks = list(ev.generated)
            lps = self._logprobs.pop(ev.id, None)
            if lps is not None or (ev.id in self.params and self.params[ev.id].logprobs):
                lps = (lps or [])[:len(toks)]          # a stop id and what was computed beyond it bring no token
            out.append(GenerationResult(ev.id, toks, _REASONS.get(ev.reason.name, ev.reason.name), ev.message, rec_pre, lps))
            self.params.pop(ev.id, None)
        return out

    def _sample(self, logits: torch.Tensor, rows) -> torch.Tensor:
        """One token per row on the device; the ids are the step's only device-to-host traffic."""
        R = len(rows)
        turn = self._turn & 1
        ps = [self.params[e.id] for e in rows]
        ids_dev = self._ids_dev2[turn][:R]
        want_lp = any(p.logprobs for p in ps)
        lp_dev = self._ids_dev2[turn][R + 4:2 * R + 4].view(torch.float32) if want_lp else None
        if all(p.greedy for p in ps) and not want_lp:
            K.argmax_rows(logits, ids_dev)
        else:
            f, i, l = self._params_np[turn]
            for r, (e, p) in enumerate(zip(rows, ps)):
                f[0, r], f[1, r] = p.temperature, p.top_p
                i[0, r], i[1, r] = p.top_k, e.start + len(e.tokens)
                l[0, r], l[1, r] = p.seed & 0x7FFFFFFFFFFFFFFF, e.id
            self._params_dev.copy_(self._params_host2[turn], non_blocking=True)
            self.h2d_bytes += self._params_dev.numel() * 4
            if self._scratch is None or self._scratch.numel() < R * logits.shape[1]:
                self._scratch = torch.empty(self.engine.max_requests * logits.shape[1], dtype=torch.float32, device=logits.device)
            K.sample_rows(logits, self._fparams[0], self._fparams[1], self._iparams[0], self._lparams[0], self._lparams[1],
                          self._iparams[1], self._scratch, ids_dev, lp_dev)
        return ids_dev

    # ------------------------------------------------------------------ steps that overlap
    def step_async(self) -> List[GenerationResult]:
        """Plans and launches the next step, then takes in the tokens of the step before it (which
        has had that long to finish).  Returns the requests that ended with those tokens."""
        prev = self._inflight
        plan = self.scheduler.plan()
        now = None
        if plan.entries:
            feed_from = ({e.id: r for r, e in enumerate(prev[0])}, prev[4]) if prev is not None else None
            rows, ids_dev = self._launch_or_rollback(plan, feed_from)
            n = len(rows)
            m = self._copy_len(rows)
            host = self._ids_host2[self._turn & 1]
            host[:m].copy_(self._ids_dev2[self._turn & 1][:m], non_blocking=True)
            ev = self._events[self._turn & 1]
            ev.record()
            self.d2h_bytes += 4 * m
            now = (rows, host, n, ev, ids_dev, m)
            self.scheduler.commit_deferred()
            self._log(plan, len(rows))
        self._inflight = now
        if prev is not None:
            self._resolve(prev)
        return self._finished()

    def advance(self) -> List[GenerationResult]:
        """One turn of the loop ``run`` makes: a step that overlaps the one before it, or a plain
        step, as the engine is configured.  ``flush`` takes in what is still in flight."""
        return self.step_async() if self.engine.cfg.async_scheduling else self.step()

    def flush(self) -> List[GenerationResult]:
        self._drain()
        return self._finished()

    def _resolve(self, flight) -> None:
        rows, host, n, ev, _, m = flight
        ev.synchronize()
        vals = host[:n + 4].tolist()
        msg = K.wait_error_message(vals[n:])
        if msg:
            # Later steps were launched on top of the broken one: nothing the running requests hold
            # can be trusted.  They are queued again and recomputed from the tokens known so far.
            torch.cuda.synchronize()
            K.read_wait_errors()
            self._inflight = None
            self.scheduler.restart_running()
            raise K.KernelError(msg)
        self._keep_logprobs(rows, host, m)
        if n:
            self.scheduler.resolve_for([(e.id, t, e.arrival) for e, t in zip(rows, vals[:n])])

    def _drain(self) -> None:
        """Takes in the tokens of a step that is still in flight."""
        if self._inflight is not None:
            flight, self._inflight = self._inflight, None
            self._resolve(flight)

    # ------------------------------------------------------------------ whole jobs
    def run(self, on_finish: Optional[Callable[[GenerationResult], None]] = None) -> Dict[int, GenerationResult]:
        """Step until nothing is left."""
        done: Dict[int, GenerationResult] = {}
        idle = 0
        while self.scheduler.has_work() or self._inflight is not None:
            before = self.steps
            for r in self.advance():
                done[r.request_id] = r
                if on_finish:
                    on_finish(r)
            idle = idle + 1 if (self.steps == before and self._inflight is None) else 0
            if idle > 2:
                raise RuntimeError("scheduler made no progress: waiting requests can never be admitted")
        return done

    def generate(self, prompts: Sequence[Sequence[int]], params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 request_ids: Optional[Sequence[int]] = None) -> List[GenerationResult]:
        """Token ids in, token ids out.  ``params`` is one SamplingParams for all or one each."""
        n = len(prompts)
        ids = list(request_ids) if request_ids is not None else [self._fresh_id() for _ in range(n)]
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * n
        for rid, prompt, p in zip(ids, prompts, plist):
            self.submit(rid, prompt, p)
        done = self.run()
        return [done[r] for r in ids]

    _next = 1

    def _fresh_id(self) -> int:
        Generator._next += 1
        return Generator._next - 1


def generate(engine: Engine, prompts: Sequence[Sequence[int]],
             params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
    """The plain entry point: lists of token ids in, lists of generated token ids out."""
    return [r.tokens for r in Generator(engine).generate(prompts, params)]


def generate_tokens(engine: Engine, seq_id: int, prompt_tokens: Sequence[int], max_tokens: int,
                    temperature: float = 0.0, stop_tokens: Optional[Sequence[int]] = None) -> List[int]:
    """One request, the reference's signature (transformer_backend.rs:643-664)."""
    p = SamplingParams(temperature=temperature, top_p=1.0, top_k=0, max_tokens=max_tokens,
                       stop_token_ids=list(stop_tokens) if stop_tokens is not None else None, seed=seq_id)
    return Generator(engine).generate([prompt_tokens], p, [seq_id])[0].tokens
