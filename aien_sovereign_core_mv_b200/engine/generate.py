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
        sc.max_context = engine.max_context
        self.scheduler = host.Scheduler(sc, engine.cache)
        self.params: Dict[int, SamplingParams] = {}
        R = engine.max_requests
        dev = engine.device
        self._ids_dev = torch.empty(R, dtype=torch.int32, device=dev)
        self._ids_host = torch.empty(R, dtype=torch.int32, pin_memory=True)
        self._fparams_host = torch.empty((2, R), dtype=torch.float32, pin_memory=True)      # temperature, top_p
        self._iparams_host = torch.empty((2, R), dtype=torch.int32, pin_memory=True)        # top_k, position
        self._lparams_host = torch.empty((2, R), dtype=torch.int64, pin_memory=True)        # seed, request id
        self._fparams = torch.empty((2, R), dtype=torch.float32, device=dev)
        self._iparams = torch.empty((2, R), dtype=torch.int32, device=dev)
        self._lparams = torch.empty((2, R), dtype=torch.int64, device=dev)
        self._scratch: Optional[torch.Tensor] = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps = 0

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
        self.scheduler.submit(int(request_id), prompt, int(p.max_tokens), stops, int(priority))
        self.params[int(request_id)] = p

    def fork(self, parent_id: int, child_id: int, params: Optional[SamplingParams] = None, priority: int = 0) -> None:
        """A running request branches: the child continues from the parent's tokens so far on shared
        cache pages (copied only where one of the two writes), with its own sampling parameters."""
        p = params or self.params.get(int(parent_id)) or SamplingParams()
        stops = list(self.engine.model.spec.stop_token_ids) if p.stop_token_ids is None else [int(t) for t in p.stop_token_ids]
        self.engine._do_copies(self.scheduler.fork(int(parent_id), int(child_id), int(p.max_tokens), stops, int(priority)))
        self.params[int(child_id)] = p

    # ------------------------------------------------------------------ one step
    def step(self) -> List[GenerationResult]:
        """Plan, run, sample, commit.  Returns the requests that finished in this step."""
        eng = self.engine
        plan = self.scheduler.plan()
        entries = plan.entries
        if entries:
            eng._do_copies(plan.copies)
            ids = [e.id for e in entries]
            counts = [len(e.tokens) for e in entries]
            flat = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int32, count=sum(counts))
            want_rows, rows = [], []
            t0 = 0
            for e, n in zip(entries, counts):
                if e.wants_logits:
                    want_rows.append(t0 + n - 1)
                    rows.append(e)
                t0 += n
            logits = eng.run_reserved(ids, counts, flat, want_rows)
            self.h2d_bytes += 4 * eng._layout(t0, len(ids), len(want_rows))[1]
            sampled: List[int] = []
            if rows:
                sampled = self._choose(logits, rows)
            self.scheduler.commit(sampled)
            self.steps += 1
            if _STEP_LOG:
                # one line per step, like the reference's AIEN_STEP_LOG (crates/aien-runtime/src/server.rs:273-293)
                print(f"step {plan.step_id}: prefill_tokens={plan.prefill_tokens} decode_tokens={plan.num_tokens - plan.prefill_tokens} "
                      f"requests={len(entries)} emitted={len(sampled)} preempted={len(plan.preempted)}", file=sys.stderr, flush=True)
        out = []
        for ev in self.scheduler.take_finished():
            rec_pre = self.scheduler.record(ev.id).preemptions
            out.append(GenerationResult(ev.id, list(ev.generated), _REASONS.get(ev.reason.name, ev.reason.name), ev.message, rec_pre))
            self.params.pop(ev.id, None)
        return out

    def _choose(self, logits: torch.Tensor, rows) -> List[int]:
        """One token per row on the device; the ids are the step's only device-to-host traffic."""
        R = len(rows)
        ps = [self.params[e.id] for e in rows]
        ids_dev = self._ids_dev[:R]
        if all(p.greedy for p in ps):
            K.argmax_rows(logits, ids_dev)
        else:
            f, i, l = self._fparams_host, self._iparams_host, self._lparams_host
            for r, (e, p) in enumerate(zip(rows, ps)):
                f[0, r], f[1, r] = p.temperature, p.top_p
                i[0, r], i[1, r] = p.top_k, e.start + len(e.tokens)
                l[0, r], l[1, r] = p.seed & 0x7FFFFFFFFFFFFFFF, e.id
            self._fparams.copy_(f, non_blocking=True)
            self._iparams.copy_(i, non_blocking=True)
            self._lparams.copy_(l, non_blocking=True)
            self.h2d_bytes += R * 24
            if self._scratch is None or self._scratch.numel() < R * logits.shape[1]:
                self._scratch = torch.empty(self.engine.max_requests * logits.shape[1], dtype=torch.float32, device=logits.device)
            K.sample_rows(logits, self._fparams[0], self._fparams[1], self._iparams[0], self._lparams[0], self._lparams[1],
                          self._iparams[1], self._scratch, ids_dev)
        self._ids_host[:R].copy_(ids_dev, non_blocking=False)
        self.d2h_bytes += 4 * R
        return self._ids_host[:R].tolist()

    # ------------------------------------------------------------------ whole jobs
    def run(self, on_finish: Optional[Callable[[GenerationResult], None]] = None) -> Dict[int, GenerationResult]:
        """Step until nothing is left."""
        done: Dict[int, GenerationResult] = {}
        idle = 0
        while self.scheduler.has_work():
            before = self.steps
            for r in self.step():
                done[r.request_id] = r
                if on_finish:
                    on_finish(r)
            idle = idle + 1 if self.steps == before else 0
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
