"""Sampling parameters and the host form of the engine's random numbers.

``SamplingParams`` carries the reference's fields with the reference's defaults
(crates/aien-abi-core/src/lib.rs:470-487: temperature 0.7, top_p 0.95, max_tokens 512) plus
``top_k`` (the reference's second generation stack has it, crates/aien-inference-abi/src/
qwen3_moe_omega.rs:3135-3160) and an explicit ``seed``.  ``stop_token_ids`` defaults to the
model's end-of-sequence ids rather than the reference's legacy ``[0, 1, 2]``.

The uniform number for the token at ``position`` of request ``request_id`` is
Philox4x32-10 with key ``seed`` and counter ``(position, 0, request_id)``: it depends on
nothing else, so a request samples the same tokens alone, batched, or recomputed after a
preemption.  (The reference derives a splitmix64 seed from the same two numbers,
crates/aien-inference-abi/src/transformer_backend.rs:45-60.)  The device kernel
(csrc/kernels/sampling.cu) computes the same function.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32_10(counter: Tuple[int, int, int, int], key: Tuple[int, int]) -> Tuple[int, int, int, int]:
    c0, c1, c2, c3 = (c & _MASK for c in counter)
    k0, k1 = (k & _MASK for k in key)
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def philox_uniform(seed: int, request_id: int, position: int) -> float:
    """The uniform number in [0, 1) (53 bits) the sampler uses for this (seed, request, position)."""
    seed &= 0xFFFFFFFFFFFFFFFF
    rid = request_id & 0xFFFFFFFFFFFFFFFF
    r = philox4x32_10((position, 0, rid & _MASK, rid >> 32), (seed & _MASK, seed >> 32))
    return float(((r[0] << 32) | r[1]) >> 11) * (1.0 / 9007199254740992.0)


@dataclass
class SamplingParams:
    temperature: float = 0.7
    top_p: float = 0.95
    top_k: int = 0
    max_tokens: int = 512
    stop_token_ids: Optional[Sequence[int]] = None      # None: the model's end-of-sequence ids
    seed: int = 0
    # Return the log-probability of every generated token with it, as the reference's outputs carry
    # it (crates/aien-abi-core/src/lib.rs:580-599, DecodeOutput::Token{logprob}): greedy, the log
    # softmax of the logits at the maximum; sampled, ln(p / kept mass) inside the set drawn from.
    logprobs: bool = False

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.001                # transformer_backend.rs:110
