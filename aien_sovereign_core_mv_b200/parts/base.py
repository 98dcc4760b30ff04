"""What a part is, and what it sees of a step.

A model is built from seven families of parts.  Five are chosen per layer by the model spec:

* **norm**           ``forward(ctx, x, delta, out_dtype) -> h``; x is the float32 residual stream
  [T, H]; ``delta`` (or None) is added to it in place first.
* **position**       describes how positions enter the mixer.  ``rotary(ctx)`` returns
  ``(cos, sin, rotary_dim)`` tables for this step's tokens (or None), which the attention mixer
  feeds to its fused kernel; a part without tables implements ``apply(ctx, q, k)`` instead.
* **mixer**          ``forward(ctx, h, run) -> y``; h and y are [T, H] in the compute dtype.
  ``cache_need()`` says what it keeps between steps: pages of keys and values (all, or a
  window), a fixed-size state slot, or nothing.
* **feed_forward**   ``forward(ctx, h) -> y``.
* **block**          arranges the others: ``forward(ctx, x, delta, run) -> delta``; the returned
  delta is added to the residual stream by whoever norms next (the next block or the final
  norm), which fuses the residual sum into the norm kernel.

Two stand at the ends of the model: the **embedding** (``forward(ctx, token_ids, x)`` fills the
float32 residual stream) and the **head** (``forward(ctx, rows, logits)`` turns normed rows
into float32 logits; it may be tied to the embedding).

Every part lists its tensors with ``param_shapes()`` (local name -> (shape, kind)) and receives
them, already on the device, through ``bind(tensors)``.  A part takes its sizes and constants
as constructor parameters and never asks which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch


# ------------------------------------------------------------------ what a mixer keeps
@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps between steps.

    kind "full" (every token's entry stays), "window" (only the last ``window`` tokens' entries
    are needed; pages behind them are given back) or "state" (one tensor of fixed size per
    request).  A paged kind names its **planes**: what is stored per token, as (name, shape)
    pairs, e.g. keys and values of grouped-query attention ``(("k", (nkv, hd)), ("v", (nkv,
    hd)))`` or one latent ``(("latent", (r,)),)``.  The engine allocates, for every plane,
    ``[runs of the group, tokens of the pool, *shape]`` in the compute dtype (or ``dtype``) and
    knows nothing else about what they hold.  "state": ``state_shape`` / ``state_dtype``."""

    kind: str
    window: int = 0
    planes: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()
    dtype: Optional[str] = None           # paged planes: None = the engine's compute dtype
    state_shape: Tuple[int, ...] = ()     # "state": per-request tensor shape
    state_dtype: str = "float32"

    @staticmethod
    def keys_and_values(kind: str, window: int, num_kv_heads: int, head_dim: int) -> "CacheNeed":
        shape = (int(num_kv_heads), int(head_dim))
        return CacheNeed(kind, int(window), (("k", shape), ("v", shape)))

    def group_key(self) -> tuple:
        return (self.kind, self.window, self.planes, self.dtype, self.state_shape, self.state_dtype)


@dataclass
class GroupView:
    """One cache group as a step sees it (device tensors).

    ``storage`` maps a plane's name to ``[runs of the group, tokens, *shape]``; a run's own part
    is ``storage[name][run.slot]``.  A state group has the one plane "state":
    ``[runs, capacity + 1, *state_shape]``; the last slot belongs to nobody (padding rows of a
    captured step are pointed at it).

    The contract of fixed-size state, all of it on the device: the state slot of request ``s`` of
    the step is ``slot_map[s]``; the request's portion is the tokens ``q_start[s]`` to
    ``q_start[s + 1]``; a portion whose first token has position 0 (``positions[q_start[s]] ==
    0``) starts a new request and must not see what the slot held before.  A mixer that follows
    this without reading anything on the host leaves ``host_reads`` False and its steps can be
    captured in CUDA graphs like any other."""

    kind: str
    page_size: int
    window: int
    max_blocks: int
    block_table: Optional[torch.Tensor]    # int32 [S, max_blocks]; None for state groups
    slot_map: Optional[torch.Tensor]       # int32 [T] token slots (paged, -1: write nothing) or [S] state slots
    storage: Dict[str, torch.Tensor]


@dataclass
class RunBinding:
    """Where one run of a layer keeps its cache."""

    group: int = -1          # cache group index, -1: none
    slot: int = -1           # index of this run's planes inside the group's storage
    writes: bool = True      # False: attend over planes another run wrote


@dataclass
class StepContext:
    """Everything a part may use during one step.  Tensors are device tensors."""

    dtype: torch.dtype                     # compute dtype: bfloat16 or float32
    num_tokens: int                        # T (may include padding rows in a captured step)
    num_seqs: int                          # S
    token_ids: torch.Tensor                # int32 [T]
    positions: torch.Tensor                # int32 [T]
    seq_of_token: torch.Tensor             # int32 [T]
    q_start: torch.Tensor                  # int32 [S+1]
    ctx_len: torch.Tensor                  # int32 [S]
    groups: List[GroupView]
    workspace: "Workspace"
    # host copies for parts that plan on the host (never read in a captured step)
    host: Optional[Mapping[str, Any]] = None
    max_q_len: int = 0                     # longest portion in the step (host knowledge)
    max_ctx_len: int = 0
    decode_only: bool = False
    prefill_tiles: Optional[Tuple[torch.Tensor, torch.Tensor, int]] = None   # (tile_seq, tile_q0, count): query tiles of entries that bring several tokens
    single_tokens: Optional[Tuple[torch.Tensor, int]] = None                 # (token indices, count) of entries that bring one token, in a mixed step
    shared: Dict[Any, Any] = field(default_factory=dict)   # per-step memo (rotary tables ...)


@dataclass(frozen=True)
class StepLimits:
    """The largest step the engine will run; parts size their scratch from it."""

    max_tokens: int
    max_seqs: int
    max_context: int
    itemsize: int          # bytes of the compute dtype


_ELEMENT_SIZE = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int32: 4, torch.int64: 8, torch.uint8: 1, torch.float64: 8}


class Workspace:
    """Scratch for one step, carved from one device buffer so that a step allocates nothing
    and its addresses repeat (which a captured CUDA graph needs).

    Three regions: a *step* region that lives until the step ends (residual stream, rotary
    tables) and two *layer* regions used alternately: ``begin_layer()`` flips to the other one
    and empties it, so what a layer returns (its pending residual delta) stays valid while the
    next layer runs, and is recycled by the layer after that."""

    def __init__(self, step_bytes: int, layer_bytes: int, device: torch.device):
        self.step_bytes = (int(step_bytes) + 255) & ~255
        self.layer_bytes = (int(layer_bytes) + 255) & ~255
        self.buf = torch.empty(self.step_bytes + 2 * self.layer_bytes, dtype=torch.uint8, device=device)
        self._base = [0, self.step_bytes, self.step_bytes + self.layer_bytes]
        self._size = [self.step_bytes, self.layer_bytes, self.layer_bytes]
        self._off = [0, 0, 0]
        self._cur = 0

    def reset(self) -> None:
        self._off = [0, 0, 0]
        self._cur = 0

    def begin_layer(self) -> None:
        self._cur = 2 if self._cur == 1 else 1
        self._off[self._cur] = 0

    def end_layers(self) -> None:
        """Later takes come from the region not holding the last layer's result."""
        self.begin_layer()

    def _take(self, region: int, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * _ELEMENT_SIZE[dtype]
        start = (self._off[region] + 255) & ~255
        if start + nbytes > self._size[region]:
            which = "step" if region == 0 else "layer"
            raise RuntimeError(
                f"{which} workspace too small: need {start + nbytes} bytes, have {self._size[region]} "
                f"(the step brings more tokens than max_batch_tokens allows)")
        self._off[region] = start + nbytes
        lo = self._base[region] + start
        return self.buf[lo:lo + nbytes].view(dtype).view(*shape)

    def take(self, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self._take(self._cur, shape, dtype)

    def take_step(self, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self._take(0, shape, dtype)


# ------------------------------------------------------------------ a norm spread over its neighbours
@dataclass
class Prenormed:
    """A residual sum whose norm is half done: the sum is already in the residual stream,
    ``xw`` = bfloat16(x * norm weight) [T, H], and ``ssq`` [parts, 16] holds partial sums of x^2 per
    token.  What is left is the factor 1/sqrt(sum(ssq[:, t])/H + eps) per row; a product is
    linear in its rows, so the consumer's first product applies it to its result
    (``parts/linear.py: linear_prenormed``)."""

    xw: torch.Tensor
    ssq: torch.Tensor
    parts: int
    eps: float
    norm: "Norm"             # the norm this stands for

    def materialise(self, ctx: "StepContext") -> torch.Tensor:
        """The normalised rows themselves, for a consumer that cannot take the factor."""
        from .. import kernels as K
        out = ctx.workspace.take(tuple(self.xw.shape), torch.bfloat16)
        K.scale_rows_ssq(self.xw, self.ssq, self.parts, self.eps, out)
        return out


@dataclass
class ResidualSink:
    """Offered to a part whose last product ends a residual branch: instead of returning the
    branch's output for the next norm to add, the product may add it to ``x`` itself and return a
    :class:`Prenormed` for ``norm`` (``parts/linear.py: linear_into_residual``)."""

    x: torch.Tensor          # float32 residual stream [T, H]
    norm: "Norm"
    weight: torch.Tensor     # the norm's weight
    eps: float


# ------------------------------------------------------------------ part base classes
class Part:
    # True: forward() reads device data on the host (a synchronisation).  Steps of a model with
    # such a part are never captured in CUDA graphs.  Leave it False and work on the device.
    host_reads = False

    def param_shapes(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """local tensor name -> (shape, kind) with kind in {"matrix", "embedding", "norm"}."""
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the tensors named by param_shapes (device tensors, stored dtype kept)."""

    def workspace_bytes(self, lim: "StepLimits") -> int:
        """Upper bound of what forward() takes from the layer workspace within `lim`."""
        return 0


class Norm(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def sink(self, ctx: StepContext, x: torch.Tensor) -> Optional[ResidualSink]:
        """A norm of the form x * f(row) * weight may let the products around it do its work in
        this step: it then returns a ResidualSink for the producer, and its forward() passes the
        Prenormed it gets as ``delta`` on to the consumer.  None: not in this step, or never."""
        return None


class Position(Part):
    def rotary(self, ctx: StepContext):
        return None

    def apply(self, ctx: StepContext, q: torch.Tensor, group: "GroupView", run: "RunBinding") -> None:
        """Called instead of the fused rotation when rotary() returns None: may change q in
        place (and what the run just wrote into its cache slots)."""
        raise NotImplementedError


class Mixer(Part):
    takes_prenormed = False      # True: forward() accepts a Prenormed as h
    feeds_residual = False       # True: forward() accepts sink=ResidualSink and may return a Prenormed

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, ctx: StepContext, h: torch.Tensor, run: RunBinding) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    takes_prenormed = False
    feeds_residual = False

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    """Token ids to the float32 residual stream."""

    def forward(self, ctx: StepContext, token_ids: torch.Tensor, x: torch.Tensor) -> None:
        """x[t] = embedding of token_ids[t]; x is float32 [T, H]."""
        raise NotImplementedError

    def tied_weight(self) -> Optional[torch.Tensor]:
        """The [vocab, hidden] matrix a head tied to this embedding multiplies by (None: cannot be tied)."""
        return None


class Head(Part):
    """Normed rows to float32 logits."""

    tied = False

    def tie(self, embedding: Embedding) -> None:
        """Called instead of bind() when the head declares itself tied."""
        raise NotImplementedError

    def forward(self, ctx: StepContext, rows: torch.Tensor, logits: torch.Tensor) -> None:
        """logits [R, vocab] float32 from rows [R, H] in the compute dtype."""
        raise NotImplementedError


def add_to_residual(ctx: StepContext, x: torch.Tensor, delta) -> None:
    """x += delta for whatever a block may hand on as pending: None, a [T, H] tensor, float32
    partial products [P, T, H], or a Prenormed (whose sum is in x already).  For blocks that do
    not fuse the residual sum into a norm."""
    from .. import kernels as K
    if delta is None or isinstance(delta, Prenormed):
        return
    K.add_residual(x, delta)


class Block(Part):
    mixer: Mixer
    # the names of the norms the arrangement uses; the decoder builds one norm per name (from
    # LayerSpec.norms, else LayerSpec.norm) and passes it to the constructor under that name
    norm_slots: Tuple[str, ...] = ()
    chains_norm = False          # True: forward() accepts next_norm= (the norm that will take its result)

    def parts(self) -> Dict[str, Part]:
        """The block's parts by the names their tensors are stored under (below the layer's
        prefix): e.g. {"norm_in": ..., "mixer": ..., "feed_forward": ...}."""
        raise NotImplementedError

    def workspace_bytes(self, lim: "StepLimits") -> int:
        return sum(p.workspace_bytes(lim) for p in self.parts().values())

    def first_norm(self) -> Optional[Norm]:
        """The norm that takes the previous block's result, if the block starts with one."""
        return None

    def forward(self, ctx: StepContext, x: torch.Tensor, delta: Optional[torch.Tensor], run: RunBinding) -> torch.Tensor:
        raise NotImplementedError
