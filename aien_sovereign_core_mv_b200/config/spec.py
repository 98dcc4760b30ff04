"""The model as data: which parts each layer is made of, and in which order layers run.

A :class:`ModelSpec` is what an architecture builder returns for a ``config.json``.  The
generic decoder builds itself from it; nothing in the parts or in the decoder knows which
architecture produced the spec.

* ``PartSpec(kind, params)`` names a registered part and gives its sizes and constants.
* ``LayerSpec`` lists the parts of one layer (block arrangement, mixer, feed-forward, the norms
  by the slot names the block declares, position encoding) and the prefix under which its
  tensors are stored.  ``ModelSpec.embedding`` and ``ModelSpec.head`` name registered parts too.
* ``RunEntry`` is one execution of a layer.  The run list may name a layer twice (shared
  weights) and a run may read the cache another run wrote (``cache`` equal to an earlier
  entry's and ``writes_cache=False``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    block: str                      # arrangement of the parts, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: Optional[PartSpec]  # None: the block has no feed-forward
    norm: Optional[PartSpec]        # the norm of every slot of the block that `norms` does not name
    position: PartSpec              # handed to the mixer
    prefix: str                     # tensor-name prefix, e.g. "model.layers.3."
    # local tensor name of a part -> name below `prefix` in the checkpoint
    names: Mapping[str, str] = field(default_factory=dict)
    # norm slot name (as the block kind declares them: Block.norm_slots) -> its norm
    norms: Mapping[str, PartSpec] = field(default_factory=dict)
    # further constructor arguments of the block
    block_params: Mapping[str, Any] = field(default_factory=dict)

    def norm_for(self, slot: str) -> PartSpec:
        ps = self.norms.get(slot, self.norm)
        if ps is None:
            raise ValueError(f"layer {self.prefix!r}: block {self.block!r} wants a norm in slot {slot!r} and the spec names none")
        return ps


@dataclass(frozen=True)
class RunEntry:
    layer: int                      # index into ModelSpec.layers
    cache: int                      # cache slot this run attends over (-1: the mixer keeps none)
    writes_cache: bool = True       # False: read a slot that an earlier run wrote


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    run_list: Tuple[RunEntry, ...]
    # Each of the three is a registered part; ``name`` in its params is the checkpoint name of its
    # tensor "weight" (``names`` maps further local names); the rest are constructor arguments.
    embedding: PartSpec             # family "embedding", e.g. kind "table"
    final_norm: PartSpec            # family "norm"
    head: PartSpec                  # family "head", e.g. kind "linear" with tied=True/False
    max_position: int
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        n = len(self.layers)
        written: Dict[int, int] = {}
        for i, run in enumerate(self.run_list):
            if not (0 <= run.layer < n):
                raise ValueError(f"run_list[{i}] names layer {run.layer}, model has {n}")
            if run.cache < 0:
                continue
            if run.writes_cache:
                if run.cache in written:
                    raise ValueError(
                        f"run_list[{i}] writes cache slot {run.cache}, which run_list[{written[run.cache]}] already writes"
                    )
                written[run.cache] = i
            elif run.cache not in written:
                raise ValueError(f"run_list[{i}] reads cache slot {run.cache} before any run writes it")


def default_run_list(num_layers: int) -> Tuple[RunEntry, ...]:
    return tuple(RunEntry(layer=i, cache=i, writes_cache=True) for i in range(num_layers))
