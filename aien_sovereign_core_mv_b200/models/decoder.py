"""The generic decoder: embedding, a run list of blocks, final norm, output head.

It is built from a :class:`ModelSpec` alone.  It knows nothing of architectures: which parts a
layer has, how many heads, whether the head is tied, in which order layers run and whose cache
a run reads are all data in the spec.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .. import kernels as K
from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..parts.base import Prenormed, Block, CacheNeed, Mixer, RunBinding, StepContext
from ..registry import make_part, part_factory


def _freeze(v):
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    if isinstance(v, (list, tuple)):
        return tuple(_freeze(x) for x in v)
    return v


class Decoder:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self._positions: Dict[tuple, object] = {}
        self.blocks: List[Block] = []
        for layer in spec.layers:
            self.blocks.append(self._build_block(layer))
        own = lambda ps: {k: v for k, v in ps.params.items() if k not in ("name", "names")}
        self.final_norm = make_part("norm", spec.final_norm.kind, size=spec.hidden_size, **own(spec.final_norm))
        self.embedding = make_part("embedding", spec.embedding.kind, vocab_size=spec.vocab_size, hidden_size=spec.hidden_size,
                                   **own(spec.embedding))
        self.head = make_part("head", spec.head.kind, vocab_size=spec.vocab_size, hidden_size=spec.hidden_size, **own(spec.head))
        self.tied = bool(getattr(self.head, "tied", False))
        # the parts outside the layers, with the spec entry that names their tensors
        self._ends = {"embedding": (self.embedding, spec.embedding), "final_norm": (self.final_norm, spec.final_norm),
                      "head": (self.head, spec.head)}
        # ---- cache groups: runs with equal needs share pools and block tables
        self.group_needs: List[CacheNeed] = []
        self.group_slots: List[int] = []          # planes (cache slots) per group
        self.bindings: List[RunBinding] = []
        slot_home: Dict[int, Tuple[int, int]] = {}
        for run in spec.run_list:
            need = self.blocks[run.layer].mixer.cache_need()
            if need is None or run.cache < 0:
                self.bindings.append(RunBinding(-1, -1, False))
                continue
            if run.writes_cache:
                key = need.group_key()
                for g, have in enumerate(self.group_needs):
                    if have.group_key() == key:
                        break
                else:
                    g = len(self.group_needs)
                    self.group_needs.append(need)
                    self.group_slots.append(0)
                slot_home[run.cache] = (g, self.group_slots[g])
                self.group_slots[g] += 1
                self.bindings.append(RunBinding(g, slot_home[run.cache][1], True))
            else:
                g, s = slot_home[run.cache]
                if self.group_needs[g].group_key() != need.group_key():
                    raise ValueError(f"a run reads cache slot {run.cache} whose layout differs from its own")
                self.bindings.append(RunBinding(g, s, False))

    # ------------------------------------------------------------------ construction
    def _position(self, ps: PartSpec):
        key = (ps.kind, _freeze(dict(ps.params)))
        if key not in self._positions:
            self._positions[key] = make_part("position", ps.kind, **dict(ps.params))
        return self._positions[key]

    def _build_block(self, layer: LayerSpec) -> Block:
        """The block kind says which norms it wants (``norm_slots``); the layer spec says what each
        is.  Nothing here knows an arrangement."""
        position = self._position(layer.position)
        mixer = make_part("mixer", layer.mixer.kind, position=position, **dict(layer.mixer.params))
        ff = None if layer.feed_forward is None else make_part("feed_forward", layer.feed_forward.kind, **dict(layer.feed_forward.params))
        norms = {}
        for slot in getattr(part_factory("block", layer.block), "norm_slots", ()):
            ps = layer.norm_for(slot)
            norms[slot] = make_part("norm", ps.kind, size=self.spec.hidden_size, **dict(ps.params))
        return make_part("block", layer.block, mixer=mixer, feed_forward=ff, **norms, **dict(layer.block_params))

    def parts(self):
        """Every part of the model, for whoever must ask all of them something."""
        out = [self.embedding, self.final_norm, self.head] + list(self._positions.values())
        for block in self.blocks:
            out.append(block)
            out.extend(block.parts().values())
        return out

    def _end_names(self):
        """(which end, local name) -> (checkpoint name, shape, kind)."""
        out = {}
        for which, (part, ps) in self._ends.items():
            names = dict(ps.params.get("names") or {})
            for local, (shape, kind) in part.param_shapes().items():
                name = names.get(local) or (ps.params.get("name") if local == "weight" else None) or f"{which}.{local}"
                out[(which, local)] = (name, tuple(shape), kind)
        return out

    # ------------------------------------------------------------------ tensors
    def _layer_names(self, li: int):
        """(part name, local name) -> checkpoint name, for layer li."""
        layer = self.spec.layers[li]
        out = {}
        for pname, part in self.blocks[li].parts().items():
            for local, (shape, kind) in part.param_shapes().items():
                key = f"{pname}.{local}"
                out[(pname, local)] = (layer.prefix + layer.names.get(key, key), shape, kind)
        return out

    def catalog(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """Every tensor the model wants: checkpoint name -> (shape, kind)."""
        cat: Dict[str, Tuple[Tuple[int, ...], str]] = {}
        ends = self._end_names()
        for (which, _), (name, shape, kind) in ends.items():
            if which == "embedding":
                cat[name] = (shape, kind)
        for li in range(len(self.blocks)):
            for (_, _), (name, shape, kind) in self._layer_names(li).items():
                cat[name] = (tuple(shape), kind)
        for (which, _), (name, shape, kind) in ends.items():
            if which != "embedding":
                cat[name] = (shape, kind)
        return cat

    def bind(self, tensors) -> None:
        """``tensors``: iterable of (checkpoint name, tensor); each is moved to the device as it
        arrives and handed to its part once the part's set is complete."""
        device = torch.device("cuda")
        owner: Dict[str, Tuple[int, str, str]] = {}
        for li in range(len(self.blocks)):
            for (pname, local), (name, _, _) in self._layer_names(li).items():
                owner[name] = (li, pname, local)
        for (which, local), (name, _, _) in self._end_names().items():
            owner[name] = (-1, which, local)
        pending: Dict[Tuple[int, str], Dict[str, torch.Tensor]] = {}
        waiting = {(-1, which) for which, (part, _) in self._ends.items() if part.param_shapes()}
        for name, t in tensors:
            t = t.to(device, non_blocking=False)
            if name not in owner:
                raise KeyError(f"tensor {name!r} belongs to no part of the model")
            li, pname, local = owner[name]
            part = self._ends[pname][0] if li < 0 else self.blocks[li].parts()[pname]
            bucket = pending.setdefault((li, pname), {})
            bucket[local] = t
            if len(bucket) == len(part.param_shapes()):
                part.bind(bucket)
                del pending[(li, pname)]
                waiting.discard((li, pname))
        if self.tied:
            self.head.tie(self.embedding)
        if pending or waiting:
            raise RuntimeError("bind: some parts did not receive all their tensors")

    # ------------------------------------------------------------------ sizes
    def layer_workspace_bytes(self, lim) -> int:
        head = lim.max_tokens * self.hidden_size * (4 + lim.itemsize) + 4096
        return max(max(b.workspace_bytes(lim) for b in self.blocks), head) + (1 << 16)

    def step_workspace_bytes(self, lim) -> int:
        n = lim.max_tokens * self.hidden_size * 4 + 4096
        for p in self._positions.values():
            if hasattr(p, "step_workspace_bytes"):
                n += p.step_workspace_bytes(lim.max_tokens)
        return n

    # ------------------------------------------------------------------ one step
    def forward(self, ctx: StepContext, want_rows: torch.Tensor, num_rows: int, logits: torch.Tensor) -> torch.Tensor:
        """Runs the step's tokens through the run list; writes float32 logits of the wanted
        rows into ``logits`` [num_rows, vocab]."""
        ws = ctx.workspace
        x = ws.take_step((ctx.num_tokens, self.hidden_size), torch.float32)
        self.embedding.forward(ctx, ctx.token_ids, x)
        delta = None
        runs = self.spec.run_list
        for i, (run, binding) in enumerate(zip(runs, self.bindings)):
            ws.begin_layer()
            block = self.blocks[run.layer]
            if block.chains_norm:
                # the norm that will take this block's result, so that the block's last product may work for it
                nxt = self.blocks[runs[i + 1].layer].first_norm() if i + 1 < len(runs) else None
                delta = block.forward(ctx, x, delta, binding, next_norm=nxt)
            else:
                delta = block.forward(ctx, x, delta, binding)
        ws.end_layers()
        if isinstance(delta, Prenormed):          # the last block has no next norm; a block of another kind may still return one
            delta = None
        if num_rows > 0:
            rows = ws.take((num_rows, self.hidden_size), torch.float32)
            K.gather_add_rows(x, delta, want_rows, rows)
            hn = self.final_norm.forward(ctx, rows, None)
            self.head.forward(ctx, hn, logits)
        return logits
