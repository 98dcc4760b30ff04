"""Bind the tensors of a checkpoint to a catalog of wanted names and shapes.

The catalog is what the model's parts declare (name -> shape).  One :class:`WeightError`
reports everything that is wrong at once: missing tensors, wrong shapes and, under
``strict``, unexpected tensors; like the reference's catalog check (crates/aien-inference-abi/
src/checkpoint.rs:28-55, 262-319) but collected instead of first-error-only.  Without ``strict``
tensors the model does not want are left unread, as the reference leaves them (it has a
MissingTensor error and none for extras; src/weights.rs:854 skips ``lm_head.weight`` of a tied
model): a tied checkpoint that still ships its head, or old files with ``rotary_emb.inv_freq``,
load.

Dtype policy: bfloat16 stays bfloat16; a tensor stored in 32 bits stays 32-bit (float16 is
widened exactly to float32); integer tables become int32.  The float32 engine widens every
floating tensor to float32, which is exact for bfloat16 values.
"""
from __future__ import annotations

import sys
from typing import Dict, List, Mapping, Sequence, Tuple

import torch

from .safetensors_io import CheckpointFiles, SafetensorsError


class WeightError(ValueError):
    """The checkpoint does not fit the model: lists missing, unexpected and misshapen tensors."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} got {list(a)}" for n, e, a in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unsupported dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOAT = ("BF16", "F16", "F32")
_INT = ("I32", "I64", "U8")


def check_catalog(entries: Mapping[str, object], catalog: Mapping[str, Tuple[int, ...]], strict: bool = False) -> List[str]:
    """Raise one WeightError if names or shapes disagree; ``entries`` has ``.shape``/``.dtype``.
    Returns the names the model does not want: alone they are an error only under ``strict``;
    beside another fault they are listed in its error."""
    missing = [n for n in catalog if n not in entries]
    extra = sorted(n for n in entries if n not in catalog)
    wrong_shape, wrong_dtype = [], []
    for n, want in catalog.items():
        e = entries.get(n)
        if e is None:
            continue
        if tuple(e.shape) != tuple(want):
            wrong_shape.append((n, tuple(want), tuple(e.shape)))
        if e.dtype not in _FLOAT and e.dtype not in _INT:
            wrong_dtype.append((n, e.dtype))
    if missing or wrong_shape or wrong_dtype or (strict and extra):
        # the error names the unwanted tensors too: a missing tensor is often one stored under another name
        raise WeightError(sorted(missing), extra, wrong_shape, wrong_dtype)
    return extra


def _catalog_elements(catalog: Mapping[str, Tuple[int, ...]]) -> int:
    total = 0
    for shape in catalog.values():
        n = 1
        for d in shape:
            n *= int(d)
        total += n
    return total


def load_checkpoint(model_dir: str, catalog: Mapping[str, Tuple[int, ...]], dtype: str, strict: bool = False) -> Dict[str, torch.Tensor]:
    """CPU tensors for every catalog name, after the catalog check.  ``dtype`` is the engine's."""
    files = CheckpointFiles(model_dir)
    try:
        check_catalog(files.entries, catalog, strict)
        files.check_budget(_catalog_elements(catalog))
        out: Dict[str, torch.Tensor] = {}
        for name in catalog:
            out[name] = convert_stored(files.tensor(name), files.entries[name].dtype, dtype)
        return out
    finally:
        files.close()


def iter_checkpoint(model_dir: str, catalog: Mapping[str, Tuple[int, ...]], dtype: str, strict: bool = False):
    """Like :func:`load_checkpoint` but yields ``(name, tensor)`` one at a time (bounded host memory)."""
    files = CheckpointFiles(model_dir)
    try:
        extra = check_catalog(files.entries, catalog, strict)
        files.check_budget(_catalog_elements(catalog))
        if extra:
            print(f"[aien-b200] {len(extra)} tensors of the checkpoint are not used by the model: "
                  + ", ".join(extra[:8]) + (" ..." if len(extra) > 8 else ""), file=sys.stderr)
        for name in catalog:
            yield name, convert_stored(files.tensor(name), files.entries[name].dtype, dtype)
    finally:
        files.close()


def convert_stored(t: torch.Tensor, stored: str, engine_dtype: str) -> torch.Tensor:
    if stored in _INT:
        return t.to(torch.int32)
    if engine_dtype == "float32":
        return t.to(torch.float32)
    if stored == "BF16":
        return t
    return t.to(torch.float32)        # F32 stays, F16 widens exactly
