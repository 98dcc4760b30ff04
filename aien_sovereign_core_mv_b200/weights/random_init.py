"""Random weights from a configuration and a seed, as tensors or as a model folder.

Every tensor's values depend only on ``(seed, tensor name)``, so a folder written twice is
byte-identical and a catalog can be filled in any order.  The distributions are this
engine's own (the reference's LCG initialiser, crates/aien-inference-abi/src/weights.rs:159-264,
is not reproduced): matrices ``N(0, std)`` with ``std = 1/sqrt(fan_in)`` unless ``init_std`` is
given, embeddings ``N(0, 1)`` (or ``init_std``), norm weights ``U(0.8, 1.2)``.  Values are
rounded to bfloat16, so the bfloat16 and float32 engines read the same numbers.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Dict, Iterator, Mapping, Optional, Tuple

import torch

from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, shape: Tuple[int, ...], kind: str, seed: int,
                  init_std: Optional[float] = None, device: str = "cpu") -> torch.Tensor:
    """``kind``: "matrix" ([out, in]), "embedding", or "norm" (a vector of scales)."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if kind == "norm":
        t = torch.rand(shape, generator=g, device=device, dtype=torch.float32) * 0.4 + 0.8
    elif kind == "embedding":
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
        t *= 1.0 if init_std is None else init_std
    elif kind == "matrix":
        std = (1.0 / math.sqrt(shape[-1])) if init_std is None else init_std
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
        t *= std
    else:
        raise ValueError(f"unknown tensor kind {kind!r}")
    return t.to(torch.bfloat16)


def random_tensors(catalog: Mapping[str, Tuple[Tuple[int, ...], str]], seed: int,
                   init_std: Optional[float] = None, device: str = "cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    for name, (shape, kind) in catalog.items():
        yield name, random_tensor(name, tuple(shape), kind, seed, init_std, device)


def write_model_folder(out_dir: str, hf_config: Mapping, catalog: Mapping[str, Tuple[Tuple[int, ...], str]],
                       seed: int, init_std: Optional[float] = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``hf_config`` with random weights."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(hf_config), f, indent=1, sort_keys=True)
    tensors: Dict[str, torch.Tensor] = dict(random_tensors(catalog, seed, init_std))
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
