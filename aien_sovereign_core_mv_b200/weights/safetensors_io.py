"""A small reader and writer for the safetensors container, by tensor name.

File layout: 8 bytes little-endian header length ``n``, ``n`` bytes of JSON mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the first
byte after the header), then the data.  The checks mirror the reference's strict reader
(crates/aien-inference-abi/src/checkpoint.rs:415-538): header size bound, offsets inside the
file, ``end - begin`` equal to the byte size of ``shape`` x ``dtype``, no overlap, no duplicate
name across shards.  A directory may hold ``model.safetensors`` or a sharded set named by
``model.safetensors.index.json`` (``weight_map``), whose shard names must be plain file names
(checkpoint.rs:642-663, 750-802).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Iterator, List, Mapping, Optional, Tuple

import numpy as np
import torch

# Bounds on what is read from disk (crates/aien-inference-abi/src/checkpoint.rs:552-556): absurd
# metadata and sparse files of absurd length are refused before anything is mapped.
MAX_INDEX_BYTES = 16 << 20
MAX_HEADER_BYTES = 256 << 20
MAX_SHARD_BYTES = 256 << 30
MAX_CHECKPOINT_BYTES = 1 << 40

_DTYPE_BYTES = {"BF16": 2, "F16": 2, "F32": 4, "I32": 4, "I64": 8, "U8": 1, "F64": 8}
_TORCH_OF = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32,
    "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8, "F64": torch.float64,
}
_NAME_OF = {v: k for k, v in _TORCH_OF.items()}
_NUMPY_VIEW = {"BF16": np.uint16, "F16": np.float16, "F32": np.float32, "I32": np.int32,
               "I64": np.int64, "U8": np.uint8, "F64": np.float64}


class SafetensorsError(ValueError):
    """The container itself is malformed (header, offsets, dtype)."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int          # absolute file offset
    end: int
    file: str


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def read_header(path: str) -> Dict[str, TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        first = f.read(8)
        if len(first) != 8:
            raise SafetensorsError(f"{path}: invalid header: file shorter than 8 bytes")
        (n,) = struct.unpack("<Q", first)
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise SafetensorsError(f"{path}: invalid header: length {n} exceeds the file or the {MAX_HEADER_BYTES}-byte limit")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: invalid header: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: invalid header: not an object")
    base = 8 + n
    entries: Dict[str, TensorEntry] = {}
    spans: List[Tuple[int, int, str]] = []
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (b, e) = meta["dtype"], tuple(int(s) for s in meta["shape"]), meta["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: invalid header: entry {name!r} lacks dtype/shape/data_offsets") from None
        if dtype not in _DTYPE_BYTES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
        if any(s < 0 for s in shape) or b < 0 or e < b:
            raise SafetensorsError(f"{path}: tensor {name!r} has a negative size or offset")
        if e - b != _numel(shape) * _DTYPE_BYTES[dtype]:
            raise SafetensorsError(
                f"{path}: tensor {name!r}: {e - b} bytes stored, shape {list(shape)} of {dtype} needs "
                f"{_numel(shape) * _DTYPE_BYTES[dtype]}"
            )
        if base + e > size:
            raise SafetensorsError(f"{path}: tensor {name!r}: offset {e} is out of bounds of the data section")
        entries[name] = TensorEntry(name, dtype, shape, base + b, base + e, path)
        spans.append((b, e, name))
    spans.sort()
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise SafetensorsError(f"{path}: tensors {n0!r} and {n1!r} overlap")
    return entries


def resolve_files(model_dir_or_file: str) -> List[str]:
    """The safetensors files of a model folder, in a fixed order."""
    p = model_dir_or_file
    if os.path.isfile(p):
        return [p]
    single = os.path.join(p, "model.safetensors")
    index = os.path.join(p, "model.safetensors.index.json")
    if os.path.exists(index):
        if os.path.getsize(index) > MAX_INDEX_BYTES:
            raise SafetensorsError(f"{index}: index exceeds {MAX_INDEX_BYTES} bytes")
        with open(index, "r", encoding="utf-8") as f:
            try:
                wm = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as e:
                raise SafetensorsError(f"{index}: invalid index: {e}") from None
        shards = sorted(set(wm.values()))
        for s in shards:
            if not isinstance(s, str) or os.path.basename(s) != s or s in ("", ".", ".."):
                raise SafetensorsError(f"{index}: shard name {s!r} is not a plain file name")
        return [os.path.join(p, s) for s in shards]
    if os.path.exists(single):
        return [single]
    raise SafetensorsError(f"{p}: no model.safetensors and no model.safetensors.index.json")


class CheckpointFiles:
    """All tensors of a model folder by name; data is memory-mapped and read on demand."""

    def __init__(self, model_dir_or_file: str):
        self.files = resolve_files(model_dir_or_file)
        self.entries: Dict[str, TensorEntry] = {}
        self.total_bytes = 0
        for path in self.files:
            if not os.path.isfile(path) or os.path.islink(path):
                raise SafetensorsError(f"{path}: not a regular file")
            size = os.path.getsize(path)
            if size > MAX_SHARD_BYTES:
                raise SafetensorsError(f"{path}: file exceeds {MAX_SHARD_BYTES} bytes")
            self.total_bytes += size
            if self.total_bytes > MAX_CHECKPOINT_BYTES:
                raise SafetensorsError(f"{path}: checkpoint exceeds the aggregate limit of {MAX_CHECKPOINT_BYTES} bytes")
            for name, e in read_header(path).items():
                if name in self.entries:
                    raise SafetensorsError(f"tensor {name!r} is stored twice ({self.entries[name].file} and {path})")
                self.entries[name] = e
        self._maps: Dict[str, mmap.mmap] = {}

    def names(self) -> List[str]:
        return list(self.entries)

    def check_budget(self, catalog_elements: int) -> None:
        """A small model must not authorise a huge payload: the files together may hold at most
        twice the catalog's bytes at two bytes an element, plus one header budget per file
        (checkpoint.rs:836-857).  Room for extra tensors and for 32-bit storage, not for more."""
        budget = min(2 * (2 * int(catalog_elements)) + len(self.files) * (MAX_HEADER_BYTES + 8), MAX_CHECKPOINT_BYTES)
        if self.total_bytes > budget:
            raise SafetensorsError(f"checkpoint of {self.total_bytes} bytes exceeds the catalog byte budget {budget}")

    def _map(self, path: str) -> mmap.mmap:
        m = self._maps.get(path)
        if m is None:
            with open(path, "rb") as f:
                m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[path] = m
        return m

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor with the stored dtype (a private copy, detached from the file)."""
        e = self.entries[name]
        buf = self._map(e.file)
        arr = np.frombuffer(buf, dtype=_NUMPY_VIEW[e.dtype], count=_numel(e.shape), offset=e.begin)
        t = torch.from_numpy(arr.copy())
        if e.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(e.shape)

    def close(self) -> None:
        for m in self._maps.values():
            m.close()
        self._maps.clear()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write ``tensors`` (CPU or device; copied to the host one at a time) to one file."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = list(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAME_OF:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAME_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((-len(blob)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)
