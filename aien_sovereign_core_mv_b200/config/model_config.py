"""Typed description of one dense decoder checkpoint, read from its ``config.json``.

Every size and constant the model needs comes from the keys of ``config.json``; nothing
here carries a default model size.  The accepted keys, their defaults and the refusals
follow the reference reader (crates/aien-inference-abi/src/model_dir.rs:39-265):

* required: ``hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
  vocab_size, rms_norm_eps, max_position_embeddings`` (model_dir.rs:116-139);
* optional: ``num_key_value_heads`` (-> heads), ``head_dim`` (-> hidden/heads, mandatory for
  Qwen3), ``rope_theta`` (-> 10000), ``rope_scaling`` (absent, null, ``default`` or ``llama3``),
  ``tie_word_embeddings`` (-> false);
* refused by field name: a ``hidden_act`` other than ``silu``, ``attention_bias`` or
  ``mlp_bias`` set, any sliding window, a ``layer_types`` entry other than
  ``full_attention``, an unknown ``rope_scaling`` type (model_dir.rs:72-111, 147-187, 213-218).

Deviation, stated: the reference refuses *unknown* Qwen3 keys by name (model_dir.rs:39-75).
Here that happens only with ``strict=True``; otherwise unknown keys that cannot change the
maths are ignored.  A missing ``eos_token_id`` gives an empty stop set instead of an error.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping, Optional, Sequence, Tuple


class ConfigError(ValueError):
    """A ``config.json`` this engine refuses; the message names the field."""


QWEN3_KNOWN_KEYS = frozenset(
    [
        "architectures", "attention_bias", "attention_dropout", "bos_token_id", "dtype",
        "eos_token_id", "head_dim", "hidden_act", "hidden_size", "initializer_range",
        "intermediate_size", "layer_types", "max_position_embeddings", "max_window_layers",
        "model_type", "num_attention_heads", "num_hidden_layers", "num_key_value_heads",
        "pad_token_id", "rms_norm_eps", "rope_scaling", "rope_theta", "sliding_window",
        "tie_word_embeddings", "torch_dtype", "transformers_version", "use_cache",
        "use_sliding_window", "vocab_size",
    ]
)

REQUIRED_KEYS = (
    "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
    "vocab_size", "rms_norm_eps", "max_position_embeddings",
)


@dataclass(frozen=True)
class Llama3RopeScaling:
    """Llama-3 frequency smoothing (crates/aien-abi-core/src/lib.rs:60-85)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class DenseDecoderConfig:
    """The typed form of a ``LlamaForCausalLM`` / ``Qwen3ForCausalLM`` ``config.json``."""

    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    max_position_embeddings: int
    rope_theta: float = 10000.0
    rope_scaling: Optional[Llama3RopeScaling] = None
    tie_word_embeddings: bool = False
    qk_norm: bool = False
    eos_token_ids: Tuple[int, ...] = ()

    # ---- derived sizes -------------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def to_hf_dict(self) -> dict:
        """The ``config.json`` that reads back into this object."""
        d: dict = {
            "architectures": [self.architecture],
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "torch_dtype": "bfloat16",
        }
        if self.architecture == "Qwen3ForCausalLM":
            d["model_type"] = "qwen3"
            d["attention_bias"] = False
        else:
            d["model_type"] = "llama"
        if self.rope_scaling is not None:
            d["rope_scaling"] = dict(rope_type="llama3", **asdict(self.rope_scaling))
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d


def _as_int(raw: Mapping[str, Any], key: str) -> int:
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer, got {v!r}")
    return v


def _parse_rope_scaling(value: Any) -> Optional[Llama3RopeScaling]:
    """model_dir.rs:147-187: absent/null/default -> plain rope, llama3 needs its four fields."""
    if value is None:
        return None
    if not isinstance(value, Mapping):
        raise ConfigError(f"rope_scaling must be an object, got {value!r}")
    rope_type = value.get("rope_type", value.get("type", "default"))
    if rope_type == "default":
        return None
    if rope_type != "llama3":
        raise ConfigError(
            f"unsupported rope_scaling rope_type {rope_type!r} (supported: default, llama3)"
        )
    out = {}
    for key in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings"):
        v = value.get(key)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"rope_scaling (llama3) has no numeric {key}")
        out[key] = v
    s = Llama3RopeScaling(
        float(out["factor"]), float(out["low_freq_factor"]), float(out["high_freq_factor"]),
        int(out["original_max_position_embeddings"]),
    )
    if s.factor <= 0 or s.high_freq_factor <= s.low_freq_factor or s.original_max_position_embeddings <= 0:
        raise ConfigError(f"rope_scaling (llama3) is degenerate: {s}")
    return s


def _eos_ids(obj: Optional[Mapping[str, Any]]) -> Optional[Tuple[int, ...]]:
    if not obj or "eos_token_id" not in obj or obj["eos_token_id"] is None:
        return None
    v = obj["eos_token_id"]
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, Sequence) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
        return tuple(v)
    raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {v!r}")


def _check_qwen3_fields(raw: Mapping[str, Any], strict: bool) -> None:
    """Refusals specific to Qwen3, each naming the field (model_dir.rs:72-111)."""
    if strict:
        unknown = sorted(k for k in raw if k not in QWEN3_KNOWN_KEYS)
        if unknown:
            raise ConfigError(f"unsupported Qwen3 config field {unknown[0]!r}")
    mt = raw.get("model_type")
    if mt != "qwen3" and (strict or mt is not None):
        raise ConfigError(f'unsupported model_type {mt!r} for Qwen3ForCausalLM (expected "qwen3")')
    hd = raw.get("head_dim")
    if isinstance(hd, bool) or not isinstance(hd, int):
        raise ConfigError("Qwen3 config.json must set head_dim (it is not hidden_size / num_attention_heads)")


def _check_window_fields(raw: Mapping[str, Any]) -> None:
    if raw.get("use_sliding_window", False) is not False:
        raise ConfigError("unsupported use_sliding_window (supported: false)")
    if raw.get("sliding_window") is not None and raw.get("use_sliding_window", None) is not False:
        # Llama-family files sometimes carry a number beside use_sliding_window=false; a
        # window that is switched on by no key is the only reading that changes nothing.
        raise ConfigError("unsupported sliding_window (supported: null)")
    types = raw.get("layer_types")
    if types is not None:
        if not isinstance(types, Sequence) or any(t != "full_attention" for t in types):
            raise ConfigError("unsupported layer_types (supported: every layer full_attention)")


def config_from_hf_dict(
    raw: Mapping[str, Any],
    generation_config: Optional[Mapping[str, Any]] = None,
    strict: bool = False,
) -> DenseDecoderConfig:
    """Build the typed configuration from the parsed ``config.json`` (model_dir.rs:192-265)."""
    if not isinstance(raw, Mapping):
        raise ConfigError("config.json is not an object")
    archs = raw.get("architectures") or []
    if not isinstance(archs, Sequence) or len(archs) != 1 or archs[0] not in ("LlamaForCausalLM", "Qwen3ForCausalLM"):
        raise ConfigError(
            f'unsupported architectures {list(archs)!r}: this engine runs ["LlamaForCausalLM"] or '
            f'["Qwen3ForCausalLM"] only'
        )
    arch = archs[0]
    missing = [k for k in REQUIRED_KEYS if k not in raw]
    if missing:
        raise ConfigError(f"config.json: missing field {missing[0]!r} (required: {', '.join(REQUIRED_KEYS)})")
    qk_norm = arch == "Qwen3ForCausalLM"
    if qk_norm:
        _check_qwen3_fields(raw, strict)
    _check_window_fields(raw)
    act = raw.get("hidden_act")
    if act is not None and act != "silu":
        raise ConfigError(f"unsupported hidden_act {act!r} (supported: silu)")
    if raw.get("attention_bias", False) or raw.get("mlp_bias", False):
        raise ConfigError("unsupported attention_bias/mlp_bias = true (no bias tensors)")

    hidden = _as_int(raw, "hidden_size")
    heads = _as_int(raw, "num_attention_heads")
    if not qk_norm and hidden % heads != 0:
        raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads}")
    head_dim = raw.get("head_dim")
    head_dim = hidden // heads if head_dim is None else _as_int(raw, "head_dim")
    if not qk_norm and head_dim * heads != hidden:
        raise ConfigError(
            f"unsupported head_dim {head_dim}: num_attention_heads * head_dim must equal hidden_size {hidden}"
        )
    kv_heads = raw.get("num_key_value_heads")
    kv_heads = heads if kv_heads is None else _as_int(raw, "num_key_value_heads")
    if heads % kv_heads != 0:
        raise ConfigError(
            f"attention geometry refused: num_attention_heads {heads} is not a multiple of "
            f"num_key_value_heads {kv_heads}"
        )
    if head_dim % 2 != 0:
        raise ConfigError(f"attention geometry refused: head_dim {head_dim} is odd (rotary pairs need an even size)")

    eps = raw["rms_norm_eps"]
    if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not (eps > 0) or not math.isfinite(eps):
        raise ConfigError(f"config.json: rms_norm_eps must be a positive number, got {eps!r}")

    # transformers >= 5 writes rope_theta / rope_type inside "rope_parameters"
    rope_params = raw.get("rope_parameters") if isinstance(raw.get("rope_parameters"), Mapping) else None
    theta = raw.get("rope_theta", rope_params.get("rope_theta") if rope_params else None)
    theta = 10000.0 if theta is None else theta
    if isinstance(theta, bool) or not isinstance(theta, (int, float)) or not (theta > 0):
        raise ConfigError(f"config.json: rope_theta must be a positive number, got {theta!r}")
    scaling_raw = raw.get("rope_scaling")
    if scaling_raw is None and rope_params is not None and rope_params.get("rope_type", "default") != "default":
        scaling_raw = rope_params
    rope_scaling = _parse_rope_scaling(scaling_raw)

    eos = _eos_ids(generation_config)
    if eos is None:
        eos = _eos_ids(raw)
    if eos is None:
        if strict:
            raise ConfigError("no eos_token_id in generation_config.json or config.json")
        eos = ()

    tie = raw.get("tie_word_embeddings", False)
    if not isinstance(tie, bool):
        raise ConfigError(f"config.json: tie_word_embeddings must be a boolean, got {tie!r}")

    return DenseDecoderConfig(
        architecture=arch,
        hidden_size=hidden,
        intermediate_size=_as_int(raw, "intermediate_size"),
        num_hidden_layers=_as_int(raw, "num_hidden_layers"),
        num_attention_heads=heads,
        num_key_value_heads=kv_heads,
        head_dim=head_dim,
        vocab_size=_as_int(raw, "vocab_size"),
        rms_norm_eps=float(eps),
        max_position_embeddings=_as_int(raw, "max_position_embeddings"),
        rope_theta=float(theta),
        rope_scaling=rope_scaling,
        tie_word_embeddings=tie,
        qk_norm=qk_norm,
        eos_token_ids=eos,
    )


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{model_dir}: no config.json") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"config.json: {e}") from None


def read_generation_config(model_dir: str) -> Optional[dict]:
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.exists(path):
        return None
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"generation_config.json: {e}") from None
