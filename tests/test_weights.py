"""Weights: container checks, binding by name, the one error that lists everything wrong,
dtype policy, random model folders."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as pm
from aien_sovereign_core_mv_b200 import WeightError, SafetensorsError, model_spec_for, write_random_model
from aien_sovereign_core_mv_b200.models import Decoder
from aien_sovereign_core_mv_b200.weights import CheckpointFiles, load_checkpoint, read_header, write_safetensors


def catalog_of(which):
    _, spec = model_spec_for(H.TINY[which])
    return {n: s for n, (s, _) in Decoder(spec).catalog().items()}


def test_random_folder_round_trip_and_determinism(tmp_path):
    a = write_random_model(str(tmp_path / "a"), H.TINY["B"], 7)
    b = write_random_model(str(tmp_path / "b"), H.TINY["B"], 7)
    c = write_random_model(str(tmp_path / "c"), H.TINY["B"], 8)
    ba, bb, bc = (open(os.path.join(d, "model.safetensors"), "rb").read() for d in (a, b, c))
    assert ba == bb and ba != bc
    cat = catalog_of("B")
    assert "lm_head.weight" not in cat and "model.layers.2.self_attn.q_norm.weight" in cat      # tied, q/k norm
    t = load_checkpoint(a, cat, "bfloat16")
    assert set(t) == set(cat) and all(v.dtype == torch.bfloat16 for v in t.values())
    t32 = load_checkpoint(a, cat, "float32")
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["model.norm.weight"], t["model.norm.weight"].float())
    # the engine's reader and the plain reader agree
    _, plain = pm.load_model_folder(a)
    for name in cat:
        assert np.array_equal(plain[name], t32[name].double().numpy())
    w = t32["model.layers.0.input_layernorm.weight"]
    assert 0.79 <= float(w.min()) and float(w.max()) <= 1.21
    assert json.load(open(os.path.join(a, "config.json")))["vocab_size"] == 512


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    d = write_random_model(str(tmp_path / "m"), H.TINY["A"], 1)
    f = CheckpointFiles(d)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16, dtype=torch.bfloat16)
    tensors["lm_head.weight"] = tensors["lm_head.weight"][:, :32].contiguous()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_checkpoint(d, catalog_of("A"), "bfloat16")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert err.wrong_shape == [("lm_head.weight", (256, 64), (256, 32))]
    msg = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected [256, 64] got [256, 32]"):
        assert needle in msg


def test_untied_config_without_lm_head_is_refused(tmp_path):
    d = write_random_model(str(tmp_path / "m"), H.TINY["B"], 1)          # tied: no lm_head stored
    raw = dict(H.TINY["B"]); raw["tie_word_embeddings"] = False
    _, spec = model_spec_for(raw)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_checkpoint(d, {n: s for n, (s, _) in Decoder(spec).catalog().items()}, "bfloat16")


def test_dtype_policy(tmp_path):
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": torch.ones(2, 3, dtype=torch.float32), "b": torch.ones(4, dtype=torch.bfloat16),
                          "c": torch.arange(5, dtype=torch.int64), "d": torch.ones(2, dtype=torch.float16)})
    cat = {"a": (2, 3), "b": (4,), "c": (5,), "d": (2,)}
    t = load_checkpoint(p, cat, "bfloat16")
    assert t["a"].dtype == torch.float32          # stored in 32 bits: stays so
    assert t["b"].dtype == torch.bfloat16
    assert t["c"].dtype == torch.int32            # integer tables become int32
    assert t["d"].dtype == torch.float32          # float16 widens exactly
    t = load_checkpoint(p, cat, "float32")
    assert t["b"].dtype == torch.float32 and t["c"].dtype == torch.int32


def _raw_file(path, header, data=b""):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + data)


def test_container_checks(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter than 8"):
        read_header(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError, match="exceeds"):
        read_header(p)
    _raw_file(p, {"t": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 6]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 8"):
        read_header(p)
    _raw_file(p, {"t": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 8]}}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="out of bounds"):
        read_header(p)
    _raw_file(p, {"t": {"dtype": "BF16", "shape": [2], "data_offsets": [0, 4]}, "u": {"dtype": "BF16", "shape": [2], "data_offsets": [2, 6]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="overlap"):
        read_header(p)
    _raw_file(p, {"t": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 1]}}, b"\0")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        read_header(p)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        CheckpointFiles(str(tmp_path))


def test_sharded_index(tmp_path):
    d = str(tmp_path)
    write_safetensors(os.path.join(d, "s1.safetensors"), {"a": torch.ones(2, dtype=torch.bfloat16)})
    write_safetensors(os.path.join(d, "s2.safetensors"), {"b": torch.zeros(3, dtype=torch.bfloat16)})
    json.dump({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    t = load_checkpoint(d, {"a": (2,), "b": (3,)}, "bfloat16")
    assert t["a"].sum() == 2 and t["b"].numel() == 3
    json.dump({"weight_map": {"a": "../s1.safetensors"}}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    with pytest.raises(SafetensorsError, match="plain file name"):
        CheckpointFiles(d)
    write_safetensors(os.path.join(d, "s2.safetensors"), {"a": torch.zeros(2, dtype=torch.bfloat16)})
    json.dump({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    with pytest.raises(SafetensorsError, match="stored twice"):
        CheckpointFiles(d)


def test_extra_tensors_load_unless_strict(tmp_path):
    """A tied checkpoint that still ships lm_head.weight, or old files with rotary_emb.inv_freq, load
    in the reference (crates/aien-inference-abi/src/weights.rs:854 skips the head of a tied model;
    checkpoint.rs has no error for extras); here too, and `strict` refuses them by name."""
    d = write_random_model(str(tmp_path / "m"), H.TINY["B"], 1)          # tied
    f = CheckpointFiles(d)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(16, dtype=torch.float32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    got = load_checkpoint(d, catalog_of("B"), "bfloat16")
    assert set(got) == set(catalog_of("B"))
    with pytest.raises(WeightError) as e:
        load_checkpoint(d, catalog_of("B"), "bfloat16", strict=True)
    assert e.value.unexpected == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"] and not e.value.missing


def test_size_caps(tmp_path, monkeypatch):
    """A small catalog does not authorise a huge payload (crates/aien-inference-abi/src/checkpoint.rs:552-556, 836-857)."""
    import aien_sovereign_core_mv_b200.weights.safetensors_io as sio
    d = write_random_model(str(tmp_path / "m"), H.TINY["A"], 1)
    cat = catalog_of("A")
    load_checkpoint(d, cat, "bfloat16")
    f = CheckpointFiles(d)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    tensors["padding"] = torch.zeros(4 * sum(t.numel() for t in tensors.values()), dtype=torch.bfloat16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    load_checkpoint(d, cat, "bfloat16")                                # inside the real budget (one header allowance)
    monkeypatch.setattr(sio, "MAX_HEADER_BYTES", 1 << 16)          # shrink the header allowance: the budget is 2 x catalog bytes
    with pytest.raises(sio.SafetensorsError, match="catalog byte budget"):
        load_checkpoint(d, cat, "bfloat16")
    monkeypatch.setattr(sio, "MAX_SHARD_BYTES", 1000)
    with pytest.raises(sio.SafetensorsError, match="file exceeds 1000 bytes"):
        load_checkpoint(d, cat, "bfloat16")
