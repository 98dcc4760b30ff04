"""The engine against the reference project's own data.

The reference ships two tiny checkpoints with logits that transformers computed in float32
(crates/aien-inference-abi/fixtures/qwen3-tiny and openwaldo-byte: q/k norm on and off, tied
head, grouped heads, nq*hd != hidden, theta 1e6 and 1e4, eps 1e-6 and 1e-5) and an independently
computed table of llama3-scaled inverse frequencies (src/model_dir.rs:409-455).  These tests
hold the product path to them, the way the reference's own tests do
(tests/qwen3_forward_parity.rs:108-188, tests/openwaldo_forward_parity.rs:34-74,
tests/qwen3_untied_head.rs:128-172).  They need the reference's files: beside this repository
as ``../reference``, or where ``AIEN_REFERENCE_DIR`` points; otherwise they are skipped.
"""
import dataclasses
import json
import os
import re
import shutil

import numpy as np
import pytest

import plain_model as pm

_REF = os.environ.get("AIEN_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
ABI = os.path.join(_REF, "crates", "aien-inference-abi")
FIX = os.path.join(ABI, "fixtures")
TOL = 1e-4            # absolute, the reference's own bound (tests/qwen3_forward_parity.rs:46)
NAMES = ["qwen3-tiny", "openwaldo-byte"]


def fixture(name):
    d = os.path.join(FIX, name)
    if not os.path.isdir(d):
        pytest.skip("reference fixtures are not mounted")
    ref = json.load(open(os.path.join(d, "forward_reference.json")))
    return d, [int(t) for t in ref["ids"]], np.array(ref["logits"], dtype=np.float64), ref.get("argmax")


# ------------------------------------------------------------------ CPU: loader and catalog
@pytest.mark.parametrize("strict", [False, True])
@pytest.mark.parametrize("name", NAMES)
def test_loader_and_catalog_bind_the_fixture(name, strict):
    from aien_sovereign_core_mv_b200.config.model_config import read_config_json, read_generation_config
    from aien_sovereign_core_mv_b200.models.decoder import Decoder
    from aien_sovereign_core_mv_b200.models.loading import model_spec_for
    from aien_sovereign_core_mv_b200.weights.loader import load_checkpoint
    d, _, _, _ = fixture(name)
    cfg, spec = model_spec_for(read_config_json(d), read_generation_config(d), strict)
    catalog = {n: s for n, (s, _) in Decoder(spec).catalog().items()}
    tensors = load_checkpoint(d, catalog, "float32", strict=strict)
    assert set(tensors) == set(catalog) and len(tensors) == (24 if name == "qwen3-tiny" else 11)
    assert all(tuple(tensors[n].shape) == tuple(catalog[n]) for n in catalog)
    assert cfg.qk_norm == (name == "qwen3-tiny") and cfg.tie_word_embeddings


def test_llama3_inverse_frequencies_match_the_reference_table():
    """Both the product's table and the plain implementation's against the reference's
    independently computed values for Llama-3.2-1B (theta 500000, head 64, factor 32, low 1,
    high 4, original 8192), read from the reference's source file."""
    path = os.path.join(ABI, "src", "model_dir.rs")
    if not os.path.isfile(path):
        pytest.skip("reference sources are not mounted")
    m = re.search(r"LLAMA32_1B_INV_FREQ: \[f64; 32\] = \[(.*?)\];", open(path).read(), re.S)
    want = np.array([float(v) for v in m.group(1).replace("\n", " ").split(",") if v.strip()])
    assert want.shape == (32,)
    from aien_sovereign_core_mv_b200.parts.rotary import inverse_frequencies
    scaling = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
    got = np.asarray(inverse_frequencies(64, 500000.0, scaling), dtype=np.float64)
    assert np.abs((got - want) / want).max() < 1e-12         # the reference's own bound (model_dir.rs:446)
    plain = np.asarray(pm.rope_inv_freq(64, 500000.0, scaling), dtype=np.float64)
    assert np.abs((plain - want) / want).max() < 1e-12
    unscaled = np.asarray(inverse_frequencies(64, 500000.0, None), dtype=np.float64)
    assert got[14] == unscaled[14] and got[31] == unscaled[31] / 32.0 and unscaled[16] / 32.0 < got[16] < unscaled[16]


# ------------------------------------------------------------------ GPU: the float32 engine
def _engine(model_dir, dtype="float32", **kw):
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    return Engine.from_folder(model_dir, EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=128, max_requests=4,
                                                     max_batch_tokens=64, **kw))


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_engine_float32_whole_token_by_token_and_prefill_then_decode(name):
    d, ids, want, argmax = fixture(name)
    eng = _engine(d)
    n = len(ids)
    whole = eng.step([(1, ids, [n - 1])]).cpu().numpy()[0]
    assert np.abs(whole - want).max() <= TOL
    if argmax is not None:
        assert int(whole.argmax()) == argmax
    for i, t in enumerate(ids):                              # one token a step
        last = eng.step([(2, [t], [0])])
    assert np.abs(last.cpu().numpy()[0] - want).max() <= TOL
    eng.step([(3, ids[:-1], [])])                            # all but the last id, then the last one decoded
    dec = eng.step([(3, ids[-1:], [0])]).cpu().numpy()[0]
    assert np.abs(dec - want).max() <= TOL
    eng.step([(4, ids[:2], [])])                             # portions of 2 + rest
    rest = eng.step([(4, ids[2:], [n - 3])]).cpu().numpy()[0]
    assert np.abs(rest - want).max() <= TOL
    eng.check_waits()


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_engine_bfloat16_stays_inside_the_reference_drift_bound(name):
    """The reference accepts max |dlogit| <= 0.15 of its reduced-precision path against the
    float32 oracle (crates/aien-inference-runtime/tests/drift/mod.rs:29)."""
    d, ids, want, argmax = fixture(name)
    got = _engine(d, "bfloat16").step([(1, ids, [len(ids) - 1])]).cpu().numpy()[0]
    assert np.abs(got - want).max() <= 0.15


@pytest.mark.gpu
def test_untied_head_uses_lm_head_not_the_embeddings(tmp_path):
    """The reference's construction (tests/qwen3_untied_head.rs:16-27): the tied fixture plus an
    lm_head.weight that is the embedding table with rows 3 and 5 swapped; the right logits are the
    oracle's with entries 3 and 5 swapped."""
    from aien_sovereign_core_mv_b200.weights.safetensors_io import CheckpointFiles, write_safetensors
    d, ids, tied, _ = fixture("qwen3-tiny")
    out = str(tmp_path / "untied")
    os.makedirs(out)
    raw = json.load(open(os.path.join(d, "config.json")))
    raw["tie_word_embeddings"] = False
    json.dump(raw, open(os.path.join(out, "config.json"), "w"))
    shutil.copy(os.path.join(d, "generation_config.json"), out)
    f = CheckpointFiles(d)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    head = tensors["model.embed_tokens.weight"].clone()
    head[[3, 5]] = head[[5, 3]]
    tensors["lm_head.weight"] = head
    write_safetensors(os.path.join(out, "model.safetensors"), tensors)
    want = tied.copy()
    want[[3, 5]] = want[[5, 3]]
    assert np.abs(want - tied).max() > 100 * TOL             # the control is not vacuous
    got = _engine(out).step([(1, ids, [len(ids) - 1])]).cpu().numpy()[0]
    assert np.abs(got - want).max() <= TOL and np.abs(got - tied).max() > 100 * TOL


@pytest.mark.gpu
def test_without_qk_norm_the_logits_are_far_from_the_reference():
    """Negative control (tests/qwen3_forward_parity.rs:171-188): the same weights run through a
    model whose mixers skip the per-head norm miss the oracle by far, so the parity above does
    exercise that norm."""
    from aien_sovereign_core_mv_b200 import Engine, EngineConfig
    from aien_sovereign_core_mv_b200.config.model_config import read_config_json, read_generation_config
    from aien_sovereign_core_mv_b200.config.spec import PartSpec
    from aien_sovereign_core_mv_b200.models.decoder import Decoder
    from aien_sovereign_core_mv_b200.models.loading import model_spec_for
    from aien_sovereign_core_mv_b200.weights.loader import iter_checkpoint
    d, ids, want, _ = fixture("qwen3-tiny")
    cfg, spec = model_spec_for(read_config_json(d), read_generation_config(d))
    layers = tuple(dataclasses.replace(l, mixer=PartSpec(l.mixer.kind, {**l.mixer.params, "qk_norm": False})) for l in spec.layers)
    model = Decoder(dataclasses.replace(spec, layers=layers))
    model.bind(iter_checkpoint(d, {n: s for n, (s, _) in model.catalog().items()}, "float32"))   # q_norm / k_norm stay unread
    eng = Engine(model, cfg, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=64, max_requests=2, max_batch_tokens=64))
    got = eng.step([(1, ids, [len(ids) - 1])]).cpu().numpy()[0]
    assert np.abs(got - want).max() > 100 * TOL
