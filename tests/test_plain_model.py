"""The plain implementation against the reference's own transformers-float32 fixtures, and
against itself on properties it must have (causality, position handling)."""
import json
import os

import numpy as np
import pytest

import plain_model as pm

# the reference project, when it is checked out beside this repository (or named by AIEN_REFERENCE_DIR)
_REF = os.environ.get("AIEN_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
FIX = os.path.join(_REF, "crates", "aien-inference-abi", "fixtures")


@pytest.mark.parametrize("name", ["qwen3-tiny", "openwaldo-byte"])
def test_fixture_logits(name):
    d = os.path.join(FIX, name)
    if not os.path.isdir(d):
        pytest.skip("reference fixtures are not mounted")
    config, weights = pm.load_model_folder(d)
    ref = json.load(open(os.path.join(d, "forward_reference.json")))
    logits = pm.decoder_forward(config, weights, ref["ids"])[-1]
    want = np.array(ref["logits"])
    assert np.abs(logits - want).max() <= 1e-4      # the reference's own bound (qwen3_forward_parity.rs:46)
    if "argmax" in ref:
        assert pm.argmax_token(logits) == ref["argmax"]


def test_golden_outputs_match():
    """The committed small outputs of the plain implementation still reproduce."""
    import golden.make_golden as mg
    path = os.path.join(os.path.dirname(__file__), "golden", "plain_tiny_logits.json")
    want = json.load(open(path))
    got = mg.compute()
    for key, rows in want.items():
        assert np.abs(np.array(got[key]) - np.array(rows)).max() <= 1e-6, key


def test_causality_and_prefix():
    import golden.make_golden as mg
    config, weights = mg.tiny_model("B")
    ids = [3, 7, 1, 50, 9, 12, 44]
    full = pm.decoder_forward(config, weights, ids)
    part = pm.decoder_forward(config, weights, ids[:4])
    assert np.abs(full[:4] - part).max() <= 1e-6


def test_rope_depends_on_relative_position_only():
    rng = np.random.default_rng(0)
    inv = pm.rope_inv_freq(16, 10000.0)
    q = rng.standard_normal((1, 1, 16)); k = rng.standard_normal((1, 1, 16))
    def score(pq, pk):
        return float((pm.apply_rope(q, [pq], inv)[0, 0] * pm.apply_rope(k, [pk], inv)[0, 0]).sum())
    assert abs(score(5, 2) - score(105, 102)) < 1e-4


def test_llama3_scaling_bands():
    s = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
    plain = pm.rope_inv_freq(128, 500000.0)
    scaled = pm.rope_inv_freq(128, 500000.0, s)
    assert scaled[0] == plain[0]                       # short wavelengths kept
    assert abs(scaled[-1] - plain[-1] / 8.0) < 1e-18   # long ones divided by factor
    assert np.all(scaled <= plain + 1e-18)


def test_sampler_rules():
    logits = np.array([0.5, 2.0, 2.0, -1.0, 1.5])
    assert pm.argmax_token(logits) == 1                          # first maximum wins
    assert pm.sample_token(logits, 0.0005, 0.9, 0, 0.99) == 1    # greedy threshold
    kept, probs = pm.kept_set(logits, 1.0, top_p=0.5)
    assert kept == [1, 2]                                        # ties to the lower id, prefix reaches 0.5
    kept, _ = pm.kept_set(logits, 1.0, top_k=1)
    assert kept == [1]
    picks = {pm.sample_token(logits, 1.0, 1.0, 0, u) for u in np.linspace(0, 0.999, 50)}
    assert picks == {0, 1, 2, 3, 4}


def test_round_bf16():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.3], dtype=np.float32)
    import torch
    want = torch.tensor(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(pm.round_bf16(x).astype(np.float32), want)
