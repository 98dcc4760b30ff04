"""Writes ``plain_tiny_logits.json``: last-row logits of the plain implementation
(``tests/plain_model.py``) on two tiny random models.

The plain implementation rests on the reference's formulas: the reference is a Rust
workspace and neither cargo nor rustc exists here, so its model code cannot be compiled or
imported for a direct comparison.  Its anchor is the pair of transformers-float32 fixtures the
reference ships (``tests/test_plain_model.py::test_fixture_logits``).  This file only pins
the plain implementation against silent change.

    python tests/golden/make_golden.py      # rewrites the JSON beside this script

The tiny models are built here with numpy alone (no engine code): values from
``numpy.random.default_rng(seed)`` rounded to bfloat16.
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import plain_model as pm  # noqa: E402

TINY = {
    "A": dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=160, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256,
              hidden_act="silu", eos_token_id=2),
    "B": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=8, num_key_value_heads=2, head_dim=32, intermediate_size=288, vocab_size=512,
              rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512,
              hidden_act="silu", eos_token_id=[1, 2]),
}


def tiny_model(which, seed=None):
    config = dict(TINY[which])
    rng = np.random.default_rng({"A": 0, "B": 1}[which] if seed is None else seed)
    H, nq, nkv, hd = config["hidden_size"], config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    I, V = config["intermediate_size"], config["vocab_size"]
    w = {}
    mat = lambda o, i: pm.round_bf16(rng.standard_normal((o, i)) / np.sqrt(i))
    norm = lambda n: pm.round_bf16(rng.uniform(0.8, 1.2, n))
    w["model.embed_tokens.weight"] = pm.round_bf16(rng.standard_normal((V, H)))
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = norm(H)
        w[p + "self_attn.q_proj.weight"] = mat(nq * hd, H)
        w[p + "self_attn.k_proj.weight"] = mat(nkv * hd, H)
        w[p + "self_attn.v_proj.weight"] = mat(nkv * hd, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, nq * hd)
        if config["architectures"][0] == "Qwen3ForCausalLM":
            w[p + "self_attn.q_norm.weight"] = norm(hd)
            w[p + "self_attn.k_norm.weight"] = norm(hd)
        w[p + "post_attention_layernorm.weight"] = norm(H)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
    w["model.norm.weight"] = norm(H)
    if not config["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(V, H)
    return config, w


def compute():
    out = {}
    for which, n in (("A", 29), ("B", 40)):
        config, w = tiny_model(which)
        ids = np.random.default_rng(100 + n).integers(0, config["vocab_size"], n)
        logits = pm.decoder_forward(config, w, ids)
        out[which] = [[float(v) for v in logits[-1][:32]], [float(v) for v in logits[n // 2][:32]]]
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain_tiny_logits.json")
    with open(path, "w") as f:
        json.dump(compute(), f)
    print("wrote", path)
