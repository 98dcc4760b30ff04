"""A plain, slow restatement of the dense decoder: whole sequences, no cache, numpy only.

It rests on the reference's FORMULAS (the reference is Rust and cannot be compiled here);
each function cites the file:line it restates, paths relative to the reference project.
It shares no code with the engine: it has its own safetensors reader, its own config
handling and its own sampler.  Like the reference's CPU oracle it keeps float32 tensors
between operations and accumulates every reduction in float64
(crates/aien-inference-abi/src/tensor.rs:26-61).  It is anchored on the reference's own
transformers-float32 fixtures by ``tests/test_plain_model.py`` when they are mounted.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


# ------------------------------------------------------------------ files
def read_safetensors(path):
    """name -> float64 array (BF16/F32 widened exactly)."""
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    data = blob[8 + n:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        if meta["dtype"] == "BF16":
            u = np.frombuffer(data[b:e], dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32)
        elif meta["dtype"] == "F32":
            a = np.frombuffer(data[b:e], dtype="<f4")
        else:
            raise ValueError(f"plain reader: dtype {meta['dtype']} of {name}")
        out[name] = a.reshape(meta["shape"]).astype(np.float64)
    return out


def f32(x):
    """Round to float32 between operations, as the reference's tensors are f32."""
    return np.asarray(x, dtype=np.float64).astype(np.float32).astype(np.float64)


# ------------------------------------------------------------------ parts
def linear(x, w):
    """out = x . W^T, W row-major [out, in], f64 dot, f32 result (tensor.rs:26-61)."""
    return f32(x @ w.T)


def rms_norm(x, weight, eps):
    """x * (1/sqrt(mean(x^2)+eps)) * w; scale in f64 cast to f32, products in f32
    (tensor.rs:94-110).  Works on the last axis, so it also is the per-head q/k norm
    (tensor.rs:114-121)."""
    x = np.asarray(x, dtype=np.float64)
    scale = (1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + float(np.float32(eps)))).astype(np.float32)
    return ((x.astype(np.float32) * scale) * weight.astype(np.float32)).astype(np.float64)


def rope_inv_freq(head_dim, theta, scaling=None):
    """inv_freq_i = theta^(-2i/d) in f64, with optional llama3 smoothing
    (crates/aien-abi-core/src/lib.rs:106-114, 69-84).  theta is held as f32 there."""
    theta = float(np.float32(theta))
    inv = np.array([1.0 / theta ** ((2 * i) / head_dim) for i in range(head_dim // 2)], dtype=np.float64)
    if scaling is None:
        return inv
    old = float(scaling["original_max_position_embeddings"])
    low_w = old / scaling["low_freq_factor"]
    high_w = old / scaling["high_freq_factor"]
    out = inv.copy()
    for i, f in enumerate(inv):
        wavelen = 2.0 * math.pi / f
        if wavelen < high_w:
            out[i] = f
        elif wavelen > low_w:
            out[i] = f / scaling["factor"]
        else:
            smooth = (old / wavelen - scaling["low_freq_factor"]) / (scaling["high_freq_factor"] - scaling["low_freq_factor"])
            out[i] = (1.0 - smooth) * f / scaling["factor"] + smooth * f
    return out


def apply_rope(v, positions, inv_freq):
    """rotate_half pairing (i, i+d/2); angle = pos*inv_freq in f64, cos/sin cast to f32,
    rotation in f32 (tensor.rs:150-188).  v: [T, heads, d]."""
    d = v.shape[-1]
    ang = np.asarray(positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    cos = np.cos(ang).astype(np.float32)[:, None, :]
    sin = np.sin(ang).astype(np.float32)[:, None, :]
    a = v[..., : d // 2].astype(np.float32)
    b = v[..., d // 2:].astype(np.float32)
    return np.concatenate([a * cos - b * sin, a * sin + b * cos], axis=-1).astype(np.float64)


def attention(q, k, v, positions, window=None, scale=None):
    """Causal grouped-query attention over whole sequences: score (q.k)/sqrt(d), softmax with
    max subtraction, out = sum p v, all in f64 (crates/aien-inference-abi/src/backend.rs:581-646,
    280-306).  q [T,nq,d], k/v [T,nkv,d]; query head h uses kv head h // (nq/nkv).
    ``window`` (not in the reference, which refuses windows; used for the engine's generic
    windowed mixer): key j is seen by query i iff 0 <= pos_i - pos_j < window."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    pos = np.asarray(positions)
    delta = pos[:, None] - pos[None, :]
    mask = delta >= 0
    if window is not None:
        mask &= delta < window
    out = np.zeros((T, nq, d))
    for h in range(nq):
        s = (q[:, h] @ k[:, h // g].T) * scale
        s = np.where(mask, s, -np.inf)
        s = np.exp(s - s.max(-1, keepdims=True))
        s /= s.sum(-1, keepdims=True)
        out[:, h] = s @ v[:, h // g]
    return f32(out)


def swiglu(gate, up):
    """silu(g)*u with silu(g)=g/(1+exp(-g)) in f64, f32 result (backend.rs:572-579)."""
    return f32(gate / (1.0 + np.exp(-gate)) * up)


def round_bf16(x):
    """Round-to-nearest-even to bfloat16 (crates/aien-kv-cache/src/lib.rs:116-126)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(x))


# ------------------------------------------------------------------ whole model
def decoder_forward(config, weights, ids, kv_round=None, return_hidden=False):
    """Logits [T, vocab] for one whole sequence (pre-norm blocks: x -> norm -> attn -> +x ->
    norm -> mlp -> +x; crates/aien-inference-abi/src/weights.rs:290-365, 389-643).
    ``config`` is the parsed config.json.  ``kv_round`` (e.g. round_bf16) is applied to k and
    v "at birth" as the cache would (transformer_backend.rs:1253-1270)."""
    H = config["hidden_size"]
    nq = config["num_attention_heads"]
    nkv = config.get("num_key_value_heads") or nq
    hd = config.get("head_dim") or H // nq
    eps = config["rms_norm_eps"]
    theta = config.get("rope_theta", 10000.0)
    scaling = config.get("rope_scaling")
    if scaling is not None and scaling.get("rope_type", scaling.get("type", "default")) == "default":
        scaling = None
    qk_norm = config["architectures"][0] == "Qwen3ForCausalLM"
    ids = np.asarray(ids, dtype=np.int64)
    T = len(ids)
    positions = np.arange(T)
    inv_freq = rope_inv_freq(hd, theta, scaling)

    x = weights["model.embed_tokens.weight"][ids]          # weights.rs:140-146
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = rms_norm(x, weights[p + "input_layernorm.weight"], eps)
        q = linear(h, weights[p + "self_attn.q_proj.weight"]).reshape(T, nq, hd)
        k = linear(h, weights[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd)
        v = linear(h, weights[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
        if qk_norm:                                          # before rope (transformer_backend.rs:1241)
            q = rms_norm(q, weights[p + "self_attn.q_norm.weight"], eps)
            k = rms_norm(k, weights[p + "self_attn.k_norm.weight"], eps)
        q = apply_rope(q, positions, inv_freq)
        k = apply_rope(k, positions, inv_freq)
        if kv_round is not None:
            k, v = kv_round(k), kv_round(v)
        o = attention(q, k, v, positions).reshape(T, nq * hd)
        x = f32(x + linear(o, weights[p + "self_attn.o_proj.weight"]))
        h = rms_norm(x, weights[p + "post_attention_layernorm.weight"], eps)
        a = swiglu(linear(h, weights[p + "mlp.gate_proj.weight"]), linear(h, weights[p + "mlp.up_proj.weight"]))
        x = f32(x + linear(a, weights[p + "mlp.down_proj.weight"]))
    xn = rms_norm(x, weights["model.norm.weight"], eps)
    head = weights["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else weights["lm_head.weight"]
    logits = linear(xn, head)                                # weights.rs:131-136
    return (logits, x) if return_hidden else logits


def load_model_folder(model_dir):
    with open(f"{model_dir}/config.json") as f:
        config = json.load(f)
    return config, read_safetensors(f"{model_dir}/model.safetensors")


# ------------------------------------------------------------------ sampling
def argmax_token(logits):
    """First maximum wins (tensor.rs:299-318)."""
    best, best_v = 0, logits[0]
    for i in range(1, len(logits)):
        if logits[i] > best_v:
            best, best_v = i, logits[i]
    return best


def kept_set(logits, temperature, top_p=1.0, top_k=0):
    """The tokens a draw may choose and their probabilities: top-k mask (k largest logits, ties
    to the lower id; crates/aien-inference-abi/src/qwen3_moe_omega.rs:3246-3272), f64 softmax of
    l/T with max subtraction, then the smallest prefix by probability (ties to the lower id)
    whose mass reaches top_p (transformer_backend.rs:122-172).  Returns (ids sorted ascending,
    probs over the full vocabulary)."""
    logits = np.asarray(logits, dtype=np.float64)
    V = len(logits)
    allowed = np.ones(V, dtype=bool)
    if top_k and 0 < top_k < V:
        order = sorted(range(V), key=lambda i: (-logits[i], i))
        allowed[:] = False
        allowed[order[:top_k]] = True
    mx = logits[allowed].max()
    probs = np.where(allowed, np.exp((logits - mx) / temperature), 0.0)
    probs /= probs.sum()
    kept = [i for i in range(V) if allowed[i]]
    if 0.0 < top_p < 1.0:
        order = sorted(kept, key=lambda i: (-probs[i], i))
        cum, keep = 0.0, 0
        for i in order:
            cum += probs[i]
            keep += 1
            if cum >= top_p:
                break
        kept = sorted(order[:keep])
    return kept, probs


def sample_token(logits, temperature, top_p, top_k, u):
    """temperature <= 0.001 is greedy (transformer_backend.rs:110-118).  Otherwise one uniform
    ``u`` in [0,1) scaled to the kept mass picks a token by walking the kept set; this engine
    walks it in token-id order (the reference walks in probability order after a nucleus cut,
    transformer_backend.rs:158-172; the distribution is the same)."""
    if temperature <= 0.001:
        return argmax_token(logits)
    kept, probs = kept_set(logits, temperature, top_p, top_k)
    mass = sum(probs[i] for i in kept)
    r = u * mass
    cum = 0.0
    for i in kept:
        cum += probs[i]
        if r < cum:
            return i
    return kept[-1]
