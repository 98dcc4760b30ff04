"""Architecture builders for the dense decoder family: ``LlamaForCausalLM`` and
``Qwen3ForCausalLM``.

Both give the same kind of model: pre-norm blocks of RMSNorm, grouped-query attention with
rotary positions, SwiGLU; Qwen3 adds the per-head RMSNorm of q and k and lets ``head_dim`` differ
from ``hidden_size / heads``.  This file is the only place that knows the tensor names of the
checkpoints (crates/aien-inference-abi/src/weights.rs:811-865, src/checkpoint.rs:262-319).
"""
from __future__ import annotations

from dataclasses import asdict

from ..config.model_config import DenseDecoderConfig, config_from_hf_dict
from ..config.spec import LayerSpec, ModelSpec, PartSpec, default_run_list
from ..registry import register_architecture

_NAMES = {
    "norm_in.weight": "input_layernorm.weight",
    "norm_post.weight": "post_attention_layernorm.weight",
    "mixer.q_proj": "self_attn.q_proj.weight",
    "mixer.k_proj": "self_attn.k_proj.weight",
    "mixer.v_proj": "self_attn.v_proj.weight",
    "mixer.o_proj": "self_attn.o_proj.weight",
    "mixer.q_norm": "self_attn.q_norm.weight",
    "mixer.k_norm": "self_attn.k_norm.weight",
    "feed_forward.gate_proj": "mlp.gate_proj.weight",
    "feed_forward.up_proj": "mlp.up_proj.weight",
    "feed_forward.down_proj": "mlp.down_proj.weight",
}


def spec_from_config(cfg: DenseDecoderConfig) -> ModelSpec:
    position = PartSpec("rotary", {
        "head_dim": cfg.head_dim, "theta": cfg.rope_theta,
        "scaling": asdict(cfg.rope_scaling) if cfg.rope_scaling is not None else None,
    })
    mixer = PartSpec("paged_attention", {
        "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
        "qk_norm": cfg.qk_norm, "qk_norm_eps": cfg.rms_norm_eps, "window": 0,
    })
    ff = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    norm = PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps})
    layers = tuple(
        LayerSpec(block="prenorm", mixer=mixer, feed_forward=ff, norm=None, norms={"norm_in": norm, "norm_post": norm},
                  position=position, prefix=f"model.layers.{i}.", names=_NAMES)
        for i in range(cfg.num_hidden_layers)
    )
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        layers=layers, run_list=default_run_list(cfg.num_hidden_layers),
        embedding=PartSpec("table", {"name": "model.embed_tokens.weight"}),
        final_norm=PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps, "name": "model.norm.weight"}),
        head=PartSpec("linear", {"name": "lm_head.weight", "tied": cfg.tie_word_embeddings}),
        max_position=cfg.max_position_embeddings, stop_token_ids=tuple(cfg.eos_token_ids),
    )


def _build(raw, generation_config=None, strict=False):
    cfg = config_from_hf_dict(raw, generation_config, strict)
    return cfg, spec_from_config(cfg)


register_architecture("LlamaForCausalLM")(_build)
register_architecture("Qwen3ForCausalLM")(_build)
