"""The dense Llama decoder (the reference's models/src/llama.rs) as a model spec.

Every layer is a pre-norm block of grouped-query attention with rotary positions
and a SwiGLU feed-forward; all sizes and constants come from the typed
configuration.  Tensor names are the checkpoint's own (models/src/llama.rs:322-325,
372-374, 414-421, 481-489).
"""
from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.model import LayerSpec, ModelSpec


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    norm = {"kind": "rmsnorm", "size": cfg.hidden_size, "eps": cfg.rms_norm_eps}
    mixer = {
        "kind": "attention", "hidden": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "scale": cfg.softmax_scale,
        "window": None,
        "position": {"kind": "rope", "head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                     "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None},
    }
    ff = {"kind": "swiglu", "hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size}
    block = {"kind": "prenorm", "norm": norm, "mixer": mixer, "feed_forward": ff}
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=[LayerSpec(f"model.layers.{i}", block) for i in range(cfg.num_hidden_layers)],
        final_norm=norm,
        head_tensor=None if cfg.tie_word_embeddings else "lm_head.weight",
        # a tied checkpoint may still store the head; rotary buffers are recomputed
        ignored_tensors=(("lm_head.weight",) if cfg.tie_word_embeddings else ()) + ("*.rotary_emb.inv_freq",),
        max_position=cfg.max_position_embeddings,
        eos_token_ids=cfg.eos_token_ids,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec, model_type="llama")
