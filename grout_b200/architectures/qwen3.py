"""Qwen3 dense decoder (``Qwen3ForCausalLM``, model_type "qwen3") as a plan.

Everything here is read from the configuration: this file holds the tensor
names of the checkpoint (src/model.rs:1372-1447, name builder 6005-6016) and the
order of the parts (src/training.rs:255-363), no sizes.
"""
from __future__ import annotations

from ..config import Qwen3Config, register_architecture
from ..parts.base import PartSpec
from ..parts.plan import LayerPlan, ModelPlan, ScheduleEntry


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    H, D = cfg.hidden_size, cfg.head_dim
    position = PartSpec("rotary_half_split", dict(head_dim=D, theta=cfg.rope_theta))
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec("gqa_attention", dict(
            hidden=H, n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
            head_dim=D, position=position, qk_norm_eps=cfg.rms_norm_eps,
            window=cfg.window_of_layer(i)))
        norm = PartSpec("rmsnorm", dict(dim=H, eps=cfg.rms_norm_eps))
        block = PartSpec("prenorm", dict(
            norm1=norm, mixer=mixer, norm2=norm,
            feedforward=PartSpec("swiglu", dict(hidden=H, intermediate=cfg.intermediate_size))))
        layers.append(LayerPlan(block, f"model.layers.{i}.", {
            "norm1": "input_layernorm.", "mixer": "self_attn.",
            "norm2": "post_attention_layernorm.", "feedforward": "mlp."}))
    return ModelPlan(
        embedding=PartSpec("token", dict(vocab=cfg.vocab_size, hidden=H)),
        embedding_prefix="model.embed_tokens.",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", dict(dim=H, eps=cfg.rms_norm_eps)),
        final_norm_prefix="model.norm.",
        head=PartSpec("linear", dict(vocab=cfg.vocab_size, hidden=H, tied=cfg.tie_word_embeddings)),
        head_prefix="lm_head.",
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        stop_tokens=cfg.eos_token_ids(),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_plan, model_types=("qwen3",))
