"""Configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

Field names are config.json's.  The reference requires thirteen keys and has no
defaults (src/config.rs:6-21); the keys that it demands but that many
checkpoints derive are defaulted here the way its packed-model parser does
(src/quantized_config.rs:79-82 rope_theta, 18-19 tie_word_embeddings).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .base import ModelConfig


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    max_position_embeddings: int
    head_dim: Optional[int] = None            # decoupled from hidden_size / heads
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    eos_token_id: Union[int, Tuple[int, ...], None] = None
    bos_token_id: Optional[int] = None
    hidden_act: str = "silu"
    attention_bias: bool = False
    rope_scaling: Optional[dict] = None
    model_type: str = "qwen3"
    architectures: Tuple[str, ...] = ("Qwen3ForCausalLM",)
    torch_dtype: Optional[str] = None

    def resolved(self):
        if self.head_dim is None:
            if self.num_attention_heads > 0:
                return self.replace(head_dim=self.hidden_size // self.num_attention_heads)
        return self

    def validate(self):
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
                    "head_dim"):
            v = getattr(self, key)
            if v is None or v <= 0:
                yield f"'{key}' must be a positive integer, found {v!r}"
                return
        # src/training.rs:184-191: even head_dim, heads divisible into groups
        if self.num_attention_heads % self.num_key_value_heads:
            yield (f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                   f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            yield f"head_dim={self.head_dim} must be even for the half-split rotation"
        if not self.rms_norm_eps > 0:
            yield f"rms_norm_eps={self.rms_norm_eps} must be positive"
        if not self.rope_theta > 0:
            yield f"rope_theta={self.rope_theta} must be positive"
        if self.hidden_act != "silu":
            yield f"hidden_act='{self.hidden_act}': only 'silu' is defined for this architecture"
        if self.attention_bias:
            # src/quantized_config.rs:113-118
            yield "attention_bias=true is not part of this architecture"
        if self.rope_scaling is not None:
            kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type", "default"))
            if kind != "default":  # src/quantized_config.rs:68-78
                yield f"rope_scaling of type '{kind}' is not supported"
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                yield "use_sliding_window=true needs a positive 'sliding_window'"
            if self.max_window_layers is not None and self.max_window_layers < 0:
                yield "'max_window_layers' must not be negative"

    # ---- derived -------------------------------------------------------
    @property
    def num_kv_groups(self) -> int:
        """src/config.rs:35-38"""
        return self.num_attention_heads // self.num_key_value_heads

    def eos_token_ids(self) -> Tuple[int, ...]:
        if self.eos_token_id is None:
            return ()
        if isinstance(self.eos_token_id, int):
            return (self.eos_token_id,)
        return tuple(self.eos_token_id)

    def window_of_layer(self, layer: int) -> Optional[int]:
        """None for a layer that sees every earlier key.  With use_sliding_window
        the first ``max_window_layers`` layers see everything and the others the
        last ``sliding_window`` keys.  (The reference refuses such a config,
        src/model.rs:1323-1326.)"""
        if not self.use_sliding_window:
            return None
        first_windowed = self.num_hidden_layers if self.max_window_layers is None \
            else self.max_window_layers
        return None if layer < first_windowed else self.sliding_window
