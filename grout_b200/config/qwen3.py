"""Configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

Field names are config.json's.  The reference has two readers of this file: a
strict one with thirteen required keys and no defaults (src/config.rs:6-21) and
a newer one that takes the rotation's constants from the ``rope_parameters``
object when the file has one, refuses every ``rope_type`` but ``default``, and
checks ``layer_types`` against the number of layers
(src/quantized_config.rs:66-83, 119-125).  This class reads both forms and
never guesses a constant of the arithmetic: the rotation base must stand in the
file (at the top level or in ``rope_parameters``; the two must agree when both
are there), the per-layer windows come from ``layer_types`` or from
``use_sliding_window`` / ``max_window_layers`` (and must agree when both are
there), and a key that stands for a term this architecture does not have
(``changes_arithmetic``) is refused unless it is switched off.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .base import ModelConfig

_LAYER_KINDS = ("full_attention", "sliding_attention")


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
    rope_theta: Optional[float] = None        # here or in rope_parameters, never guessed
    rope_parameters: Optional[dict] = None
    tie_word_embeddings: bool = False
    use_sliding_window: Optional[bool] = None
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[Tuple[str, ...]] = None
    eos_token_id: Union[int, Tuple[int, ...], None] = None
    bos_token_id: Optional[int] = None
    hidden_act: str = "silu"
    attention_bias: bool = False
    rope_scaling: Optional[dict] = None
    model_type: str = "qwen3"
    architectures: Tuple[str, ...] = ("Qwen3ForCausalLM",)
    torch_dtype: Optional[str] = None

    # Terms that other decoders have and this one has not.  Present with a value
    # that switches the term on, such a key means the checkpoint was trained
    # with arithmetic that the parts named by the plan do not do.
    changes_arithmetic = {
        "partial_rotary_factor": (None, 1.0),
        "mlp_bias": (None, False),
        "use_qk_norm": (None, True),
        "attn_logit_softcapping": (None,),
        "final_logit_softcapping": (None,),
        "query_pre_attn_scalar": (None,),
        "attention_multiplier": (None, 1.0),
        "embedding_multiplier": (None, 1.0),
        "residual_multiplier": (None, 1.0),
        "logits_scaling": (None, 1.0),
        "logit_scale": (None, 1.0),
        "attn_output_gate": (None, False),
        "num_experts": (None, 0),
        "num_local_experts": (None, 0),
        "moe_intermediate_size": (None,),
        "mlp_only_layers": (None,),
        "quantization_config": (None,),
    }

    def resolved(self):
        cfg = self
        if cfg.head_dim is None and cfg.num_attention_heads > 0:
            cfg = cfg.replace(head_dim=cfg.hidden_size // cfg.num_attention_heads)
        # src/quantized_config.rs:66-83: the rotation's constants are read from
        # rope_parameters when it is an object, else from the top level.
        if cfg.rope_theta is None and isinstance(cfg.rope_parameters, dict):
            inner = cfg.rope_parameters.get("rope_theta")
            if isinstance(inner, (int, float)) and not isinstance(inner, bool):
                cfg = cfg.replace(rope_theta=float(inner))
        return cfg

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
        yield from self._rotation_problems()
        if self.hidden_act != "silu":
            yield f"hidden_act='{self.hidden_act}': only 'silu' is defined for this architecture"
        if self.attention_bias:
            # src/quantized_config.rs:113-118
            yield "attention_bias=true is not part of this architecture"
        if self.rope_scaling is not None:
            kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type", "default"))
            if kind != "default":  # src/quantized_config.rs:68-78
                yield f"rope_scaling of type '{kind}' is not supported"
        yield from self._window_problems()

    def _rotation_problems(self):
        rp = self.rope_parameters
        if rp is not None:
            if any(isinstance(v, dict) for v in rp.values()):
                yield "'rope_parameters' per layer type is not part of this architecture"
                return
            kind = rp.get("rope_type", rp.get("type", "default"))
            if kind != "default":  # src/quantized_config.rs:71-75
                yield f"rope_parameters of rope_type '{kind}' is not supported"
            factor = rp.get("partial_rotary_factor")
            if factor is not None and factor != 1:
                yield f"rope_parameters.partial_rotary_factor={factor!r} is not supported"
            inner = rp.get("rope_theta")
            if inner is not None and (isinstance(inner, bool) or not isinstance(inner, (int, float))):
                yield f"rope_parameters.rope_theta should be a number, found {inner!r}"
            elif inner is not None and self.rope_theta is not None and float(inner) != self.rope_theta:
                yield (f"rope_theta={self.rope_theta} at the top level disagrees with "
                       f"rope_parameters.rope_theta={inner}")
        if self.rope_theta is None:  # src/config.rs:16: required, no default
            yield "required key 'rope_theta' is missing (at the top level and in 'rope_parameters')"
        elif not (self.rope_theta > 0 and self.rope_theta != float("inf")):
            yield f"rope_theta={self.rope_theta} must be positive and finite"

    def _windows_from_flags(self):
        """Per-layer kinds as use_sliding_window / max_window_layers give them, or
        None when those keys do not settle it."""
        if self.use_sliding_window is None:
            return None
        if not self.use_sliding_window:
            return ("full_attention",) * self.num_hidden_layers
        if self.max_window_layers is None:
            return None
        return tuple("sliding_attention" if i >= self.max_window_layers else "full_attention"
                     for i in range(self.num_hidden_layers))

    def _window_problems(self):
        if self.max_window_layers is not None and self.max_window_layers < 0:
            yield "'max_window_layers' must not be negative"
        from_flags = self._windows_from_flags()
        kinds = self.layer_types
        if kinds is not None:
            if len(kinds) != self.num_hidden_layers:  # src/quantized_config.rs:119-125
                yield (f"'layer_types' has {len(kinds)} entries for "
                       f"num_hidden_layers={self.num_hidden_layers}")
                return
            unknown = sorted(set(kinds) - set(_LAYER_KINDS))
            if unknown:
                yield f"'layer_types' names {unknown}; this architecture has {list(_LAYER_KINDS)}"
                return
            if from_flags is not None and from_flags != tuple(kinds):
                yield ("'layer_types' disagrees with use_sliding_window="
                       f"{self.use_sliding_window!r} / max_window_layers={self.max_window_layers!r}")
        elif self.use_sliding_window and from_flags is None:
            yield "use_sliding_window=true needs 'max_window_layers' or 'layer_types'"
        windowed = "sliding_attention" in (kinds if kinds is not None else from_flags or ())
        if (windowed or self.use_sliding_window) and \
                (self.sliding_window is None or self.sliding_window <= 0):
            yield "a layer with a sliding window needs a positive 'sliding_window'"

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
        """None for a layer that sees every earlier key, else the number of keys
        it sees.  ``layer_types`` names the kind of every layer; without it the
        first ``max_window_layers`` layers see everything and, with
        ``use_sliding_window``, the others the last ``sliding_window`` keys.  (The
        reference refuses windowed layers, src/model.rs:1323-1326,
        src/quantized_config.rs:126-131.)"""
        kinds = self.layer_types if self.layer_types is not None else self._windows_from_flags()
        if kinds is None or kinds[layer] == "full_attention":
            return None
        return self.sliding_window
