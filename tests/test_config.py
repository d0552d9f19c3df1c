"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY
from grout_b200 import architectures  # noqa: F401
from grout_b200.config import (ConfigError, GenerationConfig, Qwen3Config, known_architectures,
                               load_config, register_architecture, resolve_architecture,
                               unregister_architecture)
from grout_b200.config.base import ModelConfig


def test_reads_every_key_of_config_json():
    for name, raw in TINY.items():
        cfg = Qwen3Config.from_dict(raw)
        for k, v in raw.items():
            got = getattr(cfg, k)
            assert (list(got) if isinstance(got, tuple) else got) == v, (name, k)
        assert cfg.num_kv_groups == raw["num_attention_heads"] // raw["num_key_value_heads"]


def test_defaults_and_derived_values():
    raw = {k: v for k, v in TINY["A"].items() if k not in ("head_dim", "rms_norm_eps",
                                                          "tie_word_embeddings", "eos_token_id")}
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    assert cfg.rms_norm_eps == 1e-6 and cfg.tie_word_embeddings is False
    assert cfg.eos_token_ids() == ()
    assert Qwen3Config.from_dict(TINY["B"]).eos_token_ids() == (7, 383)
    assert Qwen3Config.from_dict(dict(TINY["A"], rope_theta=10000)).rope_theta == 10000.0


def test_all_problems_are_reported_at_once():
    raw = dict(TINY["A"])
    del raw["vocab_size"]
    raw["hidden_size"] = "64"
    raw["tie_word_embeddings"] = 1
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    msg = str(e.value)
    assert "vocab_size" in msg and "hidden_size" in msg and "tie_word_embeddings" in msg


@pytest.mark.parametrize("change,word", [
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(hidden_act="gelu"), "silu"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope_scaling"),
    (dict(use_sliding_window=True), "sliding_window"),
    (dict(use_sliding_window=True, sliding_window=8), "max_window_layers"),
    (dict(rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0}), "yarn"),
    (dict(rope_parameters={"rope_theta": 5e6}), "disagrees"),
    (dict(rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.5}), "partial"),
    (dict(rope_parameters={"full_attention": {"rope_theta": 10000.0}}), "per layer type"),
    (dict(layer_types=["full_attention"]), "entries"),
    (dict(layer_types=["full_attention", "linear_attention"]), "linear_attention"),
    (dict(layer_types=["full_attention", "sliding_attention"]), "disagrees"),
    (dict(layer_types=["full_attention", "sliding_attention"], use_sliding_window=True,
          max_window_layers=1), "positive 'sliding_window'"),
    (dict(partial_rotary_factor=0.25), "partial_rotary_factor"),
    (dict(mlp_bias=True), "mlp_bias"),
    (dict(attn_logit_softcapping=50.0), "attn_logit_softcapping"),
    (dict(use_qk_norm=False), "use_qk_norm"),
    (dict(num_experts=8), "num_experts"),
    (dict(num_hidden_layers=0), "positive"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
])
def test_refuses_what_the_architecture_does_not_define(change, word):
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(dict(TINY["A"], **change))
    assert word in str(e.value)


def test_the_rotation_base_is_never_guessed():
    raw = {k: v for k, v in TINY["A"].items() if k != "rope_theta"}
    with pytest.raises(ConfigError) as e:           # src/config.rs:16: required
        Qwen3Config.from_dict(raw)
    assert "rope_theta" in str(e.value)
    # the form that newer writers of this file use (src/quantized_config.rs:66-83)
    cfg = Qwen3Config.from_dict(dict(raw, rope_parameters={"rope_type": "default",
                                                           "rope_theta": 250000}))
    assert cfg.rope_theta == 250000.0
    both = Qwen3Config.from_dict(dict(TINY["A"], rope_parameters={"rope_theta": 10000.0}))
    assert both.rope_theta == 10000.0


def test_a_file_in_the_newer_form_is_read_or_refused_never_misread():
    """rope_parameters of another type together with a windowed layer_types once
    loaded and ran with a guessed base, no scaling and no window."""
    raw = {k: v for k, v in TINY["A"].items() if k not in ("rope_theta", "use_sliding_window")}
    raw.update(rope_parameters={"rope_type": "yarn", "rope_theta": 5e6, "factor": 2.0},
               layer_types=["full_attention", "sliding_attention"])
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    assert "yarn" in str(e.value) and "sliding_window" in str(e.value)
    raw.update(rope_parameters={"rope_type": "default", "rope_theta": 5e6}, sliding_window=24)
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.rope_theta == 5e6
    assert [cfg.window_of_layer(i) for i in range(2)] == [None, 24]


def test_neutral_values_of_foreign_terms_are_accepted():
    cfg = Qwen3Config.from_dict(dict(TINY["A"], mlp_bias=False, attn_logit_softcapping=None,
                                     partial_rotary_factor=1.0, num_experts=0, use_qk_norm=True))
    assert cfg.extra["mlp_bias"] is False


def test_window_per_layer():
    cfg = Qwen3Config.from_dict(TINY["C"])
    assert [cfg.window_of_layer(i) for i in range(4)] == [None, 40, 40, 40]
    assert Qwen3Config.from_dict(TINY["A"]).window_of_layer(1) is None
    kinds = ["sliding_attention", "full_attention", "sliding_attention", "full_attention"]
    raw = {k: v for k, v in TINY["C"].items() if k not in ("use_sliding_window", "max_window_layers")}
    cfg = Qwen3Config.from_dict(dict(raw, layer_types=kinds))
    assert [cfg.window_of_layer(i) for i in range(4)] == [40, None, 40, None]
    agree = dict(TINY["C"], layer_types=["full_attention"] + ["sliding_attention"] * 3)
    assert [Qwen3Config.from_dict(agree).window_of_layer(i) for i in range(4)] == [None, 40, 40, 40]


def test_unknown_keys_survive_a_round_trip():
    raw = dict(TINY["A"], some_future_key=[1, 2])
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.extra["some_future_key"] == [1, 2]
    assert cfg.to_dict()["some_future_key"] == [1, 2]
    assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


def test_registry_resolves_by_architecture_then_model_type(tmp_path):
    assert "Qwen3ForCausalLM" in known_architectures()
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).config_cls is Qwen3Config
    assert resolve_architecture({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError) as e:
        resolve_architecture({"architectures": ["NopeForCausalLM"], "model_type": "nope"})
    assert "Qwen3ForCausalLM" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"]))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Qwen3ForCausalLM" and cfg.hidden_size == 96
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "missing"))


def test_registering_another_architecture_needs_no_change_elsewhere():
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class OtherConfig(ModelConfig):
        width: int
        depth: int = 1

    register_architecture("OtherForCausalLM", OtherConfig, lambda c: ("plan", c.width),
                          model_types=("other",))
    try:
        arch = resolve_architecture({"model_type": "other"})
        cfg = arch.config_cls.from_dict({"width": 8})
        assert arch.plan(cfg) == ("plan", 8) and cfg.depth == 1
    finally:
        unregister_architecture("OtherForCausalLM")
    assert "OtherForCausalLM" not in known_architectures()


def test_generation_config(tmp_path):
    assert GenerationConfig.from_model_dir(str(tmp_path)) is None
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"do_sample": True, "temperature": 0.6, "top_k": 20, "top_p": 0.95,
         "eos_token_id": [151645, 151643], "pad_token_id": 151643}))
    g = GenerationConfig.from_model_dir(str(tmp_path))
    assert g.do_sample and g.top_k == 20 and g.eos_token_ids() == (151645, 151643)
    assert g.extra["pad_token_id"] == 151643
