"""Shared fixtures: tiny configurations, model folders with random weights made
in a temporary folder, and the plain implementation's view of their weights."""
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny A and B differ in every size and option; C adds a window, a head size
# that is no power of two and an odd number of groups; E is written in the other
# form of the file.
TINY = {
    "A": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256,
              hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, rope_theta=10000.0, rms_norm_eps=1e-6,
              max_position_embeddings=128, tie_word_embeddings=True, use_sliding_window=False,
              eos_token_id=255),
    "B": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=384,
              hidden_size=96, intermediate_size=224, num_hidden_layers=3, num_attention_heads=8,
              num_key_value_heads=1, head_dim=32, rope_theta=1000000.0, rms_norm_eps=1e-5,
              max_position_embeddings=256, tie_word_embeddings=False, use_sliding_window=False,
              eos_token_id=[7, 383]),
    "C": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=331,
              hidden_size=80, intermediate_size=176, num_hidden_layers=4, num_attention_heads=6,
              num_key_value_heads=3, head_dim=48, rope_theta=500000.0, rms_norm_eps=3e-6,
              max_position_embeddings=320, tie_word_embeddings=False, use_sliding_window=True,
              sliding_window=40, max_window_layers=1, eos_token_id=330),
    # heads of 64: the shapes that the tensor-memory attention and the register-resident
    # q/k preparation take
    "D": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=200,
              hidden_size=128, intermediate_size=192, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=64, rope_theta=20000.0, rms_norm_eps=2e-6,
              max_position_embeddings=512, tie_word_embeddings=True, use_sliding_window=False,
              eos_token_id=199),
    # the file as newer writers lay it out: the rotation base stands in rope_parameters
    # only, and layer_types names each layer's kind (windowed layers that do not come
    # last); heads of 80 in groups of one
    "E": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=517,
              hidden_size=112, intermediate_size=208, num_hidden_layers=3, num_attention_heads=5,
              num_key_value_heads=5, head_dim=80, rms_norm_eps=1e-5,
              rope_parameters={"rope_type": "default", "rope_theta": 70000.0},
              max_position_embeddings=384, tie_word_embeddings=True, sliding_window=17,
              layer_types=["sliding_attention", "full_attention", "sliding_attention"],
              eos_token_id=[3, 516]),
}
SEEDS = {"A": 0, "B": 2, "C": 4, "D": 6, "E": 8}


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (bfloat16 values)."""
    from grout_b200.weights import write_random_model
    base = tmp_path_factory.mktemp("models")
    out = {}
    for name, cfg in TINY.items():
        out[name] = write_random_model(cfg, SEEDS[name], str(base / name))
    return out


@pytest.fixture(scope="session")
def plain_weights(model_dirs):
    """name -> (config dict, {tensor name: CPU tensor}) read with the safetensors
    package, not with the library's own reader."""
    from safetensors import safe_open
    out = {}
    for name, d in model_dirs.items():
        with open(os.path.join(d, "config.json")) as fh:
            cfg = json.load(fh)
        with safe_open(os.path.join(d, "model.safetensors"), "pt") as f:
            w = {k: f.get_tensor(k) for k in f.keys()}
        out[name] = (cfg, w)
    return out


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
