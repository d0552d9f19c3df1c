"""Safetensors reading and writing, the loader's error, random weights (no GPU)."""
import json
import os

import pytest
import torch

from conftest import TINY
from grout_b200 import architectures  # noqa: F401
from grout_b200.config import Qwen3Config
from grout_b200.architectures.qwen3 import qwen3_plan
from grout_b200.engine.model import expected_tensors
from grout_b200.parts.base import ParamSpec
from grout_b200.weights import (Checkpoint, DictSource, FolderSource, SafetensorsError, WeightError,
                                load_params, place, random_tensor, write_random_model,
                                write_safetensors)


def test_round_trip_and_foreign_reader(tmp_path):
    from safetensors import safe_open
    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32),
         "c": torch.randn(2, 2), "d": torch.tensor(1.5), "e": torch.zeros(0, 4)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, list(t.items()), {"k": "v"})
    ck = Checkpoint(str(tmp_path))
    assert ck.names() == sorted(t)
    for k, v in t.items():
        assert ck.tensor(k).dtype == v.dtype and torch.equal(ck.tensor(k), v)
    with safe_open(path, "pt") as f:
        for k, v in t.items():
            assert torch.equal(f.get_tensor(k), v)


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), [("x", torch.ones(2))])
    write_safetensors(str(tmp_path / "s2.safetensors"), [("y", torch.zeros(3))])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    ck = Checkpoint(str(tmp_path))
    assert ck.names() == ["x", "y"] and ck.tensor("y").shape == (3,)


def test_broken_files(tmp_path):
    with pytest.raises(SafetensorsError):
        Checkpoint(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\xff" * 20)
    with pytest.raises(SafetensorsError):
        Checkpoint(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_dirs, tmp_path):
    src = FolderSource(model_dirs["B"])
    expected = expected_tensors(qwen3_plan(Qwen3Config.from_dict(TINY["B"])))
    tensors = {n: src.tensor(n) for n in src.shapes()}
    del tensors["lm_head.weight"]
    del tensors["model.layers.1.self_attn.q_norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(256)
    tensors["model.layers.2.mlp.down_proj.weight"] = torch.zeros(224, 96)
    with pytest.raises(WeightError) as e:
        load_params(expected, DictSource(tensors), torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.self_attn.q_norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.2.mlp.down_proj.weight"]
    msg = str(err)
    assert "missing (2)" in msg and "unexpected (1)" in msg and "[224, 96]" in msg and "[96, 224]" in msg


def test_tied_model_wants_no_lm_head(model_dirs):
    names = set(FolderSource(model_dirs["A"]).shapes())
    assert "lm_head.weight" not in names and "model.embed_tokens.weight" in names
    assert "lm_head.weight" in set(FolderSource(model_dirs["B"]).shapes())


def test_precision_policy():
    m, v, t = ParamSpec((2, 2)), ParamSpec((2,), "vector"), ParamSpec((2,), "table")
    bf, f32 = torch.bfloat16, torch.float32
    assert place(torch.zeros(2, 2, dtype=bf), m, bf, "cpu").dtype == bf
    assert place(torch.zeros(2, 2, dtype=f32), m, bf, "cpu").dtype == f32     # 32-bit stays
    assert place(torch.zeros(2, dtype=f32), v, bf, "cpu").dtype == f32
    assert place(torch.zeros(2, 2, dtype=torch.float16), m, bf, "cpu").dtype == bf
    assert place(torch.zeros(2, dtype=torch.int64), t, bf, "cpu").dtype == torch.int32
    assert place(torch.zeros(2, 2, dtype=bf), m, f32, "cpu").dtype == f32      # the 32-bit path widens
    assert place(torch.zeros(2, dtype=torch.int64), t, f32, "cpu").dtype == torch.int32


def test_random_weights_are_reproducible_and_have_the_stated_spread(tmp_path):
    a = write_random_model(TINY["A"], 0, str(tmp_path / "a"))
    b = write_random_model(TINY["A"], 0, str(tmp_path / "b"))
    c = write_random_model(TINY["A"], 1, str(tmp_path / "c"))
    ca, cb, cc = Checkpoint(a), Checkpoint(b), Checkpoint(c)
    assert json.load(open(os.path.join(a, "config.json"))) == TINY["A"]
    for n in ca.names():
        assert torch.equal(ca.tensor(n), cb.tensor(n))
    assert not torch.equal(ca.tensor("model.embed_tokens.weight"), cc.tensor("model.embed_tokens.weight"))
    big = random_tensor("w", ParamSpec((400, 400)), 5, torch.float32)
    assert abs(big.std().item() - 0.02) < 1e-3 and abs(big.mean().item()) < 1e-3
    vec = random_tensor("n", ParamSpec((40000,), "vector"), 5, torch.float32)
    assert abs(vec.mean().item() - 1.0) < 5e-3 and abs(vec.std().item() - 0.1) < 5e-3
    # a tensor's values do not depend on the other tensors
    assert torch.equal(random_tensor("w", ParamSpec((400, 400)), 5, torch.float32), big)
