"""Random weights from a configuration and a seed.

``write_random_model(config_dict, seed, folder)`` writes a model folder
(config.json, model.safetensors) that every loader of this format can read;
``random_tensors`` yields the same tensors without a file, for models too large
to be worth writing.  Every matrix and embedding is N(0, 0.02^2) and every
vector (norm weights) 1 + N(0, 0.1^2).  Each tensor has its own generator,
seeded from (seed, tensor name), so a tensor's values do not depend on which
other tensors are made or in which order.

The reference has no such mode in its loader; the nearest are the fixed formula
of ``NativeQwen3::tiny`` (src/training.rs:420-447) and the seeded checkpoint of
tests/reference_quantized.py:42-72.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors import write_safetensors

MATRIX_STD = 0.02
VECTOR_STD = 0.1


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, spec: ParamSpec, seed: int, dtype=torch.bfloat16,
                  device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, name))
    if spec.kind == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    x = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    if spec.kind == "vector":
        x = 1.0 + VECTOR_STD * x
    else:
        x = MATRIX_STD * x
    return x.to(dtype)


def random_tensors(expected: Dict[str, ParamSpec], seed: int, dtype=torch.bfloat16,
                   device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    for name in sorted(expected):
        yield name, random_tensor(name, expected[name], seed, dtype, device)


def write_random_model(config: dict, seed: int, folder: str, dtype=torch.bfloat16) -> str:
    """config: the raw config.json dict of a registered architecture."""
    from ..engine.model import expected_tensors   # late: the engine imports this package
    from ..config import resolve_architecture
    arch = resolve_architecture(config)
    cfg = arch.config_cls.from_dict(config)
    expected = expected_tensors(arch.plan(cfg))
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config, fh, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      list(random_tensors(expected, seed, dtype)),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
