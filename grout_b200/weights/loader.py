"""From a model folder's tensors to the parts' tensors, by name.

The model tells which tensors it expects (name, shape, kind); the checkpoint
tells which it has.  Both lists are compared before a byte is copied and every
difference is reported in one ``WeightError``: tensors that are missing,
tensors that nothing asked for, and tensors of the wrong shape.  (The reference
finds out one tensor at a time: "tensor `X` not found in index",
src/loader.rs:69, and checks no shapes but o_proj's, src/model.rs:3736-3742.)

Precision: bfloat16 stays bfloat16 and a tensor stored in 32-bit stays 32-bit;
float16 and float64 are converted to the compute dtype; integer tables become
int32.  The true 32-bit path widens everything to float32.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors import Checkpoint


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"weights of {where} do not fit the model:" if where else
                 "weights do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(exp)}" for n, got, exp in self.wrong_shape))
        super().__init__("\n".join(lines))


def check_names_and_shapes(expected: Dict[str, ParamSpec],
                           found: Dict[str, Tuple[int, ...]], where: str = "") -> None:
    missing = sorted(n for n, s in expected.items() if n not in found and not s.optional)
    unexpected = sorted(n for n in found if n not in expected)
    wrong = sorted((n, found[n], expected[n].shape) for n in expected
                   if n in found and tuple(found[n]) != tuple(expected[n].shape))
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where)


def place(t: torch.Tensor, spec: ParamSpec, compute_dtype: torch.dtype, device) -> torch.Tensor:
    """The tensor on the device in the precision it is used in."""
    if spec.kind == "table" or not t.dtype.is_floating_point:
        return t.to(device=device, dtype=torch.int32)
    if compute_dtype == torch.float32:
        return t.to(device=device, dtype=torch.float32)
    if t.dtype in (torch.bfloat16, torch.float32):
        return t.to(device=device)
    return t.to(device=device, dtype=compute_dtype)       # float16, float64


def load_params(expected: Dict[str, ParamSpec], source: "TensorSource",
                compute_dtype: torch.dtype, device) -> Callable[[str], torch.Tensor]:
    """Checks the source against ``expected`` and returns ``get(name)``."""
    check_names_and_shapes(expected, source.shapes(), source.where)

    def get(name: str) -> torch.Tensor:
        return place(source.tensor(name), expected[name], compute_dtype, device)

    return get


class TensorSource:
    """Anything that has named tensors: a model folder or a dict."""
    where = ""

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        raise NotImplementedError

    def tensor(self, name: str) -> torch.Tensor:
        raise NotImplementedError


class FolderSource(TensorSource):
    def __init__(self, model_dir: str):
        self.ck = Checkpoint(model_dir)
        self.where = model_dir

    def shapes(self):
        return {n: self.ck.entry(n).shape for n in self.ck.names()}

    def tensor(self, name):
        return self.ck.tensor(name)


class DictSource(TensorSource):
    def __init__(self, tensors: Dict[str, torch.Tensor], where: str = "given tensors"):
        self.tensors, self.where = tensors, where

    def shapes(self):
        return {n: tuple(t.shape) for n, t in self.tensors.items()}

    def tensor(self, name):
        return self.tensors[name]
