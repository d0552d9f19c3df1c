"""What every part of a layer has in common, and the registries of parts.

A model is put together from parts of five families — ``norm``, ``position``,
``mixer``, ``feedforward`` and ``block`` — plus ``embedding`` and ``head``.  A
part is built from a ``PartSpec`` (the name of its kind and its sizes and
constants), declares the tensors it needs by their local names, receives them
once, and is then called by the step function.  No part knows which model it is
in: everything it uses comes from its arguments.

Adding a part: subclass the family's base class, decorate it with
``@register_part("<family>", "<kind>")``; a plan may then name it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor that a part reads from the checkpoint.

    kind: "matrix" (a linear or embedding weight), "vector" (norm weights,
    biases and other small tensors) or "table" (integer tables, kept as int32).
    The loader keeps bfloat16 as bfloat16 and 32-bit as 32-bit for every kind;
    only the true 32-bit path widens, and only half precision is converted.
    """
    shape: Tuple[int, ...]
    kind: str = "matrix"
    optional: bool = False


@dataclass(frozen=True)
class PartSpec:
    """Which part, with which sizes and constants."""
    kind: str
    args: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ProductChoice:
    """Which kernels a linear layer's products run on (``parts.linear.Linear``
    explains the names).  It is an argument of every ``Linear``; parts hand on
    the one in their ``BuildContext``."""
    decode: str = "tc"            # "tc" | "skinny": the product for up to 64 rows
    prefill: str = "auto"         # "auto" | "library" | "pair" | "tc": the product for more rows

    def __post_init__(self):
        if self.decode not in ("tc", "skinny"):
            raise ValueError(f"decode product '{self.decode}': 'tc' or 'skinny'")
        if self.prefill not in ("auto", "library", "pair", "tc"):
            raise ValueError(f"prefill product '{self.prefill}': 'auto', 'library', 'pair' or 'tc'")


@dataclass(frozen=True)
class BuildContext:
    """Where, in which precision and on which product kernels a part computes."""
    dtype: torch.dtype            # torch.bfloat16 or torch.float32
    device: torch.device
    products: ProductChoice = ProductChoice()


class Part:
    """Base of all parts."""

    family = "part"

    def __init__(self, ctx: BuildContext):
        self.ctx = ctx

    # -- weights ----------------------------------------------------------
    def param_specs(self) -> Dict[str, ParamSpec]:
        """Local tensor name -> what is expected under that name."""
        return {}

    def load(self, params: Dict[str, torch.Tensor]) -> None:
        """Takes the tensors named by ``param_specs`` (already on the device)."""
        if params:
            raise ValueError(f"{type(self).__name__} takes no tensors")

    # -- kernels ----------------------------------------------------------
    def kernel_modules(self) -> Tuple[str, ...]:
        """Names of the CUDA sources this part launches, so that they can be
        compiled when the model is built rather than in the first step."""
        return ()

    def children(self) -> Tuple["Part", ...]:
        return ()

    # -- captured steps -----------------------------------------------------
    def captures_prompts(self) -> bool:
        """Whether a prompt step through this part may be captured as a CUDA graph
        and replayed for other prompts of the same bucket of sizes.  That holds
        when ``forward`` queues device work only and takes everything that
        differs between such prompts (how the rows divide into sequences, their
        positions, lengths and slots) from the step's device arrays, never from
        the host copies ``q_lens``, ``starts`` and ``slot_list``, which a captured
        step leaves empty.  Rows of slot -1 and sequences without rows are
        padding.  The default is False: the step then runs launch by launch.
        (Decode steps are always captured; their contract is the mixer's.)"""
        return False


_REGISTRY: Dict[Tuple[str, str], type] = {}


def register_part(family: str, kind: str):
    def deco(cls):
        _REGISTRY[(family, kind)] = cls
        cls.family = family
        cls.kind = kind
        return cls
    return deco


def unregister_part(family: str, kind: str) -> None:
    _REGISTRY.pop((family, kind), None)


def build_part(family: str, spec: PartSpec, ctx: BuildContext) -> Part:
    cls = _REGISTRY.get((family, spec.kind))
    if cls is None:
        known = sorted(k for f, k in _REGISTRY if f == family)
        raise KeyError(f"no {family} part named '{spec.kind}'; known: {known}")
    return cls(ctx, **spec.args)


def known_parts(family: Optional[str] = None):
    return sorted((f, k) for f, k in _REGISTRY if family is None or f == family)
