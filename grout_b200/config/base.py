"""Typed model configurations read from an architecture's own config.json keys.

A configuration is a frozen dataclass whose field names are the keys of
config.json.  ``ModelConfig.from_dict`` checks presence and type of every
declared key, fills declared defaults, calls the class's ``validate`` and
reports every problem it finds in one ``ConfigError``.  Keys that a class does
not declare are kept in ``extra`` so that nothing of the file is lost, except
those that a class lists in ``changes_arithmetic``: a key there stands for a
term of the model's formulas that the architecture's parts do not have, so a
file that sets it to anything but one of its neutral values is refused instead
of being run as if the key were absent.

The reference parses the same file into ``Qwen3Config`` with serde
(src/config.rs:6-33); it has no defaults, so a missing key is an error there.
"""
from __future__ import annotations

import dataclasses
import json
import os
import typing
from dataclasses import dataclass, field, fields, MISSING
from typing import Any, Union


class ConfigError(ValueError):
    """A config.json that cannot be used; the message lists every problem."""

    def __init__(self, problems, where: str = "config"):
        self.problems = list(problems)
        super().__init__(f"{where}: " + "; ".join(self.problems))


def _type_ok(value: Any, annot: Any) -> bool:
    origin = typing.get_origin(annot)
    if origin is Union:
        return any(_type_ok(value, a) for a in typing.get_args(annot))
    if origin in (list, tuple):
        (inner, *_rest) = typing.get_args(annot) or (Any,)
        return isinstance(value, (list, tuple)) and all(_type_ok(v, inner) for v in value)
    if origin is dict:
        return isinstance(value, dict)
    if annot in (tuple, list):
        return isinstance(value, (list, tuple))
    if annot is Any:
        return True
    if annot is type(None):
        return value is None
    if annot is bool:
        return isinstance(value, bool)
    if annot is int:
        return isinstance(value, int) and not isinstance(value, bool)
    if annot is float:
        return isinstance(value, (int, float)) and not isinstance(value, bool)
    if annot is str:
        return isinstance(value, str)
    return isinstance(value, annot)


def _coerce(value: Any, annot: Any) -> Any:
    """ints are accepted where a float is declared (``"rope_theta": 1000000``)."""
    if annot is float and isinstance(value, int):
        return float(value)
    if typing.get_origin(annot) is Union and float in typing.get_args(annot) \
            and isinstance(value, int) and not isinstance(value, bool) \
            and int not in typing.get_args(annot):
        return float(value)
    if isinstance(value, list):
        return tuple(value)
    return value


def _annot_name(annot: Any) -> str:
    return getattr(annot, "__name__", None) or str(annot).replace("typing.", "")


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration."""

    extra: dict = field(default_factory=dict, repr=False, compare=False, kw_only=True)

    #: undeclared key -> the values with which it changes nothing.  Any other
    #: value is a problem (subclasses replace or extend the table).
    changes_arithmetic: typing.ClassVar[dict] = {}

    # ---- reading -------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(["top level is not an object"], where)
        hints = typing.get_type_hints(cls)
        problems, values = [], {}
        declared = set()
        for f in fields(cls):
            if f.name == "extra":
                continue
            declared.add(f.name)
            annot = hints[f.name]
            if f.name in raw:
                v = raw[f.name]
                if not _type_ok(v, annot):
                    problems.append(f"key '{f.name}' should be {_annot_name(annot)}, "
                                    f"found {type(v).__name__} {v!r}")
                    continue
                values[f.name] = _coerce(v, annot)
            elif f.default is MISSING and f.default_factory is MISSING:
                problems.append(f"required key '{f.name}' is missing")
        for key, neutral in cls.changes_arithmetic.items():
            if key in raw and key not in declared and \
                    not any(raw[key] is n or (not isinstance(raw[key], bool) and n is not None
                                              and not isinstance(n, bool) and raw[key] == n)
                            for n in neutral):
                problems.append(f"key '{key}'={raw[key]!r} changes the model's arithmetic and "
                                f"this architecture has no part for it")
        if problems:
            raise ConfigError(problems, where)
        values["extra"] = {k: v for k, v in raw.items() if k not in declared}
        cfg = cls(**values)
        cfg = cfg.resolved()
        problems = list(cfg.validate())
        if problems:
            raise ConfigError(problems, where)
        return cfg

    @classmethod
    def from_model_dir(cls, model_dir: str):
        path = os.path.join(model_dir, "config.json")
        return cls.from_dict(read_json(path), path)

    # ---- hooks for subclasses -----------------------------------------
    def resolved(self):
        """Fill values that are derived from other keys when absent."""
        return self

    def validate(self):
        """Yield one sentence per problem."""
        return ()

    # ---- writing -------------------------------------------------------
    def to_dict(self) -> dict:
        out = dict(self.extra)
        for f in fields(self):
            if f.name == "extra":
                continue
            v = getattr(self, f.name)
            out[f.name] = list(v) if isinstance(v, tuple) else v
        return out

    def replace(self, **changes):
        return dataclasses.replace(self, **changes)


def read_json(path: str) -> dict:
    try:
        with open(path, "r", encoding="utf-8") as fh:
            return json.load(fh)
    except FileNotFoundError:
        raise ConfigError([f"file not found"], path) from None
    except json.JSONDecodeError as e:
        raise ConfigError([f"not valid JSON ({e})"], path) from None
