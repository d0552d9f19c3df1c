"""The optional ``generation_config.json`` of a model folder.

Restates src/config.rs:46-81 (fields, eos as an int or a list) and the clamps
that the engine applies when it reads it (src/model.rs:1340-1353).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .base import ModelConfig, read_json


@dataclass(frozen=True)
class GenerationConfig(ModelConfig):
    do_sample: Optional[bool] = None
    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    eos_token_id: Union[int, Tuple[int, ...], None] = None

    @classmethod
    def from_model_dir(cls, model_dir: str) -> Optional["GenerationConfig"]:
        path = os.path.join(model_dir, "generation_config.json")
        if not os.path.exists(path):
            return None
        return cls.from_dict(read_json(path), path)

    def eos_token_ids(self) -> Optional[Tuple[int, ...]]:
        if self.eos_token_id is None:
            return None
        if isinstance(self.eos_token_id, int):
            return (self.eos_token_id,)
        return tuple(self.eos_token_id)
