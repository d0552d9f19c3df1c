"""grout_b200: a small, whole generation library for one B200 (sm_100a).

From a model folder (config.json, safetensors) to next tokens: typed
configuration and an architecture registry, weights by tensor name, layers put
together from parts, a paged cache with one slot per sequence, one step
function for batches of unequal lengths, a generation loop with sampling, and
hand-written CUDA kernels underneath.  Importing the package compiles nothing
and needs no GPU; building an ``Engine`` does.
"""
__version__ = "0.1.0"

from .config import ConfigError, load_config, register_architecture  # noqa: F401


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    raise AttributeError(name)
