"""Python faces of the hand-written sm_100a kernels (``csrc/*.cu``)."""
from .build import build_all, compile_modules, module, KernelBuildError, loaded_modules  # noqa: F401
