"""ghostsuite_b200: GhostSuite's per-sample-gradient hot path as hand-written B200 (sm_100a) kernels.

``ghostsuite_b200.ghostEngines`` mirrors the ``ghostEngines`` package of GhostSuite (same module,
class and function names); ``ghostsuite_b200.ops`` exposes the kernels on torch CUDA tensors;
the kernels themselves live in ``libghost_b200.so`` behind the C ABI of ``include/ghost_b200.h``.
"""
from . import _lib  # noqa: F401

__version__ = "0.1.0"
__all__ = ["_lib", "__version__"]
