"""Mirror of GhostSuite's ``ghostEngines`` package on top of the B200 kernels."""
from .graddotprod_engine import GradDotProdEngine
from .engine_manager import GhostEngineManager
from .gradProjection.gradproj_engine import GradProjLoraEngine, GradProjLoRAEngine

__all__ = ["GradDotProdEngine", "GhostEngineManager", "GradProjLoraEngine", "GradProjLoRAEngine"]
