"""GradProj: Kronecker-projected per-sample gradients (mirror of ghostEngines.gradProjection)."""
from .gradproj_engine import GradProjLoraEngine, GradProjLoRAEngine, create_gradproj_engine

__all__ = ["GradProjLoraEngine", "GradProjLoRAEngine", "create_gradproj_engine"]
