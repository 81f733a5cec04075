from .engine import Engine
from .model import LayerCall, ModelPlan
from .step import StepContext, StepEntry, Workspace

__all__ = ["Engine", "LayerCall", "ModelPlan", "StepContext", "StepEntry", "Workspace"]
