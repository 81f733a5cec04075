from .engine import Engine
from .model import LayerCall, ModelPlan
from .step import StepBuilder, StepContext, StepEntry, Workspace

__all__ = ["Engine", "LayerCall", "ModelPlan", "StepBuilder", "StepContext", "StepEntry", "Workspace"]
