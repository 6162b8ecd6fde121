"""Model assembly, the step function, the generation loop and the entry points."""

from .api import Engine, build_model, load, random_weights, write_random_model
from .blueprint import LayerSpec, ModelBlueprint, PartSpec, RunSpec
from .generate import Backend, GenerationLoop, Request, Result, plan_batch
from .model import Model, StepContext, Workspace

__all__ = ["Engine", "load", "build_model", "random_weights", "write_random_model", "Model", "StepContext",
           "Workspace", "ModelBlueprint", "LayerSpec", "PartSpec", "RunSpec", "GenerationLoop", "Backend",
           "Request", "Result", "plan_batch"]
