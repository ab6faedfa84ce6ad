from .api import Model, ModelConfig
from .generate import GenerationResult, RequestTooLong, generate, plan_batches
from .step import Engine, EngineError, EngineOptions, Limits, StepContext, StepItem

__all__ = ["Model", "ModelConfig", "GenerationResult", "RequestTooLong", "generate", "plan_batches",
           "Engine", "EngineError", "EngineOptions", "Limits", "StepContext", "StepItem"]
