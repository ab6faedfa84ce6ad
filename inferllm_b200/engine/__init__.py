from .api import Model, ModelConfig
from .generate import GenerationResult, RequestTooLong, generate, generate_pipelined, plan_batches
from .step import Engine, EngineError, EngineOptions, Limits, StepContext, StepItem

__all__ = ["Model", "ModelConfig", "GenerationResult", "RequestTooLong", "generate", "generate_pipelined", "plan_batches",
           "Engine", "EngineError", "EngineOptions", "Limits", "StepContext", "StepItem"]
