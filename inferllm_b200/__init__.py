"""inferllm_b200: a small, whole LLaMA generation library for one NVIDIA B200.

The library is C++ and CUDA (`libinferllm_b200.so`, the programs `bin/llama` and `bin/trace_run`);
this package is its Python face.

    from inferllm_b200 import Model, ModelConfig
    m = Model(ModelConfig(compt_type="bfloat16", nr_ctx=4096)); m.load("model_folder")
    m.init(top_k=40, top_p=0.95, temp=0.1, repeat_penalty=1.3, repeat_last_n=64, seed=1, end_token=2)
    out = m.generate([[1, 5, 17], [1, 9]], max_new_tokens=32)
"""
from .binding import (CacheError, CacheFull, ConfigError, EngineError, KernelError, KernelLibraryError, RequestTooLong,
                      WeightError, library_errors)
from .config import (ArchConfig, LlamaConfig, config_from_dict, config_from_folder, register_architecture,
                     registered_architectures, unregister_architecture)
from .engine import Engine, EngineOptions, GenerationResult, Limits, Model, ModelConfig, StepItem, generate
from .sampling import Sampler, SamplingParams
from .weights import write_random_model

__all__ = ["ArchConfig", "CacheError", "CacheFull", "ConfigError", "LlamaConfig", "Engine", "EngineError", "EngineOptions",
           "GenerationResult", "KernelError", "KernelLibraryError", "Limits", "Model", "ModelConfig", "RequestTooLong", "StepItem",
           "generate", "config_from_dict", "config_from_folder", "register_architecture", "registered_architectures",
           "unregister_architecture", "Sampler", "SamplingParams", "WeightError", "write_random_model", "library_errors"]
__version__ = "0.2.0"
