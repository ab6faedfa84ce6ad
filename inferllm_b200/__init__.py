"""inferllm_b200: a small, whole LLaMA generation library for one NVIDIA B200.

    from inferllm_b200 import Model, ModelConfig
    m = Model(ModelConfig(compt_type="bfloat16", nr_ctx=4096)); m.load("model_folder")
    m.init(top_k=40, top_p=0.95, temp=0.1, repeat_penalty=1.3, repeat_last_n=64, seed=1, end_token=2)
    out = m.generate([[1, 5, 17], [1, 9]], max_new_tokens=32)
"""
from .config import ConfigError, LlamaConfig
from .engine import (Engine, EngineError, EngineOptions, GenerationResult, Model, ModelConfig,
                     StepItem, generate)
from .registry import (config_from_dict, config_from_folder, get_architecture,
                       register_architecture, registered_architectures)
from .sampling import Sampler, SamplingParams
from .weights import WeightError, write_random_model


def library_errors():
    """The exception classes with which the library refuses something it was asked for (a bad
    configuration, weights that do not fit, a request the cache or the kernels cannot take): what a
    command line reports in one line instead of a traceback."""
    from .cache import CacheError
    from .engine.generate import RequestTooLong
    from .kernels.lib import KernelLibraryError
    from .kernels.ops import KernelError
    from .weights.safetensors_io import SafetensorsError
    return (ConfigError, WeightError, SafetensorsError, EngineError, CacheError, RequestTooLong, KernelError,
            KernelLibraryError)


__all__ = ["ConfigError", "LlamaConfig", "Engine", "EngineError", "EngineOptions",
           "GenerationResult", "Model", "ModelConfig", "StepItem", "generate", "config_from_dict",
           "config_from_folder", "get_architecture", "register_architecture",
           "registered_architectures", "Sampler", "SamplingParams", "WeightError",
           "write_random_model", "library_errors"]
__version__ = "0.1.0"
