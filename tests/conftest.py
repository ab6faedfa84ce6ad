"""Shared fixtures: the tiny configurations, model folders with random weights (made in a
temporary folder, never committed), and the plain implementation's logits for them."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on a B200 with -m gpu)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations that differ in every size and option, plus two whose head sizes
# (64, 128) are the ones the tensor-core kernels take.
TINY = {
    "A": dict(architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=4, head_dim=16, intermediate_size=176,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=128,
              tie_word_embeddings=False, eos_token_id=2),
    "B": dict(architectures=["LlamaForCausalLM"], hidden_size=144, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=2, head_dim=24, intermediate_size=384,
              vocab_size=512, rope_theta=500000.0, rms_norm_eps=1e-6, max_position_embeddings=256,
              tie_word_embeddings=True, eos_token_id=[3, 5]),
    "C": dict(architectures=["LlamaForCausalLM"], hidden_size=320, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=520,
              vocab_size=1000, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=1024,
              tie_word_embeddings=False, eos_token_id=2),
    "D": dict(architectures=["LlamaForCausalLM"], hidden_size=200, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=328,
              vocab_size=777, rope_theta=250000.0, rms_norm_eps=3e-6, max_position_embeddings=640,
              tie_word_embeddings=True, eos_token_id=2),
}
SEEDS = {"A": 11, "B": 22, "C": 33, "D": 44}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json + model.safetensors (bfloat16 values, so that the
    float32 mode, the bfloat16 mode and the plain implementation see the same weights)."""
    from inferllm_b200 import config_from_dict, write_random_model
    out = {}
    for name, cfg in TINY.items():
        d = str(tmp_path_factory.mktemp(f"tiny{name}"))
        write_random_model(config_from_dict(cfg), d, SEEDS[name], torch.bfloat16)
        out[name] = d
    return out


@pytest.fixture(scope="session")
def plain_models(model_folders):
    import plain_llama
    return {name: plain_llama.load_weights(d) for name, d in model_folders.items()}


class PlainLogits:
    """Memoised logits of the plain implementation for (model, token sequence)."""

    def __init__(self, plain_models):
        self.models = plain_models
        self.memo = {}

    def __call__(self, name, ids):
        import plain_llama
        key = (name, tuple(ids))
        if key not in self.memo:
            cfg, w = self.models[name]
            self.memo[key] = plain_llama.forward(cfg, w, list(ids))
        return self.memo[key]


@pytest.fixture(scope="session")
def plain_logits(plain_models):
    return PlainLogits(plain_models)


def random_prompt(name, length, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(0, TINY[name]["vocab_size"], length).tolist()
