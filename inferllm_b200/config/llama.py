"""Typed configuration of the LLaMA dense decoder, read from its config.json keys.

The reference reads five integers from its own file header (`n_embd, n_head, n_layer,
n_mult, n_vocab`, src/graph/llama_like.cpp:37-44) and fixes everything else in code:
eps 1e-6 in the layers (src/graph/llama_like.cpp:77-78), rope base 10000
(src/kern/naive/naive.cpp:396), rotate-half over the whole head (:60,:82), no biases,
BOS 1 (src/core/model_imp.cpp:124), EOS 2 (application/llama/llama.cpp:175), context
2048 (application/llama/llama.cpp:25).  Here those constants are the defaults of the
corresponding config.json keys and nothing else in the package repeats them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import (ArchConfig, ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                   take)


@dataclass
class LlamaConfig(ArchConfig):
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    vocab_size: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = 1
    eos_token_id: List[int] = field(default_factory=lambda: [2])
    torch_dtype: str = "bfloat16"

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        nh = take(d, "num_attention_heads", int)
        H = take(d, "hidden_size", int)
        nkv = take(d, "num_key_value_heads", int, nh)
        if nh <= 0 or nkv <= 0 or H <= 0:
            raise ConfigError("config.json: sizes must be positive")
        if "head_dim" in d and d["head_dim"] is not None:
            hd = take(d, "head_dim", int)
        else:
            if H % nh:
                raise ConfigError(f"config.json: hidden_size {H} is not a multiple of "
                                  f"num_attention_heads {nh} and no head_dim is given")
            hd = H // nh
        if nh % nkv:
            raise ConfigError(f"config.json: num_attention_heads {nh} is not a multiple of "
                              f"num_key_value_heads {nkv}")
        if hd % 2:
            raise ConfigError(f"config.json: head_dim {hd} must be even (rotary pairs)")
        act = take(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (only 'silu')")
        for key in ("attention_bias", "mlp_bias"):
            if take(d, key, bool, False):
                raise ConfigError(f"config.json: {key}=true is not supported")
        if d.get("rope_scaling") is not None:
            raise ConfigError("config.json: rope_scaling is not supported (must be null)")
        eos = d.get("eos_token_id", 2)
        if isinstance(eos, bool) or not isinstance(eos, (int, list)):
            raise ConfigError(f"config.json: eos_token_id must be an int or a list, found {eos!r}")
        eos = [eos] if isinstance(eos, int) else [int(e) for e in eos]
        cfg = cls(
            hidden_size=H,
            num_hidden_layers=take(d, "num_hidden_layers", int),
            num_attention_heads=nh,
            intermediate_size=take(d, "intermediate_size", int),
            vocab_size=take(d, "vocab_size", int),
            num_key_value_heads=nkv,
            head_dim=hd,
            rms_norm_eps=take(d, "rms_norm_eps", float, 1e-6),
            rope_theta=take(d, "rope_theta", float, 10000.0),
            max_position_embeddings=take(d, "max_position_embeddings", int, 2048),
            tie_word_embeddings=take(d, "tie_word_embeddings", bool, False),
            bos_token_id=take(d, "bos_token_id", int, 1),
            eos_token_id=eos,
            torch_dtype=take(d, "torch_dtype", str, "bfloat16"),
        )
        for name in ("num_hidden_layers", "intermediate_size", "vocab_size",
                     "max_position_embeddings"):
            if getattr(cfg, name) <= 0:
                raise ConfigError(f"config.json: {name} must be positive")
        if cfg.rms_norm_eps <= 0 or cfg.rope_theta <= 0:
            raise ConfigError("config.json: rms_norm_eps and rope_theta must be positive")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        eos = self.eos_token_id[0] if len(self.eos_token_id) == 1 else list(self.eos_token_id)
        return {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
            "rope_scaling": None,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": eos,
            "torch_dtype": self.torch_dtype,
        }

    def model_spec(self) -> ModelSpec:
        """Layer stack of src/graph/llama_like.cpp:54-109: every layer is a pre-norm block
        of causal attention with rotate-half position encoding and a gated feed-forward;
        the layers run once each, in order, each with a cache entry of its own."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        position = PartSpec("rope_half", {
            "head_dim": self.head_dim, "rot_dim": self.head_dim, "theta": self.rope_theta,
            "max_positions": self.max_position_embeddings})
        mixer = PartSpec("attention", {
            "hidden_size": self.hidden_size, "n_heads": self.num_attention_heads,
            "n_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "window": None, "position": position})
        ffn = PartSpec("gated_mlp", {
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "activation": "silu"})
        names = {"mixer": "self_attn.", "ffn": "mlp.", "norm1": "input_layernorm.",
                 "norm2": "post_attention_layernorm."}
        layers = [LayerSpec("prenorm", mixer, ffn, norm, f"model.layers.{i}.", dict(names))
                  for i in range(self.num_hidden_layers)]
        schedule = [ScheduleEntry(i, i, True) for i in range(self.num_hidden_layers)]
        return ModelSpec(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size, layers=layers,
            schedule=schedule,
            embedding=PartSpec("embedding", {"name": "model.embed_tokens.",
                                             "vocab_size": self.vocab_size,
                                             "hidden_size": self.hidden_size}),
            final_norm=PartSpec("rmsnorm", {"name": "model.norm.", "size": self.hidden_size,
                                            "eps": self.rms_norm_eps}),
            head=PartSpec("lm_head", {"name": "lm_head.", "tied": self.tie_word_embeddings,
                                      "vocab_size": self.vocab_size,
                                      "hidden_size": self.hidden_size}),
            max_positions=self.max_position_embeddings,
            bos_token_id=self.bos_token_id, eos_token_ids=list(self.eos_token_id))
