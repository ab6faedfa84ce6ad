"""Configuration and registry (no GPU)."""
import copy
import json

import pytest
from conftest import TINY

from inferllm_b200 import ConfigError, LlamaConfig, config_from_dict, config_from_folder
from inferllm_b200.config import (ArchConfig, ModelSpec, PartSpec, ScheduleEntry, config_class, register_architecture,
                                  registered_architectures, resolve_architecture, unregister_architecture)


def test_every_key_is_read():
    cfg = config_from_dict(TINY["B"])
    assert isinstance(cfg, LlamaConfig)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads) == (144, 3, 6)
    assert (cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size) == (2, 24, 384)
    assert (cfg.vocab_size, cfg.rope_theta, cfg.rms_norm_eps) == (512, 500000.0, 1e-6)
    assert cfg.max_position_embeddings == 256 and cfg.tie_word_embeddings is True
    assert cfg.eos_token_id == [3, 5]


def test_defaults_are_the_reference_constants():
    d = dict(architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=1,
             num_attention_heads=4, intermediate_size=100, vocab_size=50)
    cfg = config_from_dict(d)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 16
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0
    assert cfg.max_position_embeddings == 2048 and cfg.tie_word_embeddings is False
    assert cfg.bos_token_id == 1 and cfg.eos_token_id == [2]


def test_round_trip_through_to_dict():
    for name in TINY:
        cfg = config_from_dict(TINY[name])
        assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size", "vocab_size", "architectures"])
def test_missing_required_key(key):
    d = copy.deepcopy(TINY["A"])
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("patch,msg", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_hidden_layers": 0}, "positive"),
    ({"rms_norm_eps": 0.0}, "positive"),
    ({"eos_token_id": "2"}, "eos_token_id"),
])
def test_validation_errors(patch, msg):
    d = copy.deepcopy(TINY["A"])
    d.update(patch)
    with pytest.raises(ConfigError, match=msg):
        config_from_dict(d)


def test_hidden_not_multiple_of_heads_needs_head_dim():
    d = copy.deepcopy(TINY["A"])
    d.pop("head_dim")
    d["hidden_size"] = 66
    with pytest.raises(ConfigError, match="head_dim"):
        config_from_dict(d)
    d["head_dim"] = 16
    assert config_from_dict(d).head_dim == 16


def test_unknown_architecture_lists_registered():
    d = copy.deepcopy(TINY["A"])
    d["architectures"] = ["NopeForCausalLM"]
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        config_from_dict(d)


def test_reference_model_names_are_aliases():
    assert resolve_architecture("llama2") == resolve_architecture("LlamaForCausalLM") == "LlamaForCausalLM"
    assert config_class("llama") is LlamaConfig
    assert isinstance(config_from_dict(TINY["A"], model_name="llama2"), LlamaConfig)


def test_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY["A"]))
    assert config_from_folder(str(tmp_path)).vocab_size == 256
    with pytest.raises(ConfigError, match="config.json"):
        config_from_folder(str(tmp_path / "nothing"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        config_from_folder(str(tmp_path))


def test_model_spec_is_data():
    spec = config_from_dict(TINY["B"]).model_spec()
    assert isinstance(spec, ModelSpec) and len(spec.layers) == 3
    assert [(e.layer, e.cache, e.writes) for e in spec.schedule] == [(i, i, True) for i in range(3)]
    m = spec.layers[1].mixer
    assert m.kind == "attention" and m["n_heads"] == 6 and m["n_kv_heads"] == 2 and m["head_dim"] == 24
    assert m["position"].kind == "rope_half" and m["position"]["theta"] == 500000.0
    assert spec.layers[0].ffn.kind == "gated_mlp" and spec.layers[0].ffn["intermediate_size"] == 384
    assert sorted(spec.layers[2].norms) == ["norm1", "norm2"]       # a spec per norm role of the block
    assert spec.layers[2].norms["norm2"]["eps"] == 1e-6 and spec.final_norm["eps"] == 1e-6
    assert spec.embedding.kind == "embedding" and spec.head.kind == "lm_head"     # parts of registries like all others
    assert spec.head["tied"] is True and spec.layers[2].prefix == "model.layers.2."


def test_schedule_validation():
    spec = config_from_dict(TINY["A"]).model_spec()
    spec.schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 0)]
    with pytest.raises(ConfigError, match="both write"):
        spec.validate()
    spec.schedule = [ScheduleEntry(0, 1, writes=False)]
    with pytest.raises(ConfigError, match="before"):
        spec.validate()
    spec.schedule = [ScheduleEntry(5, 0)]
    with pytest.raises(ConfigError, match="names layer"):
        spec.validate()
    spec.schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 0, writes=False)]
    spec.validate()


def test_registering_another_architecture():
    class ToyConfig(ArchConfig):
        def __init__(self, width=8):
            self.width = width

        @classmethod
        def from_dict(cls, d):
            if d.get("width", 8) <= 0:
                raise ValueError("width must be positive")
            return cls(d.get("width", 8))

        def to_dict(self):
            return {"architectures": ["ToyForCausalLM"], "width": self.width}

        def model_spec(self):
            base = config_from_dict(dict(TINY["A"], hidden_size=self.width * 4, head_dim=self.width)).model_spec()
            base.layers[0].norms["norm2"] = PartSpec("rmsnorm", {"size": self.width * 4, "eps": 0.5})
            return base

    register_architecture("ToyForCausalLM", ToyConfig, aliases=("toy",))
    try:
        assert "ToyForCausalLM" in registered_architectures() and resolve_architecture("toy") == "ToyForCausalLM"
        cfg = config_from_dict({"architectures": ["ToyForCausalLM"], "width": 16})
        assert isinstance(cfg, ToyConfig) and cfg.width == 16
        # the library sees the Python class's description: its tensors follow the spec the class returned
        from inferllm_b200.weights import tensor_decls
        assert tensor_decls(cfg)["model.layers.0.self_attn.q_proj.weight"][0] == (64, 64)
        with pytest.raises(ConfigError, match="width must be positive"):
            config_from_dict({"architectures": ["ToyForCausalLM"], "width": 0})
    finally:
        unregister_architecture("ToyForCausalLM")
    assert "ToyForCausalLM" not in registered_architectures()
    with pytest.raises(ConfigError, match="unknown architecture"):
        config_from_dict({"architectures": ["ToyForCausalLM"]})


def test_command_lines_report_refusals_in_one_line(tmp_path):
    """A model folder that is not one: exit code 1 and one line on standard error, no traceback."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for prog, args in (("llama", ["-m", str(tmp_path), "--prompt-ids", "1,2"]),
                       ("trace_run", ["--model", str(tmp_path), "--dtype", "float32", "--out", str(tmp_path / "o"),
                                      "--max-tokens", "64"])):
        r = subprocess.run([os.path.join(root, "bin", prog)] + args, capture_output=True, text=True,
                           stdin=subprocess.DEVNULL, timeout=300)
        assert r.returncode == 1, (prog, r.stderr)
        lines = [ln for ln in r.stderr.splitlines() if ln.strip()]
        assert len(lines) == 1 and lines[0].startswith(f"{prog}: error:") and "config.json" in lines[0], r.stderr
