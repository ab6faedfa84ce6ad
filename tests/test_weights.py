"""Safetensors reading and writing, loader errors, random model folders (no GPU)."""
import json
import os
import struct

import pytest
import torch
from conftest import TINY

from inferllm_b200 import WeightError, config_from_dict, write_random_model
from inferllm_b200.registry import get_architecture
from inferllm_b200.weights import (SafetensorsError, check_names_and_shapes, open_model_files,
                                   random_tensor, write_safetensors)
from inferllm_b200.weights.loader import storage_dtype


def _decls(name):
    cfg = config_from_dict(TINY[name])
    return get_architecture(cfg.architecture).build_model(cfg, None).tensor_decls()


def test_round_trip_and_independent_reader(tmp_path):
    ts = [("a", torch.randn(3, 5).bfloat16()), ("b", torch.arange(7, dtype=torch.int32)),
          ("c", torch.randn(4)), ("empty", torch.zeros(0, 3))]
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, ts, {"seed": 1})
    recs, files = open_model_files(str(tmp_path))
    for n, t in ts:
        got = files[0].tensor(n)
        assert got.dtype == t.dtype and torch.equal(got, t)
    from safetensors.torch import load_file
    other = load_file(p)
    for n, t in ts:
        assert torch.equal(other[n], t)


def test_declared_names_are_the_checkpoint_names():
    d = _decls("A")
    assert d["model.embed_tokens.weight"].shape == (256, 64)
    assert d["model.layers.1.self_attn.q_proj.weight"].shape == (64, 64)
    assert d["model.layers.0.mlp.down_proj.weight"].shape == (64, 176)
    assert d["model.layers.0.input_layernorm.weight"].init == "norm"
    assert d["model.norm.weight"].shape == (64,) and d["lm_head.weight"].shape == (256, 64)
    assert len(d) == 2 * 9 + 3
    b = _decls("B")
    assert "lm_head.weight" not in b  # tied
    assert b["model.layers.2.self_attn.k_proj.weight"].shape == (2 * 24, 144)
    assert b["model.layers.2.self_attn.o_proj.weight"].shape == (144, 6 * 24)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY["A"])
    d = str(tmp_path)
    write_random_model(cfg, d, 1)
    recs, files = open_model_files(d)
    tensors = {n: files[0].tensor(n).clone() for n in recs}
    for f in files:
        f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(2)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # tolerated
    tensors["lm_head.weight"] = torch.zeros(255, 64)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    recs, files = open_model_files(d)
    with pytest.raises(WeightError) as e:
        check_names_and_shapes(_decls("A"), recs)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.extra.weight" in msg
    assert "inv_freq" not in msg
    assert "wrong shapes (1)" in msg and "lm_head.weight expected [256, 64] found [255, 64]" in msg


def test_truncated_and_corrupt_files(tmp_path):
    cfg = config_from_dict(TINY["A"])
    d = str(tmp_path)
    write_random_model(cfg, d, 1)
    p = os.path.join(d, "model.safetensors")
    blob = open(p, "rb").read()
    open(p, "wb").write(blob[:len(blob) // 2])
    with pytest.raises(SafetensorsError, match="truncated"):
        open_model_files(d)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        open_model_files(d)
    open(p, "wb").write(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(SafetensorsError, match="JSON"):
        open_model_files(d)
    os.remove(p)
    with pytest.raises(SafetensorsError, match="neither"):
        open_model_files(d)


def test_sharded_folder(tmp_path):
    d = str(tmp_path)
    write_safetensors(os.path.join(d, "s1.safetensors"), [("a", torch.ones(2))])
    write_safetensors(os.path.join(d, "s2.safetensors"), [("b", torch.zeros(3))])
    json.dump({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}},
              open(os.path.join(d, "model.safetensors.index.json"), "w"))
    recs, files = open_model_files(d)
    assert set(recs) == {"a", "b"} and torch.equal(recs["b"].file.tensor("b"), torch.zeros(3))


def test_random_model_folder(tmp_path):
    cfg = config_from_dict(TINY["B"])
    d1, d2, d3 = (str(tmp_path / n) for n in ("x", "y", "z"))
    write_random_model(cfg, d1, 5)
    write_random_model(cfg, d2, 5)
    write_random_model(cfg, d3, 6)
    assert json.load(open(os.path.join(d1, "config.json")))["num_key_value_heads"] == 2
    assert config_from_dict(json.load(open(os.path.join(d1, "config.json")))) == cfg
    r1, f1 = open_model_files(d1)
    r2, f2 = open_model_files(d2)
    r3, f3 = open_model_files(d3)
    assert set(r1) == set(_decls("B"))
    for n in r1:
        assert r1[n].dtype == torch.bfloat16
        assert torch.equal(f1[0].tensor(n), f2[0].tensor(n))
    assert not torch.equal(f1[0].tensor("model.norm.weight"), f3[0].tensor("model.norm.weight"))
    w = f1[0].tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = f1[0].tensor("model.layers.0.input_layernorm.weight").float()
    assert abs(float(n.mean()) - 1.0) < 0.01


def test_random_tensor_depends_on_name_and_seed_only():
    decl = _decls("A")["model.layers.0.mlp.up_proj.weight"]
    a = random_tensor("x", decl, 1, torch.float32)
    assert torch.equal(a, random_tensor("x", decl, 1, torch.float32))
    assert not torch.equal(a, random_tensor("y", decl, 1, torch.float32))
    assert not torch.equal(a, random_tensor("x", decl, 2, torch.float32))


def test_storage_rule():
    bf, f32, f16 = torch.bfloat16, torch.float32, torch.float16
    assert storage_dtype(bf, bf, "matrix") == bf
    assert storage_dtype(f16, bf, "matrix") == bf
    assert storage_dtype(f32, bf, "norm") == f32          # stored in 32-bit stays so
    assert storage_dtype(bf, f32, "matrix") == f32        # the float32 mode widens everything
    assert storage_dtype(torch.int64, bf, "int") == torch.int32
