"""Safetensors reading and writing, loader errors, random model folders (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch
from conftest import TINY

from inferllm_b200 import WeightError, config_from_dict, write_random_model
from inferllm_b200.weights import (check_model_folder, model_files, random_values, read_tensor, storage_dtype, tensor_decls,
                                   write_safetensors)


def _decls(name):
    return tensor_decls(config_from_dict(TINY[name]))


def _bf16(t):
    return t.bfloat16().view(torch.int16).numpy().view(np.uint16)


def test_round_trip_and_independent_reader(tmp_path):
    ts = [("a", "bfloat16", _bf16(torch.randn(3, 5))), ("b", "int32", np.arange(7, dtype=np.int32)),
          ("c", "float32", np.random.default_rng(0).normal(size=4).astype(np.float32)), ("empty", "float32", np.zeros((0, 3), np.float32))]
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, ts, {"seed": 1})
    recs = model_files(str(tmp_path))
    assert recs["a"]["dtype"] == "BF16" and recs["a"]["shape"] == [3, 5] and recs["empty"]["bytes"] == 0
    for n, _, a in ts:
        assert np.array_equal(read_tensor(str(tmp_path), n), a)
    from safetensors.torch import load_file
    other = load_file(p)           # an independent reader of the container sees the same tensors
    assert torch.equal(other["a"].view(torch.int16), torch.from_numpy(ts[0][2].view(np.int16)))
    assert torch.equal(other["b"], torch.arange(7, dtype=torch.int32)) and other["empty"].shape == (0, 3)


def test_declared_names_are_the_checkpoint_names():
    d = _decls("A")
    assert d["model.embed_tokens.weight"][0] == (256, 64)
    assert d["model.layers.1.self_attn.q_proj.weight"][0] == (64, 64)
    assert d["model.layers.0.mlp.down_proj.weight"][0] == (64, 176)
    assert d["model.layers.0.input_layernorm.weight"][1] == "norm"
    assert d["model.norm.weight"][0] == (64,) and d["lm_head.weight"][0] == (256, 64)
    assert len(d) == 2 * 9 + 3
    b = _decls("B")
    assert "lm_head.weight" not in b  # tied
    assert b["model.layers.2.self_attn.k_proj.weight"][0] == (2 * 24, 144)
    assert b["model.layers.2.self_attn.o_proj.weight"][0] == (144, 6 * 24)


def _rewrite(folder, change):
    """Read all tensors of the folder, let `change` edit the dict name -> (dtype, array), write them back."""
    names = {"BF16": "bfloat16", "F32": "float32", "I32": "int32"}
    tensors = {n: (names[r["dtype"]], read_tensor(folder, n)) for n, r in model_files(folder).items()}
    change(tensors)
    write_safetensors(os.path.join(folder, "model.safetensors"), [(n, d, a) for n, (d, a) in tensors.items()])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY["A"])
    d = str(tmp_path)
    write_random_model(cfg, d, 1)
    check_model_folder(cfg, d)

    def change(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.extra.weight"] = ("float32", np.zeros(2, np.float32))
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = ("float32", np.zeros(8, np.float32))   # tolerated
        t["lm_head.weight"] = ("float32", np.zeros((255, 64), np.float32))

    _rewrite(d, change)
    with pytest.raises(WeightError) as e:
        check_model_folder(cfg, d)
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
    with pytest.raises(WeightError, match="truncated"):
        model_files(d)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        model_files(d)
    open(p, "wb").write(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(WeightError, match="JSON"):
        model_files(d)
    os.remove(p)
    with pytest.raises(WeightError, match="neither"):
        model_files(d)


def test_sharded_folder(tmp_path):
    d = str(tmp_path)
    write_safetensors(os.path.join(d, "s1.safetensors"), [("a", "float32", np.ones(2, np.float32))])
    write_safetensors(os.path.join(d, "s2.safetensors"), [("b", "float32", np.zeros(3, np.float32))])
    json.dump({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}},
              open(os.path.join(d, "model.safetensors.index.json"), "w"))
    recs = model_files(d)
    assert set(recs) == {"a", "b"} and np.array_equal(read_tensor(d, "b"), np.zeros(3, np.float32))
    assert recs["a"]["file"].endswith("s1.safetensors")
    json.dump({"weight_map": {"a": "s1.safetensors", "c": "s3.safetensors"}},
              open(os.path.join(d, "model.safetensors.index.json"), "w"))
    with pytest.raises(WeightError, match="s3.safetensors"):
        model_files(d)


def test_random_model_folder(tmp_path):
    cfg = config_from_dict(TINY["B"])
    d1, d2, d3 = (str(tmp_path / n) for n in ("x", "y", "z"))
    write_random_model(cfg, d1, 5)
    write_random_model(cfg, d2, 5)
    write_random_model(cfg, d3, 6)
    assert json.load(open(os.path.join(d1, "config.json")))["num_key_value_heads"] == 2
    assert config_from_dict(json.load(open(os.path.join(d1, "config.json")))) == cfg
    r1 = model_files(d1)
    assert set(r1) == set(_decls("B"))
    for n in r1:
        assert r1[n]["dtype"] == "BF16"
        assert np.array_equal(read_tensor(d1, n), read_tensor(d2, n))
    assert not np.array_equal(read_tensor(d1, "model.norm.weight"), read_tensor(d3, "model.norm.weight"))

    def f32(folder, name):
        return torch.from_numpy(read_tensor(folder, name).view(np.int16)).view(torch.bfloat16).float()

    w = f32(d1, "model.layers.0.mlp.gate_proj.weight")
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = f32(d1, "model.layers.0.input_layernorm.weight")
    assert abs(float(n.mean()) - 1.0) < 0.01
    # float32 and float16 folders hold the same numbers, rounded once from the float32 value
    write_random_model(cfg, d3, 5, "float32")
    full = read_tensor(d3, "model.layers.0.mlp.gate_proj.weight")
    assert full.dtype == np.float32 and torch.equal(torch.from_numpy(full).bfloat16().float(), w)


def test_random_numbers_are_the_numpy_twin_bit_for_bit():
    """The library's host generator (model folders) against its numpy twin (tests/random_twin.py); the
    device's fill kernel is compared with the same twin in the GPU tests."""
    import random_twin
    for name, init, mean in (("model.layers.0.mlp.up_proj.weight", "matrix", 0.0), ("model.norm.weight", "norm", 1.0)):
        for seed in (0, 1, 2 ** 40 + 7):
            a = random_values(seed, name, 5000, init)
            b = random_twin.random_values(seed, name, 5000, 0.02, mean)
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    a = random_values(1, "x", 100)
    assert np.array_equal(a, random_values(1, "x", 100)) and not np.array_equal(a, random_values(1, "y", 100))
    assert not np.array_equal(a, random_values(2, "x", 100))


def test_storage_rule():
    assert storage_dtype("bfloat16", "bfloat16", "matrix") == "bfloat16"
    assert storage_dtype("float16", "bfloat16", "matrix") == "bfloat16"
    assert storage_dtype("float32", "bfloat16", "norm") == "float32"          # stored in 32-bit stays so
    assert storage_dtype("bfloat16", "float32", "matrix") == "float32"        # the float32 mode widens everything
    assert storage_dtype("int64", "bfloat16", "int") == "int32"
