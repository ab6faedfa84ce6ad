"""Loading a model's tensors from safetensors by name, and writing a random model folder.

The reference looks tensors up by name as well, after translating the file's names through
an alias table (src/graph/llama_like.cpp:9-22, src/core/graph.cpp:233-257); an unknown tensor
is skipped with a log line (:311-317), a wrong size aborts (:322-326) and a tensor that the
file lacks goes unnoticed (src/core/tensor.cpp:57-59).  Here the model declares every tensor
it needs under the file's own names, and one error lists all that is missing, unexpected or
of the wrong shape before anything is copied.

Storage rule: floating-point tensors stored in 16 bits are kept in bfloat16, a tensor stored
in 32-bit stays so, integer tables become int32; in the float32 mode every floating-point
tensor is widened to float32.  Matrices are then brought to the compute dtype by the part
that owns them.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from .random_init import random_key, random_values, to_bfloat16_bits
from .safetensors_io import SafetensorsError, open_model_files, write_safetensors


class WeightError(ValueError):
    """The weight file does not fit the model; the message lists every mismatch."""


_IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)  # derived tables some exporters store


def check_names_and_shapes(decls, records) -> None:
    missing = sorted(n for n in decls if n not in records)
    unexpected = sorted(n for n in records if n not in decls and not n.endswith(_IGNORED_SUFFIXES))
    wrong = sorted((n, tuple(decls[n].shape), tuple(records[n].shape)) for n in decls
                   if n in records and tuple(records[n].shape) != tuple(decls[n].shape))
    if not (missing or unexpected or wrong):
        return
    lines = ["the weight file does not match the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(
            f"{n} expected {list(e)} found {list(f)}" for n, e, f in wrong))
    raise WeightError("\n".join(lines))


def storage_dtype(stored: torch.dtype, runtime_dtype: torch.dtype, init: str) -> torch.dtype:
    if init == "int" or not stored.is_floating_point:
        return torch.int32
    if runtime_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_model_weights(model, folder: str) -> None:
    """Check the folder's tensors against `model.tensor_decls()` and hand them to the parts."""
    decls = model.tensor_decls()
    try:
        records, files = open_model_files(folder)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    try:
        check_names_and_shapes(decls, records)
        rt = model.rt

        def fetch(name):
            rec = records[name]
            t = rec.file.tensor(name)
            return t.to(device=rt.device, dtype=storage_dtype(rec.dtype, rt.dtype, decls[name].init))

        model.load_tensors(fetch)
    finally:
        for f in files:
            f.close()


# ---- random weights


def random_tensor(name: str, decl, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """Matrices N(0, 0.02), norm weights 1 + N(0, 0.02), each from the stream of (seed, tensor
    name), so a tensor does not depend on which others exist.  The numbers are defined bit by bit
    (`weights.random_init`, `csrc/random_init.h`): on a CUDA device they are made by the fill kernel,
    on the host by numpy, and both give the same tensor."""
    if decl.init == "int":
        return torch.zeros(decl.shape, dtype=torch.int32, device=device)
    n = 1
    for d in decl.shape:
        n *= int(d)
    mean = 1.0 if decl.init == "norm" else 0.0
    if torch.device(device).type == "cuda":
        from ..kernels import ops
        store = dtype if dtype in (torch.float32, torch.bfloat16) else torch.float32
        out = torch.empty(decl.shape, dtype=store, device=device)
        ops.fill_random(out, random_key(seed, name), 0.02, mean)
        return out.to(dtype)
    vals = random_values(seed, name, n, 0.02, mean)
    if dtype == torch.bfloat16:
        t = torch.from_numpy(to_bfloat16_bits(vals).view("int16")).view(torch.bfloat16)
    else:
        t = torch.from_numpy(vals).to(dtype)
    return t.reshape(decl.shape)


def write_random_model(config, folder: str, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write `config.json` and `model.safetensors` with random weights for `config`
    (a typed configuration of a registered architecture)."""
    from ..registry import get_architecture

    os.makedirs(folder, exist_ok=True)
    model = get_architecture(config.architecture).build_model(config, None)
    decls = model.tensor_decls()
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                        torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    tensors = [(name, random_tensor(name, decl, seed, dtype)) for name, decl in decls.items()]
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed})
    return folder


def init_random_weights(model, seed: int) -> None:
    """Fill a model on its device with random weights without going through a file (for
    sizes where writing and reading tens of gigabytes would only cost time)."""
    decls = model.tensor_decls()
    rt = model.rt
    store = torch.float32 if rt.is_f32 else torch.bfloat16

    def fetch(name):
        return random_tensor(name, decls[name], seed, store, device=rt.device)

    model.load_tensors(fetch)
