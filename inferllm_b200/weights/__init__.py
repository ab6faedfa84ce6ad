"""Weight files as Python sees them: what a model folder holds, whether it fits a configuration,
random model folders.  The reader, the writer, the check and the generator are the C++ core's
(`weights/safetensors.h`, `weights/loader.h`)."""
from __future__ import annotations

import ctypes
import json
from typing import Dict, List, Tuple

import numpy as np

from .. import binding as _b
from ..binding import SafetensorsError, WeightError   # noqa: F401

_NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "F64": np.float64, "I64": np.int64, "I32": np.int32,
       "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}


def tensor_decls(config) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """Every tensor the model of a configuration reads from a weight file: name -> (shape, init)."""
    return {n: (tuple(s), i) for n, s, i in _b.call_json(_b.lib().illm_tensor_decls, config.handle())}


def check_model_folder(config, folder: str) -> None:
    """WeightError listing every missing tensor, every unexpected one and every wrong shape."""
    _b.check(_b.lib().illm_check_model_folder(config.handle(), folder.encode()))


def write_random_model(config, folder: str, seed: int, dtype="bfloat16") -> str:
    """Write config.json and model.safetensors with random weights for `config` (matrices N(0, 0.02),
    norm weights 1 + N(0, 0.02), from the stream of (seed, tensor name))."""
    name = str(dtype).replace("torch.", "")
    _b.check(_b.lib().illm_write_random_model(config.handle(), folder.encode(), int(seed), name.encode()))
    return folder


def model_files(folder: str) -> Dict[str, dict]:
    """All tensor records of a model folder: name -> {"dtype", "shape", "file", "bytes"}."""
    return _b.call_json(_b.lib().illm_model_files, folder.encode())


def read_tensor(folder: str, name: str) -> np.ndarray:
    """A tensor of a model folder as a numpy array (bfloat16 as its 16 bits, uint16)."""
    rec = model_files(folder)[name]
    arr = np.empty(rec["bytes"], dtype=np.uint8)
    _b.check(_b.lib().illm_model_files_read(folder.encode(), name.encode(), arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes))
    return arr.view(_NP[rec["dtype"]]).reshape(rec["shape"])


def write_safetensors(path: str, tensors: List[Tuple[str, str, np.ndarray]], metadata=None) -> None:
    """Write (name, dtype name, array) triples; a bfloat16 tensor is given as its uint16 bits."""
    arrays = [np.ascontiguousarray(a) for _, _, a in tensors]
    ptrs = (ctypes.c_void_p * max(len(arrays), 1))(*[a.ctypes.data for a in arrays])
    desc = [[n, d, list(a.shape)] for (n, d, _), a in zip(tensors, arrays)]
    _b.check(_b.lib().illm_write_safetensors(path.encode(), json.dumps(desc).encode(), ptrs,
                                             json.dumps(metadata or {}).encode()))


def storage_dtype(stored: str, runtime: str, init: str = "matrix") -> str:
    return _b.call_text(_b.lib().illm_storage_dtype, stored.encode(), runtime.encode(), init.encode())


def random_values(seed: int, name: str, n: int, init: str = "matrix") -> np.ndarray:
    """float32 [n]: the library's own values 0..n-1 of the random tensor `name`."""
    out = np.empty(n, dtype=np.float32)
    _b.check(_b.lib().illm_random_values(int(seed), name.encode(), n, init.encode(), out.ctypes.data_as(ctypes.c_void_p)))
    return out
