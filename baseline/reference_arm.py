"""The reference arm of bench.py: MegEngine/InferLLM itself, unmodified, timed on this machine.

The reference is a CMake C++ project, so "installing" it means building it: its sources are
copied as they are to `baseline/_ref/InferLLM`, built with its own CMakeLists into
`baseline/_ref/build_gpu` (-DENABLE_GPU=ON: its CUDA kernels and cuBLAS SGEMM) and
`baseline/_ref/build_cpu` (its x86 kernels), and `baseline/ref_bench.cpp` is linked against the
static library of each.  That program drives the reference's public `inferllm::Model`
(include/model.h) the way its own command line does and times `decode_iter`.

The reference computes in float32, one sequence at a time, so the arm measures: batch 1,
float32, a model with the LLaMA-2-7B layer sizes and `layers` of its 32 layers (the file holds
float32 weights: 0.81 GB per layer), context 512.  The GPU build is tried first; if it is not
there, does not start or does not finish cleanly, the CPU build runs and the line says why.
"""
from __future__ import annotations

import json
import os
import shutil
import struct
import subprocess
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SRC_CANDIDATES = (os.path.join(REF, "InferLLM"), os.environ.get("ILLM_REFERENCE_SRC", ""))
SIZES_7B = dict(hidden=4096, heads=32, intermediate=11008, vocab=32000)


def word_of(i: int) -> bytes:
    """Token i's word in the model file's vocabulary (the same rule as in ref_bench.cpp)."""
    return bytes(ord("a") + ((i >> s) & 15) for s in (12, 8, 4, 0))


def write_reference_model(path: str, layers: int, seed: int = 0, sizes=SIZES_7B) -> int:
    """A random LLaMA in the reference's container (application/llama/convert.py:69-143,
    src/core/graph.cpp:270-333): float32 matrices N(0, 0.02), norm weights 1 + N(0, 0.02), tensor
    names the checkpoint's own (the reference maps them, src/graph/llama_like.cpp:9-22)."""
    import numpy as np
    H, nh, I, V = sizes["hidden"], sizes["heads"], sizes["intermediate"], sizes["vocab"]
    rng = np.random.default_rng(seed)
    params = struct.pack("<5i", H, nh, layers, I, V)
    vocab = b"".join(struct.pack("<I", 4) + word_of(i) for i in range(V))
    param_off = 4 + 5 * 4
    vocab_off = param_off + len(params)
    tensor_off = vocab_off + len(vocab)

    def tensors():
        yield "model.embed_tokens.weight", (V, H), "matrix"
        for i in range(layers):
            p = f"model.layers.{i}."
            yield p + "input_layernorm.weight", (H,), "norm"
            for n in ("q", "k", "v", "o"):
                yield p + f"self_attn.{n}_proj.weight", (H, H), "matrix"
            yield p + "post_attention_layernorm.weight", (H,), "norm"
            yield p + "mlp.gate_proj.weight", (I, H), "matrix"
            yield p + "mlp.up_proj.weight", (I, H), "matrix"
            yield p + "mlp.down_proj.weight", (H, I), "matrix"
        yield "model.norm.weight", (H,), "norm"
        yield "lm_head.weight", (V, H), "matrix"

    with open(path, "wb") as f:
        f.write(struct.pack("<i", 0x123456))
        f.write(struct.pack("<5i", param_off, len(params), vocab_off, len(vocab), tensor_off))
        f.write(params)
        f.write(vocab)
        for name, shape, kind in tensors():
            nb = name.encode()
            f.write(struct.pack("<3i", len(shape), len(nb), 0))
            f.write(struct.pack(f"<{len(shape)}i", *shape))
            f.write(nb)
            rows = shape[0] if len(shape) == 2 else 1
            cols = shape[-1]
            for r0 in range(0, rows, 4096):          # a piece at a time: the file is several GB
                n = min(4096, rows - r0)
                a = rng.standard_normal((n, cols), dtype=np.float32) * np.float32(0.02)
                if kind == "norm":
                    a += np.float32(1.0)
                f.write(a.tobytes())
    return os.path.getsize(path)


def _run(cmd, cwd=None, timeout=1500, log=None):
    r = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True, timeout=timeout)
    if log:
        with open(log, "w") as f:
            f.write(r.stdout + r.stderr)
    return r


def _source_dir():
    for s in SRC_CANDIDATES:
        if s and os.path.isfile(os.path.join(s, "CMakeLists.txt")):
            return s
    return None


def build(kind: str) -> str:
    """Build the reference (`kind`: "gpu" or "cpu") and the timing program; returns the program's
    path.  Raises RuntimeError with a one-line reason."""
    out = os.path.join(REF, f"build_{kind}")
    exe = os.path.join(out, "ref_bench")
    harness = os.path.join(HERE, "ref_bench.cpp")
    src = _source_dir()
    lib = os.path.join(out, "libInferLLM.a")
    if os.path.isfile(exe) and os.path.getmtime(exe) >= os.path.getmtime(harness):
        return exe
    if src is None:
        raise RuntimeError("the reference's sources are neither under baseline/_ref/InferLLM nor at $ILLM_REFERENCE_SRC")
    if src != SRC_CANDIDATES[0]:                  # keep a copy beside the build, as it is
        dst = os.path.join(REF, "InferLLM")
        if not os.path.isdir(dst):
            os.makedirs(REF, exist_ok=True)
            shutil.copytree(src, dst)
        src = dst
    os.makedirs(out, exist_ok=True)
    gpu_lib = os.path.join(out, "libInferLLMGPU.a")
    if not os.path.isfile(lib) or (kind == "gpu" and not os.path.isfile(gpu_lib)):
        flags = ["-DCMAKE_POLICY_VERSION_MINIMUM=3.5"]
        targets = ["InferLLM"]
        if kind == "gpu":
            flags += ["-DENABLE_GPU=ON", "-DCMAKE_POLICY_DEFAULT_CMP0146=OLD", "-DCUDA_TOOLKIT_ROOT_DIR=/usr/local/cuda",
                      "-DCUDA_NVCC_FLAGS=-gencode;arch=compute_100,code=sm_100"]
            targets.append("InferLLMGPU")
        r = _run(["cmake", src, *flags], cwd=out, log=os.path.join(out, "cmake.log"))
        if r.returncode != 0:
            raise RuntimeError(f"cmake of the reference ({kind}) failed, see {out}/cmake.log")
        r = _run(["make", f"-j{min(8, os.cpu_count() or 2)}", *targets], cwd=out, log=os.path.join(out, "make.log"))
        if r.returncode != 0:
            raise RuntimeError(f"make of the reference ({kind}) failed, see {out}/make.log")
    cmd = ["g++", "-std=c++11", "-O2", "-Wno-multichar", "-I", os.path.join(src, "include"), harness, lib]
    if kind == "gpu":
        cmd += [gpu_lib, "-L/usr/local/cuda/lib64", "-lcublas", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"]
    cmd += ["-lpthread", "-o", exe]
    r = _run(cmd, log=os.path.join(out, "link.log"))
    if r.returncode != 0:
        raise RuntimeError(f"linking ref_bench ({kind}) failed, see {out}/link.log")
    return exe


def measure(kind: str, model_path: str, ctx: int, context_tokens: int, warmup: int, steps: int,
            threads: int, timeout: int = 1200) -> dict:
    exe = build(kind)
    r = _run([exe, model_path, kind, str(threads), str(ctx), str(context_tokens), str(warmup), str(steps)],
             timeout=timeout, log=os.path.join(REF, f"run_{kind}.log"))
    if r.returncode != 0:
        tail = (r.stderr or r.stdout).strip().splitlines()[-1:] or [""]
        raise RuntimeError(f"the reference's {kind} run ended with code {r.returncode}: {tail[0][:160]}")
    for line in reversed(r.stdout.splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    raise RuntimeError(f"the reference's {kind} run printed no result")


def run(steps: int, warmup: int, layers: int = 4, context_tokens: int = 512, gpu_visible: bool = True) -> dict:
    """The reference arm's JSON line (a dict).  Never raises for a reference that cannot run:
    that is reported as {"impl": "reference", "unavailable": why}."""
    notes = []
    tmp = tempfile.mkdtemp(prefix="illm_ref_")
    model_path = os.path.join(tmp, "llama_7b_layers.bin")
    try:
        t0 = time.time()
        nbytes = write_reference_model(model_path, layers)
        notes.append(f"model file {nbytes / 2**30:.1f} GiB written in {time.time() - t0:.0f} s")
        ctx = 2048
        res = None
        for kind in (("gpu", "cpu") if gpu_visible else ("cpu",)):
            try:
                res = measure(kind, model_path, ctx, context_tokens, max(3, warmup), steps,
                              threads=min(16, os.cpu_count() or 4))
                break
            except (RuntimeError, subprocess.TimeoutExpired, OSError) as e:
                notes.append(f"{kind} arm: {e}")
        if res is None:
            return {"impl": "reference", "unavailable": "; ".join(notes)[:400]}
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    ms = res["own_timer_ms_per_token"] if res["own_timer_ms_per_token"] > 0 else res["wall_ms_per_token"]
    return {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048-token prompt",
        "value": round(1e3 / ms, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": max(3, warmup),
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic: random token ids, random-init weights N(0, 0.02)",
        "impl": "reference",
        "config": {"model": "LLaMA-2-7B layer sizes", "global_batch": 1, "seq_len": context_tokens,
                   "parallelism": "none (1 GPU)" if res["device"] == "gpu" else f"none (CPU, {res['threads']} threads)",
                   "layers": layers, "layers_of_config": 32, "hidden": SIZES_7B["hidden"], "heads": SIZES_7B["heads"],
                   "kv_heads": SIZES_7B["heads"], "head_dim": 128, "intermediate": SIZES_7B["intermediate"],
                   "vocab": SIZES_7B["vocab"], "context_len": context_tokens, "device": res["device"],
                   "timer": "the reference's own (decode_summary), execute calls of decode_iter",
                   "like_for_like": "points.ref_like_* of the repo's line: batch 1, same layers, context 512",
                   "l2": f"inputs larger than L2 ({layers * 0.81 + 0.52:.1f} GB of float32 weights read per step)"},
        "e2e": {"value": round(1e3 / res["wall_ms_per_token"], 2), "unit": "tokens/s",
                "note": "wall clock around decode_iter: token in and sampled token out on the host every step",
                "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4 * SIZES_7B["vocab"]},
        "feed_context_s": res["feed_s"], "notes": notes,
        "timed_window_unix": [res.get("timed_begin_unix"), res.get("timed_end_unix")],
    }
