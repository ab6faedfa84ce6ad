"""Compiling the CUDA sources of `inferllm_b200/csrc` into one shared library for sm_100a.

nvcc is called directly (no torch headers are involved: the entry points are plain C
functions that take device pointers), so a build from scratch takes well under a minute.
The library is kept in `csrc/_build/` inside the package when that folder can be written,
else in a per-user folder under the system's temporary directory; a stamp of the sources
and flags beside it says whether it is current.  Progress lines go to stderr.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libinferllm_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _log(msg):
    print(f"[inferllm_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("ILLM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $ILLM_NVCC, PATH and /usr/local/cuda/bin): the "
                     "CUDA kernels of inferllm_b200 cannot be compiled, and there is no other path")


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stamp() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("ILLM_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    local = os.path.join(CSRC, "_build")
    if _writable_dir(local):
        return local
    alt = os.path.join(tempfile.gettempdir(), f"inferllm_b200_build_{os.getuid()}")
    if _writable_dir(alt):
        return alt
    raise BuildError(f"no writable folder for the compiled kernels (tried {local} and {alt})")


def current_library():
    """Path of an up-to-date library if one exists (in-tree first), else None."""
    want = _stamp()
    cands = [os.path.join(CSRC, "_build"),
             os.path.join(tempfile.gettempdir(), f"inferllm_b200_build_{os.getuid()}")]
    if os.environ.get("ILLM_BUILD_DIR"):
        cands.insert(0, os.environ["ILLM_BUILD_DIR"])
    for d in cands:
        lib, st = os.path.join(d, LIB_NAME), os.path.join(d, "stamp.txt")
        if os.path.isfile(lib) and os.path.isfile(st):
            with open(st) as f:
                have = f.read().strip()
            if have == want:
                return lib
    return None


def build(force: bool = False, verbose: bool = True, extra_flags=()) -> str:
    """Compile what is stale and return the path of the shared library."""
    if not force:
        lib = current_library()
        if lib:
            return lib
    nvcc = find_nvcc()
    out = build_dir()
    stamp = _stamp()
    srcs = sources()
    if verbose:
        _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {out} (first call only)")
    t0 = time.time()

    def compile_one(src):
        obj = os.path.join(out, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _log(f"  compiled {src} ({time.time() - t0:.0f} s)")
        if r.stderr.strip() and verbose and "-Xptxas" in " ".join(extra_flags):
            _log(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, srcs))
    lib = os.path.join(out, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(os.path.join(out, "stamp.txt"), "w") as f:
        f.write(stamp + "\n")
    if verbose:
        _log(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
