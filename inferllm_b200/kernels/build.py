"""Compiling inferllm_b200 for sm_100a: the CUDA kernels of `csrc/`, the C++ core beside them (one
shared library, `libinferllm_b200.so`) and the two programs `illm_llama` and `illm_trace_run`.

nvcc compiles the `.cu` files and g++ the `.cpp` files (no framework headers are involved: the
kernels' entry points are plain C functions that take device pointers, and the core is plain
C++17 over the CUDA runtime and cuBLAS), so a build from scratch takes about a minute.  The results
are kept in `csrc/_build/` inside the package when that folder can be written, else in a per-user
folder under the system's temporary directory; a stamp per object file says whether it is current,
so a change rebuilds only what it touches.  Progress lines go to stderr.

    python inferllm_b200/kernels/build.py [--force]
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

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG, "csrc")
LIB_NAME = "libinferllm_b200.so"
PROGRAMS = {"illm_llama": "programs/llama.cpp", "illm_trace_run": "programs/trace_run.cpp"}
CORE_DIRS = ("util", "config", "weights", "device", "cache", "kernels", "parts", "models", "engine", "sampling", "binding")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wno-unused-function", "-ffp-contract=off"]


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


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("no C++ compiler found (looked at $CXX, g++ and c++)")


def cuda_home(nvcc: str) -> str:
    return os.path.dirname(os.path.dirname(os.path.realpath(nvcc)))


def sources():
    """(relative path, kind) of everything that goes into the library."""
    out = [(os.path.join("csrc", f), "cu") for f in sorted(os.listdir(CSRC)) if f.endswith(".cu")]
    for d in CORE_DIRS:
        full = os.path.join(PKG, d)
        if os.path.isdir(full):
            out += [(os.path.join(d, f), "cpp") for f in sorted(os.listdir(full)) if f.endswith(".cpp")]
    return out


def _headers_hash() -> str:
    h = hashlib.sha256()
    for d in ("csrc", "programs") + CORE_DIRS:
        full = os.path.join(PKG, d)
        if not os.path.isdir(full):
            continue
        for f in sorted(os.listdir(full)):
            if f.endswith((".h", ".cuh")):
                h.update(f"{d}/{f}".encode())
                with open(os.path.join(full, f), "rb") as fh:
                    h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def _source_stamp(rel: str, headers: str) -> str:
    h = hashlib.sha256(headers.encode())
    with open(os.path.join(PKG, rel), "rb") as fh:
        h.update(fh.read())
    return h.hexdigest()


def _stamp() -> str:
    headers = _headers_hash()
    h = hashlib.sha256(headers.encode())
    for rel, _ in sources() + [(p, "cpp") for p in PROGRAMS.values()]:
        h.update(_source_stamp(rel, headers).encode())
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
    raise BuildError(f"no writable folder for the compiled library (tried {local} and {alt})")


def _candidates():
    cands = [os.path.join(CSRC, "_build"),
             os.path.join(tempfile.gettempdir(), f"inferllm_b200_build_{os.getuid()}")]
    if os.environ.get("ILLM_BUILD_DIR"):
        cands.insert(0, os.environ["ILLM_BUILD_DIR"])
    return cands


def current_library():
    """Path of an up-to-date library (with its programs beside it) if one exists, in-tree first."""
    want = _stamp()
    for d in _candidates():
        lib, st = os.path.join(d, LIB_NAME), os.path.join(d, "stamp.txt")
        if os.path.isfile(lib) and os.path.isfile(st) and all(os.path.isfile(os.path.join(d, p)) for p in PROGRAMS):
            with open(st) as f:
                if f.read().strip() == want:
                    return lib
    return None


def build(force: bool = False, verbose: bool = True, extra_flags=()) -> str:
    """Compile what is stale and return the path of the shared library."""
    if not force:
        lib = current_library()
        if lib:
            return lib
    nvcc, cxx = find_nvcc(), find_cxx()
    inc = os.path.join(cuda_home(nvcc), "include")
    out = build_dir()
    # one builder per folder at a time: a second process that starts meanwhile waits and then finds the
    # finished library instead of compiling into the same object files
    import fcntl
    lock = open(os.path.join(out, ".lock"), "w")
    try:
        fcntl.flock(lock, fcntl.LOCK_EX | fcntl.LOCK_NB)
    except OSError:
        if verbose:
            _log("another process is compiling the library; waiting for it")
        fcntl.flock(lock, fcntl.LOCK_EX)
    try:
        if not force:
            lib = current_library()
            if lib:
                return lib
        return _build_locked(nvcc, cxx, inc, out, force, verbose, extra_flags)
    finally:
        fcntl.flock(lock, fcntl.LOCK_UN)
        lock.close()


def _build_locked(nvcc, cxx, inc, out, force, verbose, extra_flags) -> str:
    headers = _headers_hash()
    srcs = sources()
    t0 = time.time()
    todo = []
    for rel, kind in srcs:
        obj = os.path.join(out, rel.replace(os.sep, "_").rsplit(".", 1)[0] + ".o")
        stamp = _source_stamp(rel, headers) + " " + " ".join(extra_flags)
        st_path = obj + ".stamp"
        fresh = False
        if not force and os.path.isfile(obj) and os.path.isfile(st_path):
            with open(st_path) as f:
                fresh = f.read() == stamp
        todo.append((rel, kind, obj, stamp, fresh))
    stale = [t for t in todo if not t[4]]
    if verbose and stale:
        _log(f"compiling {len(stale)} of {len(todo)} sources for sm_100a into {out} (first call only)")

    def compile_one(item):
        rel, kind, obj, stamp, fresh = item
        if fresh:
            return obj
        src = os.path.join(PKG, rel)
        if kind == "cu":
            cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-I", CSRC, "-I", PKG, "-c", src, "-o", obj]
        else:
            cmd = [cxx, *CXX_FLAGS, "-I", PKG, "-I", inc, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"compiling {rel} failed:\n{r.stdout}\n{r.stderr}")
        with open(obj + ".stamp", "w") as f:
            f.write(stamp)
        if verbose:
            _log(f"  compiled {rel} ({time.time() - t0:.0f} s)")
        if r.stderr.strip() and verbose and "-Xptxas" in " ".join(extra_flags):
            _log(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, todo))
    lib = os.path.join(out, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-lcublas"], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    for prog, rel in PROGRAMS.items():
        exe = os.path.join(out, prog)
        tmp = exe + f".tmp{os.getpid()}"
        cmd = [cxx, *CXX_FLAGS, "-I", PKG, "-I", inc, os.path.join(PKG, rel), "-o", tmp, f"-L{out}", "-linferllm_b200",
               "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda_home(nvcc), "lib64")]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"building {prog} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, exe)
    with open(os.path.join(out, "stamp.txt"), "w") as f:
        f.write(_stamp() + "\n")
    if verbose:
        _log(f"built {lib} and {', '.join(PROGRAMS)} in {time.time() - t0:.0f} s")
    return lib


def program(name: str) -> str:
    """Path of a built program (`illm_llama`, `illm_trace_run`), building first if anything is stale."""
    return os.path.join(os.path.dirname(build()), name)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
