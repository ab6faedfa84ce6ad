"""Loading the compiled kernel library and declaring its C entry points.

There is no other implementation behind these functions: if the library cannot be
built or loaded, `load()` raises and nothing of the engine runs.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

from . import build as _build

_lib = None

P, I, F, LL = c_void_p, c_int, c_float, c_longlong

_SIGNATURES = {
    "illm_embedding": [P, P, I, P, I, I, I, P, P],
    "illm_add_rmsnorm": [P, P, P, I, P, I, P, I, I, F, I, P],
    "illm_residual_add": [P, P, I, LL, P],
    "illm_swiglu": [P, P, I, I, I, P],
    "illm_rope_kv_write": [P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, I, P, P],
    "illm_attention_generic": [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P],
    "illm_attention_decode": [P, I, P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, F, I, P],
    "illm_attention_decode_supported": [I, I, I],
    "illm_attention_decode_gqa": [P, I, P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, F, I, P],
    "illm_attention_decode_ring": [P, I, P, P, LL, P, I, P, P, P, P, P, I, I, I, I, I, I, F, I, P, P],
    "illm_attention_decode_ring_rope": [P, P, I, LL, P, I, I, I, P, P, LL, P, I, P, P, P, P, P, I, I, I, I, I, I, F, I,
                                        P, P, P],
    "illm_attention_prefill": [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P],
    "illm_gemm_bf16_tc": [P, P, P, I, I, I, I, P, I, P, P, I],
    "illm_splitk_reduce": [P, P, I, LL, I, P],
    "illm_add_rmsnorm_partials": [P, P, I, LL, P, I, P, I, P, I, I, F, I, P],
    "illm_rope_kv_write_partials": [P, P, I, LL, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, I, P, P],
    "illm_gemm_bf16_tc2": [P, P, P, I, I, I, I, I, P, P],
    "illm_swiglu_partials": [P, I, LL, P, I, I, P],
    "illm_gemm_bf16_tc_tune": [I],
    "illm_gemm_bf16_tc_gated": [P, P, P, I, I, I, P, P],
    "illm_set_pdl": [I],
    "illm_launch_count": [],
    "illm_attention_prefill_tc": [P, I, I, P, P, LL, P, I, P, P, P, I, I, I, I, I, I, I, F, P, P],
    "illm_gemm_f32_nt": [P, P, P, I, I, I, I, I, I, P],
    "illm_argmax": [P, I, I, I, P, P, P, P],
    "illm_sample": [P, I, I, I, P, P, I, F, F, I, F, P, P, P, P],
    "illm_sample_scratch_elems": [I, I, I, F],
    "illm_fill_random": [P, I, LL, ctypes.c_ulonglong, F, F, P],
    "illm_poison_pages": [P, P, LL, I, LL, P, I, P],
    "illm_selftest_wait_timeout": [P, P, LL, I, P],
}


class KernelLibraryError(RuntimeError):
    pass


def load():
    """The ctypes handle of the kernel library, building it first if it is stale."""
    global _lib
    if _lib is not None:
        return _lib
    try:
        path = _build.build()
        lib = ctypes.CDLL(path)
    except (OSError, _build.BuildError) as e:
        raise KernelLibraryError(
            f"the CUDA kernel library of inferllm_b200 is not available ({e}); "
            "there is no fallback path") from e
    for name, args in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise KernelLibraryError(f"{path} lacks the entry point {name}: rebuild with "
                                     "`python -m inferllm_b200.kernels.build --force`") from None
        fn.argtypes = args
        fn.restype = c_longlong if name in ("illm_launch_count", "illm_sample_scratch_elems") else c_int
    _lib = lib
    return lib
