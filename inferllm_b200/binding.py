"""The Python side of the C binding: loading `libinferllm_b200.so` (building it first if it is
stale), the exceptions that the library's error classes become, and small helpers for the other
modules of the package, which are thin faces over the library's C entry points
(`binding/c_api_*.cpp`).  There is no other implementation behind them: if the library cannot be
built or loaded, `lib()` raises and nothing runs.
"""
from __future__ import annotations

import ctypes
import json
import os
from ctypes import POINTER, byref, c_char_p, c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p

from .kernels import build as _build


class ConfigError(ValueError):
    """A config.json that cannot be used: missing key, wrong type or unsupported value."""


class WeightError(ValueError):
    """The weight file does not fit the model (the message lists every mismatch) or cannot be read."""


SafetensorsError = WeightError


class CacheError(RuntimeError):
    """Misuse of the cache: a slot that is not live, a page freed twice, and the like."""


class CacheFull(CacheError):
    """No free slot, or not enough free pages for the step."""


class EngineError(RuntimeError):
    pass


class KernelError(RuntimeError):
    pass


class RequestTooLong(ValueError):
    pass


class KernelLibraryError(RuntimeError):
    pass


_ERRORS = {1: ConfigError, 2: WeightError, 3: CacheError, 4: CacheFull, 5: EngineError, 6: KernelError,
           7: RequestTooLong, 8: ValueError}


def library_errors():
    """The exception classes with which the library reports what a caller can cause."""
    return (ConfigError, WeightError, CacheError, EngineError, KernelError, RequestTooLong, KernelLibraryError,
            _build.BuildError)


_lib = None
P, I, LL, ULL, F, D, S = c_void_p, c_int, c_longlong, c_ulonglong, c_float, c_double, c_char_p
PP, PI, PLL = POINTER(c_void_p), POINTER(c_int), POINTER(c_longlong)

# argument types of the entry points (the result is an int status unless named in _RESTYPES)
_SIGNATURES = {
    "illm_last_error": [PI], "illm_free": [P],
    "illm_config_from_json": [S, S, PP], "illm_config_from_folder": [S, S, PP], "illm_config_free": [P],
    "illm_config_to_json": [P, PP], "illm_config_architecture": [P, PP], "illm_config_model_spec": [P, PP],
    "illm_model_spec_validate": [S], "illm_registered_architectures": [PP], "illm_resolve_architecture": [S, PP],
    "illm_registered_parts": [S, PP], "illm_register_architecture": [S, S, P, P], "illm_unregister_architecture": [S],
    "illm_tensor_decls": [P, PP], "illm_check_model_folder": [P, S], "illm_write_random_model": [P, S, ULL, S],
    "illm_storage_dtype": [S, S, S, PP], "illm_random_values": [ULL, S, LL, S, P], "illm_model_files": [S, PP],
    "illm_model_files_read": [S, S, P, LL], "illm_write_safetensors": [S, S, P, S],
    "illm_pool_create": [I, S, PP], "illm_pool_free_handle": [P], "illm_pool_alloc": [P, I, PI],
    "illm_pool_release": [P, PI, I], "illm_pool_check": [P], "illm_pool_stats": [P, PI, PI], "illm_pool_is_held": [P, I],
    "illm_ledger_create": [I, I, I, I, PP], "illm_ledger_free_handle": [P], "illm_ledger_pages_needed": [P, I, LL],
    "illm_ledger_reserve": [P, I, LL], "illm_ledger_release_outside_window": [P, I, LL], "illm_ledger_release_all": [P, I],
    "illm_ledger_release_beyond": [P, I, LL], "illm_ledger_row": [P, I, I, PI], "illm_ledger_check": [P],
    "illm_ledger_pool": [P], "illm_ledger_pages": [P, I, PI, PI, I],
    "illm_cache_create": [S, I, I, I, LL, PP], "illm_cache_wrap": [P], "illm_cache_free_handle": [P],
    "illm_cache_alloc_slot": [P, PI], "illm_cache_free_slot": [P, I], "illm_cache_reset": [P], "illm_cache_check": [P],
    "illm_cache_plan_step": [P, PI, PI, I, PI, PLL, PI], "illm_cache_commit_step": [P, I], "illm_cache_abandon_step": [P, I],
    "illm_cache_stats": [P, PP],
    "illm_generate_with_callbacks": [P, I, PI, PI, LL, PI, I, PP], "illm_plan_batches": [PI, I, LL, I, I, I, LL, PP],
    "illm_engine_create": [P, S, PP], "illm_engine_from_folder": [S, S, S, PP], "illm_engine_free": [P],
    "illm_engine_load_folder": [P, S], "illm_engine_load_random": [P, ULL], "illm_engine_new_sequence": [P, PI],
    "illm_engine_end_sequence": [P, I], "illm_engine_sequence_length": [P, I, PLL], "illm_engine_limits": [P, PLL],
    "illm_engine_step": [P, I, PI, PI, PI, PI, PI, P, P, PP, P], "illm_engine_order": [P, P, I], "illm_engine_warm_up": [P, LL, PI, I],
    "illm_engine_check_device_errors": [P], "illm_engine_cache": [P], "illm_engine_info": [P, PP], "illm_engine_set_gemm": [P, S],
    "illm_launch_count_total": [], "illm_set_pdl_enabled": [I], "illm_uniform_for": [LL, LL, LL],
    "illm_sampling_params_validate": [S], "illm_sampler_create": [P, S, PP], "illm_sampler_free": [P],
    "illm_sampler_choose": [P, P, I, LL, PI, PI, PI, PI, PP],
    "illm_model_create": [S, S, PP], "illm_model_free": [P], "illm_model_load": [P, S], "illm_model_load_random": [P, P, ULL],
    "illm_model_init": [P, ctypes.c_uint, F, F, F, I, LL, I], "illm_model_engine": [P, PP], "illm_model_end_tokens": [P, PP],
    "illm_model_get_remain_token": [P, POINTER(ctypes.c_uint)], "illm_model_reset_token": [P], "illm_model_prefill": [P, PI, I],
    "illm_model_decode": [P, PI, I, PI], "illm_model_decode_iter": [P, PI], "illm_model_decode_summary": [P, PP],
    "illm_model_warm_up": [P, LL, PI, I], "illm_model_generate": [P, I, PI, PI, LL, PI, I, P, P, PP],
    "illm_test_device": [P, PP], "illm_test_device_rewind": [P], "illm_test_device_info": [P, PI, PP, PP],
    "illm_copy_device": [P, P, P, LL], "illm_op_linear": [P, S, P, LL, LL, P, LL, I, I, I, PP, PP, PI],
    "illm_op_linear_gated": [P, S, P, LL, LL, P, LL, I, PP], "illm_policy_gemm_tc_splits": [LL, LL, LL, I],
    "illm_policy_ring_splits": [LL, I, LL, I, I], "illm_policy_attention_supported": [I, I, I, I, I, I],
    "illm_policy_attention_kernels": [I, I, I, I, I, PP],
    "illm_register_foreign_part": [S, S, P], "illm_unregister_part": [S, S],
    "illm_sandbox_create": [S, S, I, I, I, LL, P, PP], "illm_sandbox_free": [P], "illm_sandbox_cache": [P], "illm_sandbox_device": [P],
    "illm_sandbox_build": [P, S, S, PP], "illm_part_free": [P], "illm_part_describe": [P, PP], "illm_sandbox_load": [P, P, S],
    "illm_sandbox_tie": [P, P], "illm_sandbox_begin_step": [P, PI, PI, I, PI, PI, I], "illm_sandbox_commit_step": [P],
    "illm_sandbox_abandon_step": [P], "illm_sandbox_step_info": [P, P], "illm_sandbox_cache_info": [P, I, I, P],
    "illm_sandbox_mixer_forward": [P, P, P, LL, LL, I, I, PP, PLL], "illm_sandbox_ffn_forward": [P, P, P, LL, LL, PP, PLL],
    "illm_stream_create": [P, P, LL, LL, PP], "illm_stream_free": [P], "illm_stream_add": [P, P, I], "illm_stream_flush": [P],
    "illm_stream_has_pending": [P], "illm_sandbox_norm_forward": [P, P, P, P, LL, PP], "illm_sandbox_block": [P, S, P, P, S, PP],
    "illm_block_free": [P], "illm_block_norm_roles": [S, PP], "illm_sandbox_block_forward": [P, P, P, I, I],
}
_RESTYPES = {"illm_last_error": c_char_p, "illm_free": None, "illm_config_free": None, "illm_pool_free_handle": None,
             "illm_ledger_free_handle": None, "illm_cache_free_handle": None, "illm_engine_free": None, "illm_sampler_free": None,
             "illm_model_free": None, "illm_sandbox_free": None, "illm_part_free": None, "illm_stream_free": None,
             "illm_block_free": None, "illm_cache_wrap": c_void_p, "illm_ledger_pool": c_void_p, "illm_engine_cache": c_void_p,
             "illm_sandbox_cache": c_void_p, "illm_sandbox_device": c_void_p, "illm_launch_count_total": c_longlong,
             "illm_set_pdl_enabled": None, "illm_uniform_for": c_float}


def lib():
    """The ctypes handle of the library, building it first if it is stale."""
    global _lib
    if _lib is not None:
        return _lib
    try:
        path = _build.build()
        handle = ctypes.CDLL(path)
    except (OSError, _build.BuildError) as e:
        raise KernelLibraryError(f"the library of inferllm_b200 is not available ({e}); there is no fallback path") from e
    for name, args in _SIGNATURES.items():
        try:
            fn = getattr(handle, name)
        except AttributeError:
            raise KernelLibraryError(f"{path} lacks the entry point {name}: rebuild with "
                                     "`python inferllm_b200/kernels/build.py --force`") from None
        fn.argtypes = args
        fn.restype = _RESTYPES.get(name, c_int)
    _lib = handle
    return handle


def check(rc: int):
    """Raise the exception that belongs to a non-zero status of an entry point."""
    if rc == 0:
        return
    code = c_int(0)
    msg = lib().illm_last_error(byref(code)).decode("utf-8", "replace")
    raise _ERRORS.get(code.value, RuntimeError)(msg)


def take_string(ptr: c_void_p) -> str:
    """The text behind a `char*` that an entry point returned, which is then freed."""
    try:
        return ctypes.cast(ptr, c_char_p).value.decode("utf-8", "replace")
    finally:
        lib().illm_free(ptr)


def call_json(fn, *args):
    """Call an entry point whose last argument is a `char**` result and parse it as JSON."""
    out = c_void_p()
    check(fn(*args, byref(out)))
    return json.loads(take_string(out))


def call_text(fn, *args) -> str:
    out = c_void_p()
    check(fn(*args, byref(out)))
    return take_string(out)


def ints(values):
    """A C array of int from a sequence (kept alive by the caller for the duration of the call)."""
    values = list(values)
    return (c_int * max(len(values), 1))(*values)


def enc(text) -> bytes:
    return None if text is None else str(text).encode()
