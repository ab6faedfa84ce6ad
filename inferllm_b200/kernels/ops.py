"""Single kernels of the library called from Python, for the tests of each kernel alone and for
the kernel benchmarks (`bench.py --kernels`); the engine does not go through this module.

Every function takes CUDA tensors, allocates the outputs and scratch with torch, launches one
kernel entry point of `csrc/` on torch's current stream and returns without synchronising.  A size
that a kernel cannot take is refused with a `KernelError` that names it.  Which kernel the engine
picks for which sizes is decided in the C++ core (`kernels/ops.h`): `linear`, `linear_gated` and the
policy functions here ask it, so the choices tested are the ones that run.
"""
from __future__ import annotations

import ctypes

import torch

from .. import binding as _b
from ..binding import KernelError   # noqa: F401


def load():
    return _b.lib()

_DT = {torch.float32: 0, torch.bfloat16: 1}
MAX_HEAD_DIM_GENERIC = 256
MAX_NORM_WIDTH = 200 * 1024 // 4


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle (asked for at every launch: the short way, since a prompt
    step of a few hundred tokens is bound by what the host spends per launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


P_, I_, F_, LL_ = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
_KERNEL_SIGNATURES = {
    "illm_embedding": [P_, P_, I_, P_, I_, I_, I_, P_, P_],
    "illm_add_rmsnorm": [P_, P_, P_, I_, P_, I_, P_, I_, I_, F_, I_, P_],
    "illm_residual_add": [P_, P_, I_, LL_, P_],
    "illm_swiglu": [P_, P_, I_, I_, I_, P_],
    "illm_rope_kv_write": [P_, P_, P_, P_, P_, I_, P_, P_, I_, I_, I_, I_, I_, I_, I_, I_, I_, P_, P_],
    "illm_attention_generic": [P_, I_, P_, P_, P_, I_, P_, P_, P_, I_, I_, I_, I_, I_, I_, I_, F_, P_],
    "illm_attention_decode": [P_, I_, P_, P_, P_, I_, P_, P_, P_, P_, P_, I_, I_, I_, I_, I_, I_, F_, I_, P_],
    "illm_attention_decode_supported": [I_, I_, I_],
    "illm_attention_decode_gqa": [P_, I_, P_, P_, P_, I_, P_, P_, P_, P_, P_, I_, I_, I_, I_, I_, I_, F_, I_, P_],
    "illm_attention_decode_ring": [P_, I_, P_, P_, LL_, P_, I_, P_, P_, P_, P_, P_, I_, I_, I_, I_, I_, I_, F_, I_, P_, P_],
    "illm_attention_decode_ring_rope": [P_, P_, I_, LL_, P_, I_, I_, I_, P_, P_, LL_, P_, I_, P_, P_, P_, P_, P_, I_, I_, I_, I_, I_, I_,
                                        F_, I_, P_, P_, P_],
    "illm_attention_prefill": [P_, I_, P_, P_, P_, I_, P_, P_, P_, I_, I_, I_, I_, I_, I_, I_, F_, P_],
    "illm_gemm_bf16_tc": [P_, P_, P_, I_, I_, I_, I_, P_, I_, P_, P_, I_],
    "illm_splitk_reduce": [P_, P_, I_, LL_, I_, P_],
    "illm_add_rmsnorm_partials": [P_, P_, I_, LL_, P_, I_, P_, I_, P_, I_, I_, F_, I_, P_],
    "illm_rope_kv_write_partials": [P_, P_, I_, LL_, P_, P_, P_, P_, I_, P_, P_, I_, I_, I_, I_, I_, I_, I_, I_, I_, P_, P_],
    "illm_gemm_bf16_tc2": [P_, P_, P_, I_, I_, I_, I_, I_, P_, P_],
    "illm_swiglu_partials": [P_, I_, LL_, P_, I_, I_, P_],
    "illm_gemm_bf16_tc_gated": [P_, P_, P_, I_, I_, I_, P_, P_],
    "illm_attention_prefill_tc": [P_, I_, I_, P_, P_, LL_, P_, I_, P_, P_, P_, I_, I_, I_, I_, I_, I_, I_, F_, P_, P_],
    "illm_gemm_f32_nt": [P_, P_, P_, I_, I_, I_, I_, I_, I_, P_, P_],
    "illm_argmax": [P_, I_, I_, I_, P_, P_, P_, P_],
    "illm_sample": [P_, I_, I_, I_, P_, P_, I_, F_, F_, I_, F_, P_, P_, P_, P_],
    "illm_sample_scratch_elems": [I_, I_, I_, F_],
    "illm_fill_random": [P_, I_, LL_, ctypes.c_ulonglong, F_, F_, P_],
    "illm_poison_pages": [P_, P_, LL_, I_, LL_, P_, I_, P_],
    "illm_selftest_wait_timeout": [P_, P_, LL_, I_, P_],
}
_declared = False


def _declare():
    """Argument types of the kernels' own entry points (declared on first use)."""
    global _declared
    if _declared:
        return
    h = _b.lib()
    for name, args in _KERNEL_SIGNATURES.items():
        fn = getattr(h, name)
        fn.argtypes = args
        fn.restype = LL_ if name == "illm_sample_scratch_elems" else I_
    _declared = True


_plain_load = load


def load():   # noqa: F811
    _declare()
    return _plain_load()


_replayed = 0


def launch_count() -> int:
    """How many kernels of this package have been launched: the library counts every kernel it
    launches (a launch into a stream capture once), replays of captured graphs are added by
    `count_launches`.  Library products (cuBLAS) are not counted."""
    return int(_b.lib().illm_launch_count_total()) + _replayed


def count_launches(n: int) -> None:
    """Account for kernels launched by replaying a captured graph."""
    global _replayed
    _replayed += n


def _check(code, what):
    if code != 0:
        if code == 10001:
            raise KernelError(f"{what}: the kernel refused its arguments")
        raise KernelError(f"{what}: CUDA error {code}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _need(t, name, dtype=None, dim=None):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: inferllm_b200 has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} must have {dim} dimensions, found shape {tuple(t.shape)}")
    # rows of a multiple of 16 bytes are read 16 bytes at a time (the address is looked at first: it
    # is almost always aligned, and these checks run a few hundred times per step)
    if t.data_ptr() & 15 and t.dtype.is_floating_point and t.numel() and (t.shape[-1] * t.element_size()) % 16 == 0:
        raise KernelError(f"{name} must start on a 16-byte boundary")


def act_code(dtype):
    if dtype not in _DT:
        raise KernelError(f"unsupported dtype {dtype}: the kernels take float32 and bfloat16")
    return _DT[dtype]


# The library chooses a kernel for every new shape of a product, which costs a prompt step whose
# token count it has not seen before about 4.5 ms (7B size: 9.5 to 10 ms for a prompt of a never
# seen length of 200 to 300 tokens, 5.2 ms for one seen before), and prompts come in every length.
# Activations of prompt steps are therefore allocated with their rows rounded up to a multiple of
# 64, of which the caller sees the first M; `linear` hands the library the whole buffer and gives
# back the first M rows of the result, so the library only ever sees multiples of 64.  The rows
# beyond M are never initialised and never read back: a row of a product depends on its own row
# of the input only.
LIBRARY_ROW_BUCKET = 64


def _rows(M, cols, dtype, device):
    """An uninitialised [M, cols] activation; for prompt-sized M the head of a buffer of whole buckets."""
    if dtype == torch.bfloat16 and M > LIBRARY_ROW_BUCKET and M % LIBRARY_ROW_BUCKET:
        padded = -(-M // LIBRARY_ROW_BUCKET) * LIBRARY_ROW_BUCKET
        return torch.empty((padded, cols), dtype=dtype, device=device)[:M]
    return torch.empty((M, cols), dtype=dtype, device=device)


def _whole_buckets(x):
    """The buffer of whole buckets behind an activation made by `_rows`, or None."""
    M, K = x.shape
    if M > LIBRARY_ROW_BUCKET and M % LIBRARY_ROW_BUCKET and x.storage_offset() == 0:
        padded = -(-M // LIBRARY_ROW_BUCKET) * LIBRARY_ROW_BUCKET
        if x.untyped_storage().nbytes() >= padded * K * x.element_size():
            return x.as_strided((padded, K), (K, 1))
    return None


def embedding(ids, table, err):
    """ids int32 [T], table [V, H] (float32 or bfloat16) -> float32 [T, H]."""
    _need(ids, "ids", torch.int32, 1)
    _need(table, "table", None, 2)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=ids.device)
    _check(load().illm_embedding(_ptr(ids), _ptr(table), act_code(table.dtype), _ptr(out), T, H, V,
                                 _ptr(err), _stream()), "embedding")
    return out


def add_rmsnorm(resid, delta, weight, eps, out_dtype, rows=None, write_resid=True):
    """y = rmsnorm(resid (+ delta)) * weight; resid is updated in place when `write_resid`.
    `rows` (int32 [K]) gathers: only those rows are normed and y is [K, H]."""
    _need(resid, "resid", torch.float32, 2)
    H = resid.shape[1]
    if H > MAX_NORM_WIDTH:
        raise KernelError(f"rmsnorm: width {H} exceeds the {MAX_NORM_WIDTH} that one block's "
                          "shared memory holds")
    partials = None
    if isinstance(delta, SplitKPartials):
        if out_dtype == torch.bfloat16 and H % 8 == 0 and H <= 16384 and tuple(delta.shape) == tuple(resid.shape):
            partials, delta = delta, None
        else:
            delta = delta.materialize(out_dtype)
    if delta is not None:
        _need(delta, "delta", out_dtype, 2)
        if delta.shape != resid.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match resid {tuple(resid.shape)}")
    _need(weight, "norm weight", None, 1)
    if weight.numel() != H:
        raise KernelError(f"norm weight has {weight.numel()} elements, the rows have {H}")
    n = resid.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    y = _rows(n, H, out_dtype, resid.device)
    if partials is not None:
        _check(load().illm_add_rmsnorm_partials(
            _ptr(resid), _ptr(partials.ws), partials.splits, partials.rows * partials.cols, _ptr(weight),
            act_code(weight.dtype), _ptr(y), act_code(out_dtype), _ptr(rows), n, H, float(eps),
            1 if write_resid else 0, _stream()), "add_rmsnorm_partials")
        return y
    _check(load().illm_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(weight), act_code(weight.dtype),
                                   _ptr(y), act_code(out_dtype), _ptr(rows), n, H, float(eps),
                                   1 if write_resid else 0, _stream()), "add_rmsnorm")
    return y


def residual_add(resid, delta):
    if isinstance(delta, SplitKPartials):
        delta = delta.materialize(torch.bfloat16)
    _need(resid, "resid", torch.float32)
    _need(delta, "delta")
    if delta.shape != resid.shape:
        raise KernelError("residual_add: shapes differ")
    _check(load().illm_residual_add(_ptr(resid), _ptr(delta), act_code(delta.dtype), resid.numel(),
                                    _stream()), "residual_add")


def swiglu(gu):
    """silu(gate) * up of a packed projection [T, 2I] whose columns 2i, 2i + 1 are gate and up of
    output i -> [T, I].  `gu` may be `SplitKPartials` (bfloat16 result)."""
    if isinstance(gu, SplitKPartials):
        T, I2 = gu.shape
        if I2 % 16 == 0:
            out = _rows(T, I2 // 2, torch.bfloat16, gu.device)
            _check(load().illm_swiglu_partials(_ptr(gu.ws), gu.splits, gu.rows * gu.cols, _ptr(out), T, I2 // 2,
                                               _stream()), "swiglu_partials")
            return out
        gu = gu.materialize(torch.bfloat16)
    _need(gu, "gu", None, 2)
    T, I2 = gu.shape
    if I2 % 2:
        raise KernelError("swiglu: the packed projection must have an even number of columns")
    out = _rows(T, I2 // 2, gu.dtype, gu.device)
    _check(load().illm_swiglu(_ptr(gu), _ptr(out), act_code(gu.dtype), T, I2 // 2, _stream()), "swiglu")
    return out


def _test_device():
    """The library's device context for calls outside an engine, on torch's current stream."""
    dev = ctypes.c_void_p()
    _b.check(_b.lib().illm_test_device(ctypes.c_void_p(_stream() or 1), ctypes.byref(dev)))    # 1: cudaStreamLegacy (0 would mean "none")
    return dev


_info_dev = None


def _info_device():
    """One device context whose error word and figures serve every call of this module outside an
    engine, whatever torch's current stream is (a context of its own per stream would be created,
    with an allocation, inside a stream capture)."""
    global _info_dev
    if _info_dev is None:
        _info_dev = ctypes.c_void_p()
        _b.check(_b.lib().illm_test_device(ctypes.c_void_p(1), ctypes.byref(_info_dev)))
    return _info_dev


def _take(dev, ptr, shape, dtype, device):
    out = torch.empty(shape, dtype=dtype, device=device)
    if out.numel():
        _b.check(_b.lib().illm_copy_device(dev, out.data_ptr(), ptr, out.numel() * out.element_size()))
    return out


def linear_gated(x, w, backend=None):
    """silu(gate) * up of x [M, K] . w [2I, K]^T, where w's rows 2i, 2i + 1 are the gate and the up
    row of output i -> [M, I], by the kernel the engine picks for these sizes (`ops::linear_gated`)."""
    _need(x, "x", None, 2)
    _need(w, "w", x.dtype, 2)
    dev = _test_device()
    _b.check(_b.lib().illm_test_device_rewind(dev))
    out = ctypes.c_void_p()
    _b.check(_b.lib().illm_op_linear_gated(dev, (backend or _GEMM_BACKEND).encode(), x.data_ptr(), x.shape[0], x.shape[1],
                                           w.data_ptr(), w.shape[0], act_code(x.dtype), ctypes.byref(out)))
    return _take(dev, out, (x.shape[0], w.shape[0] // 2), x.dtype, x.device)


def rope_kv_write(qkv, cos_sin, rot_dim, token_pos, token_seq, block_table, k_cache, v_cache,
                  n_heads, n_kv_heads, head_dim, page_size, write_kv, err):
    """Rotate Q (and K) of the packed projection in place and store K, V in the cache pages.
    `cos_sin` float32 [positions, rot_dim/2, 2] or None with rot_dim 0.  Returns the tensor whose
    first n_heads*head_dim columns hold the rotated queries: `qkv` itself, or, if `qkv` came as
    `SplitKPartials`, a new tensor (the slices are added up on the way)."""
    partials = None
    if isinstance(qkv, SplitKPartials):
        if head_dim % 8 == 0 and rot_dim % 16 == 0 and k_cache is not None and k_cache.dtype == torch.bfloat16:
            partials = qkv
            qkv = torch.empty(partials.shape, dtype=torch.bfloat16, device=partials.device)
        else:
            qkv = qkv.materialize(torch.bfloat16)
    _need(qkv, "qkv", None, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"qkv width {qkv.shape[1]} is not (heads + 2 kv heads) * head_dim")
    for name, t in (("token_pos", token_pos), ("token_seq", token_seq)):
        _need(t, name, torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    if write_kv:
        _need(k_cache, "k_cache", qkv.dtype, 4)
        _need(v_cache, "v_cache", qkv.dtype, 4)
        if tuple(k_cache.shape[1:]) != (n_kv_heads, page_size, head_dim):
            raise KernelError(f"cache pages {tuple(k_cache.shape)} do not match "
                              f"[pages, {n_kv_heads}, {page_size}, {head_dim}]")
    n_pos = 0
    if rot_dim:
        _need(cos_sin, "cos_sin", torch.float32, 3)
        if cos_sin.shape[1] != rot_dim // 2:
            raise KernelError("cos_sin table does not match rot_dim")
        n_pos = cos_sin.shape[0]
    if partials is not None:
        _check(load().illm_rope_kv_write_partials(
            _ptr(qkv), _ptr(partials.ws), partials.splits, partials.rows * partials.cols,
            _ptr(cos_sin) if rot_dim else None, _ptr(token_pos), _ptr(token_seq), _ptr(block_table),
            block_table.shape[1], _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None,
            act_code(qkv.dtype), T, n_heads, n_kv_heads, head_dim, rot_dim, page_size, 1 if write_kv else 0,
            n_pos, _ptr(err), _stream()), "rope_kv_write_partials")
        return qkv
    _check(load().illm_rope_kv_write(
        _ptr(qkv), _ptr(cos_sin) if rot_dim else None, _ptr(token_pos), _ptr(token_seq),
        _ptr(block_table), block_table.shape[1], _ptr(k_cache) if write_kv else None,
        _ptr(v_cache) if write_kv else None, act_code(qkv.dtype), T, n_heads, n_kv_heads, head_dim,
        rot_dim, page_size, 1 if write_kv else 0, n_pos, _ptr(err), _stream()), "rope_kv_write")
    return qkv


def attention_generic(qkv, k_cache, v_cache, block_table, token_pos, token_seq, n_heads,
                      n_kv_heads, head_dim, page_size, window, scale):
    """Attention of each token (query heads in the first n_heads*head_dim columns of `qkv`)
    over its sequence's cache pages; returns [T, n_heads*head_dim]."""
    if head_dim % 8 or head_dim > MAX_HEAD_DIM_GENERIC:
        raise KernelError(f"attention: head size {head_dim} is not supported (multiples of 8 up to "
                          f"{MAX_HEAD_DIM_GENERIC})")
    if n_heads % n_kv_heads:
        raise KernelError("attention: heads must be a multiple of kv heads")
    _need(qkv, "qkv", None, 2)
    _need(k_cache, "k_cache", qkv.dtype, 4)
    _need(v_cache, "v_cache", qkv.dtype, 4)
    T = qkv.shape[0]
    out = _rows(T, n_heads * head_dim, qkv.dtype, qkv.device)
    _check(load().illm_attention_generic(
        _ptr(qkv), qkv.shape[1], _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
        block_table.shape[1], _ptr(token_pos), _ptr(token_seq), _ptr(out), act_code(qkv.dtype), T,
        n_heads, n_kv_heads, head_dim, page_size, int(window or 0), float(scale), _stream()),
        "attention_generic")
    return out


DECODE_CHUNK = 256


def attention_decode_supported(dtype, n_heads, n_kv_heads, head_dim, page_size) -> bool:
    return dtype == torch.bfloat16 and n_heads % n_kv_heads == 0 and bool(
        load().illm_attention_decode_supported(head_dim, n_heads // n_kv_heads, page_size))


def attention_decode(qkv, k_cache, v_cache, block_table, token_pos, token_seq, n_heads, n_kv_heads,
                     head_dim, page_size, window, scale, max_len):
    """bfloat16 attention of single tokens, split over chunks of 256 keys and merged in a fixed
    order.  `max_len` bounds the sequence lengths of the launch (it sizes the grid and the
    scratch, not the result)."""
    _need(qkv, "qkv", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    T = qkv.shape[0]
    n_chunks = max(1, -(-int(max_len) // DECODE_CHUNK))
    part_acc = torch.empty((T, n_heads, n_chunks, head_dim), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((T, n_heads, n_chunks, 2), dtype=torch.float32, device=qkv.device)
    out = _rows(T, n_heads * head_dim, torch.bfloat16, qkv.device)
    for t0 in range(0, T, 65535):
        t1 = min(T, t0 + 65535)
        _check(load().illm_attention_decode(
            _ptr(qkv[t0:t1]), qkv.shape[1], _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
            block_table.shape[1], _ptr(token_pos[t0:t1]), _ptr(token_seq[t0:t1]), _ptr(part_acc[t0:t1]),
            _ptr(part_ml[t0:t1]), _ptr(out[t0:t1]), t1 - t0, n_heads, n_kv_heads, head_dim, page_size,
            int(window or 0), float(scale), n_chunks, _stream()), "attention_decode")
    return out


GQA_DECODE_CHUNK = 128
GQA_DECODE_MIN_GROUP = 4        # from this many query heads per KV head on, the MMA kernel is the faster one


def attention_decode_gqa_supported(dtype, n_heads, n_kv_heads, head_dim) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % n_kv_heads == 0
            and 2 <= n_heads // n_kv_heads <= 16)


def attention_decode_gqa(qkv, k_cache, v_cache, block_table, token_pos, token_seq, n_heads, n_kv_heads,
                         head_dim, page_size, window, scale, max_len):
    """bfloat16 attention of single tokens with grouped heads on warp-level MMAs (the query heads
    of a KV head are the rows of one tile), split over chunks of 128 keys and merged in a fixed
    order.  Any page size, group sizes 2..16, head size 64 or 128."""
    _need(qkv, "qkv", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    T = qkv.shape[0]
    n_chunks = max(1, -(-int(max_len) // GQA_DECODE_CHUNK))
    part_acc = torch.empty((T, n_heads, n_chunks, head_dim), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((T, n_heads, n_chunks, 2), dtype=torch.float32, device=qkv.device)
    out = _rows(T, n_heads * head_dim, torch.bfloat16, qkv.device)
    for t0 in range(0, T, 65535):
        t1 = min(T, t0 + 65535)
        _check(load().illm_attention_decode_gqa(
            _ptr(qkv[t0:t1]), qkv.shape[1], _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
            block_table.shape[1], _ptr(token_pos[t0:t1]), _ptr(token_seq[t0:t1]), _ptr(part_acc[t0:t1]),
            _ptr(part_ml[t0:t1]), _ptr(out[t0:t1]), t1 - t0, n_heads, n_kv_heads, head_dim, page_size,
            int(window or 0), float(scale), n_chunks, _stream()), "attention_decode_gqa")
    return out


RING_DECODE_MAX_SPLITS = 32


def attention_decode_ring_supported(dtype, n_heads, n_kv_heads, head_dim, page_size) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % n_kv_heads == 0
            and n_heads // n_kv_heads <= 16 and page_size % 64 == 0)


def attention_decode_ring_splits(T, n_kv_heads, max_len, head_dim=128, n_sms=None) -> int:
    """Blocks per (token, kv head) of the ring decode attention: the engine's policy
    (`ops::attention_decode_ring_splits`), for the SM count of the current device unless given."""
    return int(_b.lib().illm_policy_ring_splits(int(T), int(n_kv_heads), int(max_len), int(head_dim), int(n_sms or n_sms_of_device())))


def attention_decode_ring(qkv, k_cache, v_cache, block_table, token_pos, token_seq, n_heads, n_kv_heads,
                          head_dim, page_size, window, scale, max_len, splits=None, rope=None):
    """bfloat16 attention of single tokens as a stream: K/V tiles of 64 keys by TMA through a ring
    of shared-memory stages, the query heads of a KV head as rows of warp-level MMAs, the tiles
    of a token dealt round-robin to `splits` blocks and merged in a fixed order.  Group sizes
    1..16, head size 64 or 128, pages of a multiple of 64 positions.

    `rope` = (cos_sin table or None, rot_dim, write_kv, step error word): the kernel also does what
    `rope_kv_write` does (rotation of Q and of the new K row, K and V into the cache pages); `qkv`
    is then the unrotated packed projection, as a bfloat16 tensor or as `SplitKPartials`."""
    partials = None
    if isinstance(qkv, SplitKPartials):
        if rope is None:
            raise KernelError("attention_decode_ring: unreduced slices need the fused position encoding")
        partials = qkv
        T = partials.rows
        width = partials.cols
    else:
        _need(qkv, "qkv", torch.bfloat16, 2)
        T, width = qkv.shape
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    if rope is not None and width != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"qkv width {width} is not (heads + 2 kv heads) * head_dim")
    out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=k_cache.device)
    for t0 in range(0, T, 65535):
        t1 = min(T, t0 + 65535)
        n = attention_decode_ring_splits(t1 - t0, n_kv_heads, max_len, head_dim) if splits is None else int(splits)
        part_acc = part_ml = None
        if n > 1:
            part_acc = torch.empty((t1 - t0, n_heads, n, head_dim), dtype=torch.float32, device=out.device)
            part_ml = torch.empty((t1 - t0, n_heads, n, 2), dtype=torch.float32, device=out.device)
        if rope is None:
            _check(load().illm_attention_decode_ring(
                _ptr(qkv[t0:t1]), width, _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(block_table),
                block_table.shape[1], _ptr(token_pos[t0:t1]), _ptr(token_seq[t0:t1]), _ptr(part_acc), _ptr(part_ml),
                _ptr(out[t0:t1]), t1 - t0, n_heads, n_kv_heads, head_dim, page_size, int(window or 0), float(scale),
                n, _ptr(tc_error_word(out.device)), _stream()), "attention_decode_ring")
            continue
        table, rot_dim, write_kv, step_err = rope
        n_pos = 0
        if rot_dim:
            _need(table, "cos_sin", torch.float32, 3)
            if table.shape[1] != rot_dim // 2:
                raise KernelError("cos_sin table does not match rot_dim")
            n_pos = table.shape[0]
        if T > 65535:
            raise KernelError("attention_decode_ring with the position encoding inside takes at most 65535 tokens")
        _check(load().illm_attention_decode_ring_rope(
            None if partials is not None else _ptr(qkv),
            _ptr(partials.ws) if partials is not None else None,
            partials.splits if partials is not None else 0,
            T * width if partials is not None else 0,
            _ptr(table) if rot_dim else None, int(rot_dim), n_pos, 1 if write_kv else 0, _ptr(k_cache), _ptr(v_cache),
            k_cache.shape[0], _ptr(block_table), block_table.shape[1], _ptr(token_pos[t0:t1]), _ptr(token_seq[t0:t1]),
            _ptr(part_acc), _ptr(part_ml), _ptr(out[t0:t1]), t1 - t0, n_heads, n_kv_heads, head_dim, page_size,
            int(window or 0), float(scale), n, _ptr(tc_error_word(out.device)), _ptr(step_err), _stream()),
            "attention_decode_ring_rope")
    return out


def attention_prefill_supported(dtype, n_heads, n_kv_heads, head_dim) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % n_kv_heads == 0


def attention_prefill(qkv, k_cache, v_cache, block_table, cu_q, seq_lens, max_q, n_heads, n_kv_heads,
                      head_dim, page_size, window, scale):
    """bfloat16 tensor-core attention of whole prompts (or chunks that continue a sequence).
    `cu_q` int32 [B+1]: token offsets of the sequences in the step; `seq_lens` int32 [B]: their
    lengths after the step; `max_q`: the most tokens one sequence brings."""
    _need(qkv, "qkv", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    T, B = qkv.shape[0], seq_lens.numel()
    out = _rows(T, n_heads * head_dim, torch.bfloat16, qkv.device)
    _check(load().illm_attention_prefill(
        _ptr(qkv), qkv.shape[1], _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(cu_q), _ptr(seq_lens), _ptr(out), B, int(max_q), n_heads, n_kv_heads, head_dim, page_size,
        int(window or 0), float(scale), _stream()), "attention_prefill")
    return out


def attention_prefill_tc_supported(dtype, n_heads, n_kv_heads, head_dim, page_size) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % n_kv_heads == 0
            and page_size % 64 == 0)


def attention_prefill_tc(qkv, k_cache, v_cache, block_table, cu_q, seq_lens, max_q, n_heads, n_kv_heads,
                         head_dim, page_size, window, scale):
    """The tcgen05 / TMA version of `attention_prefill` (head size 64 or 128, pages of a
    multiple of 64 positions)."""
    _need(qkv, "qkv", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    T, B = qkv.shape[0], seq_lens.numel()
    out = _rows(T, n_heads * head_dim, torch.bfloat16, qkv.device)
    _check(load().illm_attention_prefill_tc(
        _ptr(qkv), qkv.shape[1], T, _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(block_table),
        block_table.shape[1], _ptr(cu_q), _ptr(seq_lens), _ptr(out), B, int(max_q), n_heads, n_kv_heads,
        head_dim, page_size, int(window or 0), float(scale), _ptr(tc_error_word(qkv.device)), _stream()),
        "attention_prefill_tc")
    return out


def attention(qkv, kv, ctx, n_heads, n_kv_heads, head_dim, window, scale):
    """Attention of the step's tokens over the cache entry `kv` (a KVView): picks the kernel
    for the dtype, head size and kind of step."""
    group = n_heads // n_kv_heads if n_kv_heads else 0
    # grids and scratch of the decode kernels are sized for the longest sequence the cache allows,
    # so that the launch is the same at every step
    if ctx.is_decode and attention_decode_ring_supported(qkv.dtype, n_heads, n_kv_heads, head_dim, kv.page_size):
        return attention_decode_ring(qkv, kv.k, kv.v, kv.block_table, ctx.token_pos, ctx.token_seq,
                                     n_heads, n_kv_heads, head_dim, kv.page_size, window, scale,
                                     ctx.max_seq_len)
    if ctx.is_decode and (group >= GQA_DECODE_MIN_GROUP or not attention_decode_supported(
            qkv.dtype, n_heads, n_kv_heads, head_dim, kv.page_size)) and attention_decode_gqa_supported(
            qkv.dtype, n_heads, n_kv_heads, head_dim):
        return attention_decode_gqa(qkv, kv.k, kv.v, kv.block_table, ctx.token_pos, ctx.token_seq,
                                    n_heads, n_kv_heads, head_dim, kv.page_size, window, scale,
                                    ctx.max_seq_len)
    if ctx.is_decode and attention_decode_supported(qkv.dtype, n_heads, n_kv_heads, head_dim, kv.page_size):
        return attention_decode(qkv, kv.k, kv.v, kv.block_table, ctx.token_pos, ctx.token_seq,
                                n_heads, n_kv_heads, head_dim, kv.page_size, window, scale,
                                ctx.max_seq_len)
    if not ctx.is_decode and attention_prefill_tc_supported(qkv.dtype, n_heads, n_kv_heads, head_dim,
                                                            kv.page_size):
        return attention_prefill_tc(qkv, kv.k, kv.v, kv.block_table, ctx.cu_q, ctx.seq_lens, ctx.max_q,
                                    n_heads, n_kv_heads, head_dim, kv.page_size, window, scale)
    if not ctx.is_decode and attention_prefill_supported(qkv.dtype, n_heads, n_kv_heads, head_dim):
        return attention_prefill(qkv, kv.k, kv.v, kv.block_table, ctx.cu_q, ctx.seq_lens, ctx.max_q,
                                 n_heads, n_kv_heads, head_dim, kv.page_size, window, scale)
    return attention_generic(qkv, kv.k, kv.v, kv.block_table, ctx.token_pos, ctx.token_seq,
                             n_heads, n_kv_heads, head_dim, kv.page_size, window, scale)


def gemm_f32(x, w):
    """float32 x [M, K] . w [N, K]^T -> [M, N] with float32 FMA accumulation."""
    _need(x, "x", torch.float32, 2)
    _need(w, "w", torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is {tuple(w.shape)}")
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    for m0 in range(0, M, 65535 * 64):
        m1 = min(M, m0 + 65535 * 64)
        _check(load().illm_gemm_f32_nt(_ptr(x[m0:m1]), _ptr(w), _ptr(out[m0:m1]), m1 - m0, N, K, K, K,
                                       N, _ptr(tc_error_word(x.device)), _stream()), "gemm_f32")
    return out


def n_sms_of_device() -> int:
    """Multiprocessors of the current device (148 without one: what the CPU tests of the policies use)."""
    if not torch.cuda.is_available():
        return 148
    n, tc, st = ctypes.c_int(), ctypes.c_void_p(), ctypes.c_void_p()
    _b.lib().illm_test_device_info(_info_device(), ctypes.byref(n), ctypes.byref(tc), ctypes.byref(st))
    return n.value


def tc_error_word(device=None):
    """The error word of the tensor-core kernels' bounded waits, of the library's device context for
    calls outside an engine: an int32 tensor [1] that views it."""
    from ..engine import device_view
    n, tc, st = ctypes.c_int(), ctypes.c_void_p(), ctypes.c_void_p()
    _b.lib().illm_test_device_info(_info_device(), ctypes.byref(n), ctypes.byref(tc), ctypes.byref(st))
    return device_view(tc.value, (1,), torch.int32, torch.cuda.current_device())


class SplitKPartials:
    """The K slices of a split matrix product that have not been added up yet: float32
    [splits, M, N].  `add_rmsnorm` and `rope_kv_write` take it in place of the finished tensor
    and do the addition themselves (ascending order of the slice, as the stand-alone reduction
    does), which saves a kernel per product in a decode step; `materialize` is for everyone else."""

    def __init__(self, ws: torch.Tensor):
        self.ws = ws
        self.splits, self.rows, self.cols = ws.shape
        self.shape = (self.rows, self.cols)
        self.device = ws.device

    def materialize(self, dtype=torch.bfloat16) -> torch.Tensor:
        out = torch.empty(self.shape, dtype=dtype, device=self.device)
        _check(load().illm_splitk_reduce(_ptr(self.ws), _ptr(out), act_code(dtype), self.rows * self.cols,
                                         self.splits, _stream()), "splitk_reduce")
        return out


def gemm_tc_splits(M, N, K, n_sms=None):
    """How many slices of K a decode-sized product (M <= 64) is cut into: the engine's policy
    (`ops::gemm_tc_splits`)."""
    return int(_b.lib().illm_policy_gemm_tc_splits(int(M), int(N), int(K), int(n_sms or n_sms_of_device())))


def gemm_bf16_tc(x, w, out_dtype=torch.bfloat16, splits=None, defer_reduce=False):
    """bfloat16 x [M, K] . w [N, K]^T on tcgen05 tensor cores, float32 accumulation.
    `defer_reduce`: if the product is split over K, return its slices as `SplitKPartials`
    instead of adding them up."""
    _need(x, "x", torch.bfloat16, 2)
    _need(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is {tuple(w.shape)}")
    if K % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        raise KernelError(f"gemm_bf16_tc: K = {K} must be a multiple of 8 and the operands 16-byte aligned")
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if splits is None:
        splits = gemm_tc_splits(M, N, K)
    else:
        k_iters = -(-K // 64)
        splits = max(1, min(int(splits), k_iters))
        splits = -(-k_iters // -(-k_iters // splits))
    if M > 64:
        splits = 1
    ws = torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None
    defer = bool(defer_reduce and splits > 1)
    _check(load().illm_gemm_bf16_tc(_ptr(x), _ptr(w), _ptr(out), act_code(out_dtype), M, N, K, _ptr(ws),
                                    splits, _ptr(tc_error_word(x.device)), _stream(), 1 if defer else 0),
           "gemm_bf16_tc")
    return SplitKPartials(ws) if defer else out


def gemm_bf16_tc_gated(x, w):
    """silu(gate) * up of bfloat16 x [M <= 64, K] . w [2I, K]^T (rows 2i, 2i + 1: gate and up of output
    i) -> [M, I] bfloat16, the activation applied to the accumulators (no split of K)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or N % 2 or M > 64 or K % 8:
        raise KernelError(f"gemm_bf16_tc_gated: x {tuple(x.shape)}, w {tuple(w.shape)}: at most 64 rows, K a multiple of 8, "
                          "an even number of weight rows")
    out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    _check(load().illm_gemm_bf16_tc_gated(_ptr(x), _ptr(w), _ptr(out), M, N, K, _ptr(tc_error_word(x.device)), _stream()),
           "gemm_bf16_tc_gated")
    return out


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch of the package's kernels (on by default)."""
    _b.lib().illm_set_pdl_enabled(1 if on else 0)


def gemm_bf16_tc2(x, w, out_dtype=torch.bfloat16, gated=False):
    """bfloat16 x [M, K] . w [N, K]^T on pairs of SMs (tcgen05 cta_group::2), for prompts.
    `gated`: w's rows 2i, 2i + 1 are the gate and the up row of output i and the result is
    silu(gate) * up, [M, N / 2]."""
    _need(x, "x", torch.bfloat16, 2)
    _need(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is {tuple(w.shape)}")
    if K % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or (gated and N % 2):
        raise KernelError(f"gemm_bf16_tc2: K = {K} must be a multiple of 8, the operands 16-byte aligned"
                          " and a gated weight an even number of rows")
    out = _rows(M, N // 2 if gated else N, out_dtype, x.device)
    _check(load().illm_gemm_bf16_tc2(_ptr(x), _ptr(w), _ptr(out), act_code(out_dtype), 1 if gated else 0, M, N, K,
                                     _ptr(tc_error_word(x.device)), _stream()), "gemm_bf16_tc2")
    return out


_GEMM_BACKEND = "auto"


def gemm_backend() -> str:
    return _GEMM_BACKEND


def set_gemm_backend(name: str) -> None:
    """Which kernels `linear` and `linear_gated` of this module ask for when no `backend` is given:
    "auto" | "tc" | "library" (see `ops::GemmBackend`; an engine has its own setting)."""
    global _GEMM_BACKEND
    if name not in ("tc", "library", "auto"):
        raise ValueError("gemm backend must be 'tc', 'library' or 'auto'")
    _GEMM_BACKEND = name


def linear(x, w, out_dtype=None, defer_reduce=False, backend=None):
    """x [M, K] . w [N, K]^T by the kernel the engine picks for these sizes (`ops::linear`).
    `defer_reduce=True` allows the result to come back as `SplitKPartials`."""
    _need(x, "x", None, 2)
    _need(w, "w", x.dtype, 2)
    out_dtype = out_dtype or x.dtype
    dev = _test_device()
    _b.check(_b.lib().illm_test_device_rewind(dev))
    out, ws, splits = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int()
    M, N = x.shape[0], w.shape[0]
    _b.check(_b.lib().illm_op_linear(dev, (backend or _GEMM_BACKEND).encode(), x.data_ptr(), M, x.shape[1], w.data_ptr(), N,
                                     act_code(x.dtype), act_code(out_dtype), 1 if defer_reduce else 0, ctypes.byref(out),
                                     ctypes.byref(ws), ctypes.byref(splits)))
    if ws.value:
        return SplitKPartials(_take(dev, ws, (splits.value, M, N), torch.float32, x.device))
    return _take(dev, out, (M, N), out_dtype, x.device)


def argmax(logits):
    """float32 [B, V] -> int32 [B], the lowest id among equal maxima (two passes: chunks of 2048
    elements, then the chunks' results)."""
    _need(logits, "logits", torch.float32, 2)
    B, V = logits.shape
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    n_chunks = -(-V // 2048)
    for b0 in range(0, B, 65535):
        b1 = min(B, b0 + 65535)
        sv = torch.empty((b1 - b0, n_chunks), dtype=torch.float32, device=logits.device)
        si = torch.empty((b1 - b0, n_chunks), dtype=torch.int32, device=logits.device)
        _check(load().illm_argmax(_ptr(logits[b0:b1]), b1 - b0, V, V, _ptr(out[b0:b1]), _ptr(sv), _ptr(si),
                                  _stream()), "argmax")
    return out


def sample(logits, uniforms, temp, top_k=0, top_p=1.0, repeat_penalty=1.0, last_tokens=None):
    """Temperature / repetition penalty / top-k / top-p sampling, one draw per row.
    `uniforms` float32 [B] in [0, 1); `last_tokens` int32 [B, n] (-1 pads) or None."""
    _need(logits, "logits", torch.float32, 2)
    _need(uniforms, "uniforms", torch.float32, 1)
    B, V = logits.shape
    if uniforms.numel() != B:
        raise KernelError("sample: one uniform number per row is needed")
    n_last = 0
    if last_tokens is not None:
        _need(last_tokens, "last_tokens", torch.int32, 2)
        n_last = last_tokens.shape[1]
    z = torch.empty((B, V), dtype=torch.float32, device=logits.device)
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    for b0 in range(0, B, 65535):
        b1 = min(B, b0 + 65535)
        # temperature alone and top_k <= 64 run in two passes over chunks of the row and need scratch
        n_scratch = int(load().illm_sample_scratch_elems(b1 - b0, V, int(top_k), float(top_p)))
        scratch = torch.empty((n_scratch,), dtype=torch.int32, device=logits.device) if n_scratch else None
        _check(load().illm_sample(_ptr(logits[b0:b1]), b1 - b0, V, V, _ptr(z[b0:b1]),
                                  _ptr(last_tokens[b0:b1]) if last_tokens is not None else None, n_last, float(temp),
                                  float(repeat_penalty), int(top_k), float(top_p), _ptr(uniforms[b0:b1]),
                                  _ptr(out[b0:b1]), _ptr(scratch), _stream()), "sample")
    return out


def fill_random(out, key: int, std: float, mean: float = 0.0):
    """out[i] = mean + std * z_i, z_i value i of the stream `key` (`weights.random_init.random_key`);
    float32 or bfloat16, in place."""
    _need(out, "out")
    _check(load().illm_fill_random(_ptr(out), act_code(out.dtype), out.numel(), int(key), float(std), float(mean),
                                   _stream()), "fill_random")
    return out


def poison_pages(k, v, pages):
    """Fill the given pages (int32 tensor on the device) of the cache tensors k, v
    [entries, pages, kv heads, page_size, head_dim] with NaN, in every entry."""
    _need(k, "k", None, 5)
    _need(v, "v", k.dtype, 5)
    _need(pages, "pages", torch.int32, 1)
    page_bytes = k.shape[2] * k.shape[3] * k.shape[4] * k.element_size()
    _check(load().illm_poison_pages(_ptr(k), _ptr(v), k.shape[1] * page_bytes, k.shape[0], page_bytes, _ptr(pages),
                                    pages.numel(), _stream()), "poison_pages")


def selftest_wait_timeout(err=None, limit_clocks: int = 1 << 20, code: int = 4):
    """Runs the bounded mbarrier wait of the tensor-core kernels on a barrier nobody arrives at, with
    a short limit.  `err`: the int32 error word to raise (a tensor [1]; default the word of this
    module's own device context; `Engine.info()["tc_error_word"]` is an engine's).  Returns (error word,
    1 if the wait reported its time-out, clocks waited); the word is left set."""
    if err is None:
        err = tc_error_word()
    result = torch.zeros(2, dtype=torch.int64, device=err.device)
    _check(load().illm_selftest_wait_timeout(_ptr(err), _ptr(result), int(limit_clocks), int(code), _stream()),
           "selftest_wait_timeout")
    r = result.tolist()
    return int(err.item()), int(r[0]), int(r[1])

