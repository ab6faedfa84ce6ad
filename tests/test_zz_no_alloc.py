"""The decode-attention entry point that brings its own scratch memory (GPU).

Some callers of the kernel library cannot allocate on the device (all memory already given to
their own pool, a real-time loop, an open stream capture).  For them the library exports
`illm_attention_decode_static`, which keeps its partial results in an array inside the library
instead of caller-provided scratch.  This test calls it through the exported C symbol, twice in
a row with different batches (the array keeps the first call's leftovers), and compares with the
regular entry point.  This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, lens, nh, nkv, d, page):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lens) + 2
    width = max(-(-n // page) for n in lens)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    for b, n in enumerate(lens):
        for lp in range(-(-n // page)):
            table[b, lp] = order.pop()
    kc = torch.randn(n_pages, nkv, page, d, generator=g).bfloat16().cuda()
    vc = torch.randn(n_pages, nkv, page, d, generator=g).bfloat16().cuda()
    T = len(lens)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g).bfloat16().cuda()
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    seq = torch.arange(T, dtype=torch.int32).cuda()
    return qkv, kc, vc, table.cuda(), pos, seq


def _call_static(fn, qkv, kc, vc, table, pos, seq, nh, nkv, d, page, window, scale, max_len):
    T = qkv.shape[0]
    out = torch.zeros((T, nh * d), dtype=torch.bfloat16, device="cuda")
    msg = ctypes.create_string_buffer(512)
    allocations = torch.cuda.memory_stats()["allocation.all.allocated"]
    rc = fn(qkv.data_ptr(), qkv.shape[1], kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.shape[1],
            pos.data_ptr(), seq.data_ptr(), out.data_ptr(), T, nh, nkv, d, page, window, scale, max_len,
            msg, len(msg), torch.cuda.current_stream().cuda_stream)
    # the call itself took nothing from torch's allocator either (the library has no other)
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocations
    return rc, out, msg.value.decode()


def test_static_scratch_entry_point_matches_the_regular_one():
    from inferllm_b200.kernels import ops
    from inferllm_b200.kernels.lib import load

    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = load().illm_attention_decode_static
    fn.argtypes = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, ctypes.c_char_p, I, P]
    fn.restype = I

    nh, nkv, d, page = 8, 2, 128, 16
    scale = 1.0 / math.sqrt(d)
    for seed, lens, max_len in ((1, [700, 1, 256, 257, 1000], 1024), (2, [3, 300], 512)):
        args = _case(seed, lens, nh, nkv, d, page)
        want = ops.attention_decode(*args, nh, nkv, d, page, None, scale, max_len)
        rc, got, msg = _call_static(fn, *args, nh, nkv, d, page, 0, scale, max_len)
        assert rc == 0, msg
        torch.cuda.synchronize()
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 2 ** -7 * want.float().abs().max().item(), f"lens {lens}: max difference {diff}"

    # a call that needs more than the built-in array is refused with both sizes in the message
    args = _case(3, [5] * 64, 32, 32, 128, 16)
    rc, _, msg = _call_static(fn, *args, 32, 32, 128, 16, 0, scale, 8192)
    assert rc == 10002 and "33554432" in msg and "scratch" in msg
