"""The decode-attention entry point that brings its own scratch memory (GPU).

Some callers of the kernel library cannot allocate on the device (all memory already given to
their own pool, a real-time loop, an open stream capture).  For them the library exports
`illm_attention_decode_static`, which keeps its partial results in an array inside the library
instead of caller-provided scratch.  This test calls it through the exported C symbol, twice in
a row with different batches (the array keeps the first call's leftovers), and compares with the
regular entry point and with a plain attention written out in the test.  This file sorts last on purpose: a run that stops at the first failure has
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
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()           # the driver's figure: it sees every cudaMalloc of the process
    rc = fn(qkv.data_ptr(), qkv.shape[1], kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.shape[1],
            pos.data_ptr(), seq.data_ptr(), out.data_ptr(), T, nh, nkv, d, page, window, scale, max_len,
            msg, len(msg), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    # the call took no device memory: neither from the driver nor (it has no other source) from torch
    assert free_after >= free_before, f"{free_before - free_after} bytes of device memory went away during the call"
    return rc, out, msg.value.decode()


def _plain_rows(qkv, kc, vc, table, lens, nh, nkv, d, page, window, scale, which):
    """Attention of the last token of the sequences `which`, written out in float64."""
    out = {}
    g = nh // nkv
    for b in which:
        n = lens[b]
        lo = max(0, n - window) if window else 0
        keys = torch.stack([kc[int(table[b, p // page]), :, p % page] for p in range(lo, n)]).double().cpu()
        vals = torch.stack([vc[int(table[b, p // page]), :, p % page] for p in range(lo, n)]).double().cpu()
        q = qkv[b, :nh * d].double().cpu().view(nh, d)
        rows = []
        for h in range(nh):
            s = (keys[:, h // g] @ q[h]) * scale
            p_ = torch.softmax(s, dim=0)
            rows.append(p_ @ vals[:, h // g])
        out[b] = torch.cat(rows)
    return out


def test_static_scratch_entry_point_matches_the_regular_one():
    from inferllm_b200.binding import lib as load
    from inferllm_b200.kernels import ops

    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = load().illm_attention_decode_static
    fn.argtypes = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, ctypes.c_char_p, I, P]
    fn.restype = I

    nh, nkv, d, page = 8, 2, 128, 16
    scale = 1.0 / math.sqrt(d)
    # two calls in a row with other batches and other numbers of key chunks (the array keeps what the
    # first call left), a window, and sequences that end exactly at max_len, on a chunk boundary
    for seed, lens, max_len, window in ((1, [700, 1, 256, 257, 1000, 1024], 1024, 0), (2, [3, 300], 512, 0),
                                        (4, [512, 100, 513, 2048], 2048, 300), (5, [256], 256, 0)):
        args = _case(seed, lens, nh, nkv, d, page)
        want = ops.attention_decode(*args, nh, nkv, d, page, window or None, scale, max_len)
        rc, got, msg = _call_static(fn, *args, nh, nkv, d, page, window, scale, max_len)
        assert rc == 0, msg
        torch.cuda.synchronize()
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 2 ** -7 * want.float().abs().max().item(), f"lens {lens}: max difference {diff}"
        qkv, kc, vc, table = args[0], args[1], args[2], args[3]
        for b, ref in _plain_rows(qkv, kc, vc, table.cpu(), lens, nh, nkv, d, page, window, scale, range(len(lens))).items():
            e = (got[b].double().cpu() - ref).abs().max().item()
            assert e <= 2 ** -7 * ref.abs().max().item(), f"lens {lens}, sequence {b}: {e} from the plain attention"

    # just under the array's size: 126 tokens x 32 heads x 16 chunks x (128 + 2) floats = 33,546,240 of
    # 33,554,432 bytes, so the second half of the layout (maxima and sums behind the partial outputs)
    # ends 8 KiB before the array does; a few long sequences among many short ones
    nh2, nkv2 = 32, 4
    lens = [int(x) for x in torch.randint(1, 200, (126,), generator=torch.Generator().manual_seed(9))]
    lens[0], lens[60], lens[125] = 4096, 3000, 4095
    args = _case(6, lens, nh2, nkv2, d, page)
    want = ops.attention_decode(*args, nh2, nkv2, d, page, None, scale, 4096)
    rc, got, msg = _call_static(fn, *args, nh2, nkv2, d, page, 0, scale, 4096)
    assert rc == 0, msg
    assert torch.equal(got, want), "the largest call that fits differs from the regular entry point"
    for b, ref in _plain_rows(args[0], args[1], args[2], args[3].cpu(), lens, nh2, nkv2, d, page, 0, scale,
                              (0, 60, 125, 7)).items():
        e = (got[b].double().cpu() - ref).abs().max().item()
        assert e <= 2 ** -7 * ref.abs().max().item(), f"sequence {b} of the largest call: {e} from the plain attention"

    # a call that needs more than the built-in array is refused with both sizes in the message
    args = _case(3, [5] * 64, 32, 32, 128, 16)
    rc, _, msg = _call_static(fn, *args, 32, 32, 128, 16, 0, scale, 8192)
    assert rc == 10002 and "33554432" in msg and "scratch" in msg
