"""Each CUDA kernel alone against its plain reference, at sizes other than the tiny models'
(GPU).  Inputs of the bfloat16 cases are bfloat16 values, so the reference sees the same
numbers and only the kernel's own rounding is left."""
import math

import numpy as np
import plain_llama as plain
import pytest
import torch

from inferllm_b200.kernels import ops

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(x, dtype=None):
    t = torch.as_tensor(x)
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda().contiguous()


def f64(t):
    return t.detach().double().cpu().numpy()


def maxrel(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def err_word():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def library_rope_table(d, rot, theta, positions):
    """The cos/sin table that the library's own rotate-half position encoding builds for these
    constants: float32 [positions, rot / 2, 2] (a copy)."""
    from inferllm_b200.config import PartSpec
    from inferllm_b200.engine import device_view
    from inferllm_b200.parts import PartSandbox
    sandbox = PartSandbox({}, "bfloat16")
    part = sandbox.build("position", PartSpec("rope_half", dict(head_dim=d, rot_dim=rot, theta=theta, max_positions=positions)))
    info = part.describe()
    assert info["rot_dim"] == rot and info["positions"] == positions and info["takes_partials"]
    return device_view(info["rotation_table"], (positions, rot // 2, 2), torch.float32).clone()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("V,H", [(50, 24), (1000, 4096), (333, 1001)])
def test_embedding(dtype, V, H):
    g = torch.Generator().manual_seed(V)
    table = torch.randn(V, H, generator=g).to(DT[dtype])
    ids = torch.randint(0, V, (37,), generator=g, dtype=torch.int32)
    err = err_word()
    out = ops.embedding(dev(ids), dev(table), err)
    assert out.dtype == torch.float32
    assert np.array_equal(f64(out), plain.embed(ids.numpy(), f64(table)))
    assert int(err.item()) == 0
    bad = ids.clone()
    bad[5] = V
    out = ops.embedding(dev(bad), dev(table), err)
    assert int(err.item()) == 1 and float(out[5].abs().max()) == 0.0


@pytest.mark.parametrize("dtype,wdtype", [("float32", "float32"), ("bfloat16", "bfloat16"),
                                          ("bfloat16", "float32")])
@pytest.mark.parametrize("T,H,eps", [(5, 64, 1e-5), (3, 4096, 1e-6), (17, 1000, 1e-3), (2, 11008, 1e-5)])
def test_add_rmsnorm(dtype, wdtype, T, H, eps):
    g = torch.Generator().manual_seed(H)
    resid = torch.randn(T, H, generator=g) * 3
    delta = (torch.randn(T, H, generator=g)).to(DT[dtype])
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(DT[wdtype])
    tol = 1e-6 if dtype == "float32" else 2 ** -8
    # plain norm
    r = dev(resid)
    y = ops.add_rmsnorm(r, None, dev(w), eps, DT[dtype])
    assert maxrel(f64(y), plain.rms_norm(f64(resid), f64(w), eps)) <= tol
    assert torch.equal(r.cpu(), resid)
    # add + norm, stream updated
    y = ops.add_rmsnorm(r, dev(delta), dev(w), eps, DT[dtype])
    x = f64(resid) + f64(delta)
    assert maxrel(f64(y), plain.rms_norm(x, f64(w), eps)) <= tol
    assert maxrel(f64(r), x) <= 1e-7
    # gathered rows, stream untouched
    rows = torch.tensor([T - 1, 0], dtype=torch.int32)
    r2 = dev(resid)
    y = ops.add_rmsnorm(r2, dev(delta), dev(w), eps, DT[dtype], rows=dev(rows), write_resid=False)
    assert y.shape == (2, H)
    assert maxrel(f64(y), plain.rms_norm(x[[T - 1, 0]], f64(w), eps)) <= tol
    assert torch.equal(r2.cpu(), resid)
    ops.residual_add(r2, dev(delta))
    assert maxrel(f64(r2), x) <= 1e-7


def test_rmsnorm_refuses_rows_wider_than_a_block_can_hold():
    with pytest.raises(ops.KernelError, match="width"):
        ops.add_rmsnorm(torch.zeros(1, 60000, device="cuda"), None, torch.ones(60000, device="cuda"),
                        1e-5, torch.float32)


def test_operands_off_a_16_byte_boundary_are_refused():
    """Rows of a multiple of 16 bytes are read 16 bytes at a time: a view that starts elsewhere is
    refused before any kernel runs; rows of another width are read element by element and taken."""
    H = 64
    resid = torch.zeros(4 * H + 1, dtype=torch.float32, device="cuda")[1:].view(4, H)
    w = torch.ones(H, dtype=torch.float32, device="cuda")
    with pytest.raises(ops.KernelError, match="16-byte boundary"):
        ops.add_rmsnorm(resid, None, w, 1e-5, torch.float32)
    x = torch.randn(3 * 40 + 3, device="cuda")[3:].view(3, 40)
    with pytest.raises(ops.KernelError, match="16-byte boundary"):
        ops.gemm_f32(x, torch.randn(5, 40, device="cuda"))
    H = 50                                            # 200-byte rows: no 16-byte accesses, any start will do
    base = torch.randn(4 * H + 1, device="cuda")
    resid = base[1:].view(4, H)
    w = torch.randn(H, device="cuda")
    ref = plain.rms_norm(f64(resid), f64(w), 1e-5)
    got = ops.add_rmsnorm(resid, None, w, 1e-5, torch.float32)
    assert maxrel(f64(got), ref) < 1e-5
    x = torch.randn(3 * 37 + 1, device="cuda")[1:].view(3, 37)
    wt = torch.randn(6 * 37 + 1, device="cuda")[1:].view(6, 37)
    assert maxrel(f64(ops.gemm_f32(x, wt)), f64(x) @ f64(wt).T) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,I", [(1, 176), (9, 11008), (300, 100), (70000, 8)])
def test_swiglu(dtype, T, I):
    g = torch.Generator().manual_seed(I)
    gu = (torch.randn(T, 2 * I, generator=g) * 2).to(DT[dtype])
    out = ops.swiglu(dev(gu))
    x = f64(gu)
    ref = plain.silu(x[:, 0::2]) * x[:, 1::2]          # gate and up of an output are neighbours
    assert maxrel(f64(out), ref) <= (1e-6 if dtype == "float32" else 2 ** -8)


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 70, 18), (64, 64, 16), (65, 129, 100), (200, 33, 7),
                                   (8, 1000, 4096), (130, 50, 30)])
def test_gemm_f32(M, N, K):
    g = torch.Generator().manual_seed(M * N + K)
    x, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    out = ops.gemm_f32(dev(x), dev(w))
    assert maxrel(f64(out), plain.linear(f64(x), f64(w))) <= 1e-6 * math.sqrt(K)


def test_gemm_f32_is_true_float32_and_row_invariant():
    """Values that a reduced-precision product would lose, and the same bits for a row whatever
    else is in the matrix."""
    K = 512
    x = torch.full((70, K), 1.0)
    x[:, 0] = 1.0 + 2.0 ** -20        # lost by tf32 (10 bits) and by bfloat16 operands
    w = torch.zeros(3, K)
    w[:, 0] = 1.0
    out = ops.gemm_f32(dev(x), dev(w)).cpu()
    assert float(out[0, 0]) == 1.0 + 2.0 ** -20
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(133, 300, generator=g), torch.randn(77, 300, generator=g)
    full = ops.gemm_f32(dev(x), dev(w)).cpu()
    for r in (0, 64, 132):
        one = ops.gemm_f32(dev(x[r:r + 1]), dev(w)).cpu()
        assert torch.equal(one[0], full[r])


@pytest.mark.parametrize("M,N,K", [(5, 96, 64), (2048, 300, 128), (1, 1000, 4096)])
def test_linear_bf16(M, N, K):
    g = torch.Generator().manual_seed(K)
    x, w = torch.randn(M, K, generator=g).bfloat16(), torch.randn(N, K, generator=g).bfloat16()
    ref = plain.linear(f64(x), f64(w))
    out32 = ops.linear(dev(x), dev(w), out_dtype=torch.float32)
    assert out32.dtype == torch.float32 and maxrel(f64(out32), ref) <= 1e-5
    out = ops.linear(dev(x), dev(w))
    assert out.dtype == torch.bfloat16 and maxrel(f64(out), ref) <= 2 ** -8


@pytest.mark.parametrize("M,N,K", [
    (1, 128, 64), (8, 4096, 4096), (3, 200, 72), (16, 130, 512), (17, 384, 1000), (64, 1000, 320),
    (65, 256, 64), (128, 256, 128), (300, 520, 328), (2048, 777, 200), (130, 100, 4096), (1, 32000, 256)])
@pytest.mark.parametrize("out", ["bfloat16", "float32"])
def test_gemm_bf16_tc(M, N, K, out):
    """The tcgen05 product: token counts on both sides of the decode/prompt switch, sizes that
    are no multiple of any tile, K with a ragged last slice, split K."""
    g = torch.Generator().manual_seed(M + N + K)
    x, w = torch.randn(M, K, generator=g).bfloat16(), torch.randn(N, K, generator=g).bfloat16()
    got = ops.gemm_bf16_tc(dev(x), dev(w), DT[out])
    assert got.dtype == DT[out] and tuple(got.shape) == (M, N)
    ref = plain.linear(f64(x), f64(w))
    assert maxrel(f64(got), ref) <= (2e-6 * math.sqrt(K) if out == "float32" else 2 ** -8)
    assert int(ops.tc_error_word(got.device).item()) == 0


@pytest.mark.parametrize("M,N,K", [(129, 256, 64), (256, 512, 128), (300, 520, 328), (2048, 1000, 200),
                                   (1000, 4096, 4096), (65, 300, 72)])
@pytest.mark.parametrize("out", ["bfloat16", "float32"])
def test_gemm_bf16_tc2(M, N, K, out):
    """The product on pairs of SMs: ragged token tiles, weight rows that are no multiple of the
    tile or of its halves, a ragged last slice of K, more tiles than SM pairs."""
    g = torch.Generator().manual_seed(M + N + K)
    x, w = torch.randn(M, K, generator=g).bfloat16(), torch.randn(N, K, generator=g).bfloat16()
    got = ops.gemm_bf16_tc2(dev(x), dev(w), DT[out])
    assert got.dtype == DT[out] and tuple(got.shape) == (M, N)
    assert int(ops.tc_error_word(got.device).item()) == 0
    ref = plain.linear(f64(x), f64(w))
    assert maxrel(f64(got), ref) <= (2e-6 * math.sqrt(K) if out == "float32" else 2 ** -8)


@pytest.mark.parametrize("M,I,K", [(300, 128, 64), (2048, 640, 328), (130, 11008, 256), (129, 100, 72)])
def test_gemm_bf16_tc2_gated(M, I, K):
    """Gate and up rows in turn: the epilogue of the SM-pair kernel applies silu(gate) * up."""
    g = torch.Generator().manual_seed(I)
    x = torch.randn(M, K, generator=g).bfloat16()
    wg, wu = (torch.randn(I, K, generator=g) * 0.1).bfloat16(), (torch.randn(I, K, generator=g) * 0.1).bfloat16()
    packed = torch.stack((wg, wu), dim=1).reshape(2 * I, K)
    got = ops.gemm_bf16_tc2(dev(x), dev(packed), torch.bfloat16, gated=True)
    assert tuple(got.shape) == (M, I) and int(ops.tc_error_word(got.device).item()) == 0
    ref = plain.silu(plain.linear(f64(x), f64(wg))) * plain.linear(f64(x), f64(wu))
    assert maxrel(f64(got), ref) <= 2 ** -7


@pytest.mark.parametrize("M,I,K", [(1, 128, 64), (8, 11008, 4096), (3, 100, 72), (16, 65, 512), (17, 300, 1000),
                                   (64, 500, 320), (40, 1000, 2048)])
def test_linear_gated(M, I, K):
    """The packed gate/up product with the activation: as the epilogue of the decode-sized tcgen05
    kernel where K is not split, through the slices where it is, after the library product
    otherwise; all give silu(x Wg^T) * (x Wu^T)."""
    g = torch.Generator().manual_seed(I + M)
    x = torch.randn(M, K, generator=g).bfloat16()
    wg, wu = (torch.randn(I, K, generator=g) * 0.1).bfloat16(), (torch.randn(I, K, generator=g) * 0.1).bfloat16()
    packed = dev(torch.stack((wg, wu), dim=1).reshape(2 * I, K))
    ref = plain.silu(plain.linear(f64(x), f64(wg))) * plain.linear(f64(x), f64(wu))
    try:
        for backend in ("tc", "library", "auto"):
            ops.set_gemm_backend(backend)
            got = ops.linear_gated(dev(x), packed)
            assert tuple(got.shape) == (M, I) and int(ops.tc_error_word(got.device).item()) == 0
            assert maxrel(f64(got), ref) <= 2 ** -7, backend
    finally:
        ops.set_gemm_backend("auto")


def test_gemm_bf16_tc_rows_do_not_depend_on_the_batch():
    g = torch.Generator().manual_seed(1)
    x, w = torch.randn(40, 1024, generator=g).bfloat16(), torch.randn(512, 1024, generator=g).bfloat16()
    full = ops.gemm_bf16_tc(dev(x), dev(w), torch.float32).cpu()
    one = ops.gemm_bf16_tc(dev(x[7:8]), dev(w), torch.float32).cpu()
    # same split of K and same order of accumulation whatever the number of tokens up to 64
    assert torch.equal(one[0], full[7])
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.gemm_bf16_tc(dev(x[:, :1020]), dev(w[:, :1020]))


def test_unreduced_split_k_slices_feed_norm_and_rope():
    """A decode-sized product may hand its K slices on unreduced: the norm and the rotation kernel
    add them up themselves and must give what the finished tensor gives."""
    g = torch.Generator().manual_seed(2)
    M, H = 5, 1024
    x, w = torch.randn(M, 4096, generator=g).bfloat16(), (torch.randn(H, 4096, generator=g) * 0.05).bfloat16()
    part = ops.gemm_bf16_tc(dev(x), dev(w), defer_reduce=True)
    assert isinstance(part, ops.SplitKPartials) and part.splits > 1 and part.shape == (M, H)
    full = ops.gemm_bf16_tc(dev(x), dev(w), torch.float32)
    assert torch.equal(part.materialize(torch.float32), full)      # same slices, same order
    assert maxrel(f64(full), plain.linear(f64(x), f64(w))) <= 1e-4
    resid = torch.randn(M, H, generator=g)
    wn = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    r1, r2 = dev(resid), dev(resid)
    y1 = ops.add_rmsnorm(r1, part, dev(wn), 1e-5, torch.bfloat16)
    ref_x = f64(resid) + f64(full)
    assert maxrel(f64(r1), ref_x) <= 1e-6 and maxrel(f64(y1), plain.rms_norm(ref_x, f64(wn), 1e-5)) <= 2 ** -8
    rows = torch.tensor([4, 1], dtype=torch.int32)
    y2 = ops.add_rmsnorm(r2, part, dev(wn), 1e-5, torch.bfloat16, rows=dev(rows), write_resid=False)
    assert torch.equal(r2.cpu(), resid) and maxrel(f64(y2), plain.rms_norm(ref_x[[4, 1]], f64(wn), 1e-5)) <= 2 ** -8
    r3 = dev(resid)
    ops.residual_add(r3, part)
    assert maxrel(f64(r3), ref_x) <= 2 ** -8 * np.abs(f64(full)).max()
    # the gated activation takes slices too
    wg = (torch.randn(512, 4096, generator=g) * 0.05).bfloat16()
    pg = ops.gemm_bf16_tc(dev(x), dev(wg), defer_reduce=True, splits=4)
    fg = f64(pg.materialize(torch.float32))
    assert maxrel(f64(ops.swiglu(pg)), plain.silu(fg[:, 0::2]) * fg[:, 1::2]) <= 2 ** -7
    # the packed projection of an attention layer: 3 heads + 2 x 1 kv heads of 64 channels
    nh, nkv, d, page = 3, 1, 64, 16
    wq = (torch.randn((nh + 2 * nkv) * d, 4096, generator=g) * 0.05).bfloat16()
    part = ops.gemm_bf16_tc(dev(x), dev(wq), defer_reduce=True, splits=4)
    qkv_full = part.materialize(torch.float32)
    rope_table = library_rope_table(d, d, 1e4, 64)
    kc = torch.zeros(4, nkv, page, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    table = torch.tensor([[2, 0]], dtype=torch.int32).cuda()
    pos = torch.tensor([3, 4, 5, 16, 17], dtype=torch.int32).cuda()
    seq = torch.zeros(M, dtype=torch.int32).cuda()
    out = ops.rope_kv_write(part, rope_table, d, pos, seq, table, kc, vc, nh, nkv, d, page, True, err_word())
    src = f64(qkv_full).reshape(M, nh + 2 * nkv, d)
    want = plain.rope_rotate_half(src[:, :nh + nkv], pos.cpu().numpy(), 1e4)
    assert maxrel(f64(out).reshape(M, nh + 2 * nkv, d)[:, :nh], want[:, :nh]) <= 2 ** -8
    for i, p_ in enumerate(pos.tolist()):
        pg = int(table[0, p_ // page])
        assert maxrel(f64(kc)[pg, :, p_ % page], want[i, nh:]) <= 2 ** -8
        assert maxrel(f64(vc)[pg, :, p_ % page], src[i, nh + nkv:]) <= 2 ** -8
    # a rotation over the first 32 of the 64 channels only: the other channels of Q and K are the sums
    # of the slices, unrotated
    rot = 32
    rope32_table = library_rope_table(d, rot, 1e4, 64)
    kc.zero_()
    vc.zero_()
    out = ops.rope_kv_write(part, rope32_table, rot, pos, seq, table, kc, vc, nh, nkv, d, page, True, err_word())
    want = plain.rope_rotate_half(src[:, :nh + nkv], pos.cpu().numpy(), 1e4, rot_dim=rot)
    assert maxrel(f64(out).reshape(M, nh + 2 * nkv, d)[:, :nh], want[:, :nh]) <= 2 ** -8
    for i, p_ in enumerate(pos.tolist()):
        pg = int(table[0, p_ // page])
        assert maxrel(f64(kc)[pg, :, p_ % page], want[i, nh:]) <= 2 ** -8


# ---- rope + cache write, attention: a hand-made paged cache


class Paged:
    """Sequences of given lengths in a paged cache whose pages are dealt out in a shuffled
    order; K and V of every position are known, so the plain reference can run on them."""

    def __init__(self, lens, nkv, d, page, dtype, seed=0, spare_pages=3):
        g = torch.Generator().manual_seed(seed)
        self.lens, self.nkv, self.d, self.page = lens, nkv, d, page
        self.width = max(-(-n // page) for n in lens) + 1
        n_pages = sum(-(-n // page) for n in lens) + spare_pages
        order = torch.randperm(n_pages, generator=g).tolist()
        self.table = torch.full((len(lens), self.width), -1, dtype=torch.int32)
        for b, n in enumerate(lens):
            for lp in range(-(-n // page)):
                self.table[b, lp] = order.pop()
        self.k = [torch.randn(n, nkv, d, generator=g).to(dtype) for n in lens]
        self.v = [torch.randn(n, nkv, d, generator=g).to(dtype) for n in lens]
        # unused places hold NaN: a kernel that reads beyond a sequence's keys shows it
        self.kc = torch.full((n_pages, nkv, page, d), float("nan"), dtype=dtype)
        self.vc = torch.full((n_pages, nkv, page, d), float("nan"), dtype=dtype)
        for b, n in enumerate(lens):
            for p in range(n):
                pg = int(self.table[b, p // page])
                self.kc[pg, :, p % page] = self.k[b][p]
                self.vc[pg, :, p % page] = self.v[b][p]


def plain_attention_rows(q, k, v, pos, nh, nkv, scale, window):
    """Plain attention of query rows at absolute positions `pos` over keys 0..len-1."""
    s = plain.attention_scores(q, k, nh, nkv)
    n_k = k.shape[0]
    t = np.arange(n_k)[None, :]
    hide = t > np.asarray(pos)[:, None]
    if window:
        hide |= t < np.asarray(pos)[:, None] - window + 1
    s = np.where(hide[None], -np.inf, s * scale)
    return plain.weighted_values(plain.softmax_rows(s), v, nh, nkv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (4, 4, 16, 8, None), (6, 2, 24, 16, None), (8, 1, 64, 64, None), (5, 5, 128, 32, None),
    (3, 1, 256, 16, None), (4, 2, 40, 8, 13), (2, 2, 128, 64, 64)])
def test_attention_generic(dtype, nh, nkv, d, page, window):
    lens = [1, 37, 130, 64]
    pc = Paged(lens, nkv, d, page, DT[dtype], seed=d)
    g = torch.Generator().manual_seed(7)
    # queries: all positions of sequence 1 (a prompt), the last of the others (decode), and
    # a mid-sequence chunk of sequence 2
    rows = [(1, p) for p in range(lens[1])] + [(0, 0), (2, 129), (3, 63)] + [(2, p) for p in range(60, 70)]
    T = len(rows)
    q = torch.randn(T, nh, d, generator=g).to(DT[dtype])
    qkv = torch.cat([q.reshape(T, nh * d), torch.zeros(T, 2 * nkv * d, dtype=DT[dtype])], dim=1)
    seq = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    pos = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    out = ops.attention_generic(dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(pos), dev(seq),
                                nh, nkv, d, page, window, scale)
    got = f64(out)
    assert np.isfinite(got).all()
    for b in range(len(lens)):
        idx = [i for i, r in enumerate(rows) if r[0] == b]
        ref = plain_attention_rows(f64(q[idx]), f64(pc.k[b]), f64(pc.v[b]), [rows[i][1] for i in idx],
                                   nh, nkv, scale, window)
        assert maxrel(got[idx], ref) <= (2e-6 if dtype == "float32" else 2 ** -7)


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (4, 4, 128, 64, None), (8, 2, 128, 16, None), (8, 1, 128, 64, None), (6, 2, 64, 8, None),
    (3, 3, 64, 64, None), (16, 2, 64, 32, None), (4, 2, 128, 64, 300), (2, 1, 64, 8, 5)])
def test_attention_decode(nh, nkv, d, page, window):
    """The split-key decode kernel: sequences that end inside the first chunk, exactly on a chunk
    border, and several chunks long."""
    lens = [1, 255, 256, 257, 700, 1024, 3]
    pc = Paged(lens, nkv, d, page, torch.bfloat16, seed=d + nh)
    g = torch.Generator().manual_seed(3)
    T = len(lens)
    q = torch.randn(T, nh, d, generator=g).bfloat16()
    qkv = torch.cat([q.reshape(T, nh * d), torch.zeros(T, 2 * nkv * d, dtype=torch.bfloat16)], dim=1)
    seq = torch.arange(T, dtype=torch.int32)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    assert ops.attention_decode_supported(torch.bfloat16, nh, nkv, d, page)
    for max_len in (1024, 4096):      # the grid's size must not change the result
        out = ops.attention_decode(dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(pos), dev(seq),
                                   nh, nkv, d, page, window, scale, max_len)
        got = f64(out)
        assert np.isfinite(got).all()
        for b in range(T):
            ref = plain_attention_rows(f64(q[b:b + 1]), f64(pc.k[b]), f64(pc.v[b]), [lens[b] - 1], nh, nkv, scale, window)
            assert maxrel(got[b:b + 1], ref) <= 2 ** -7, f"sequence of {lens[b]} keys"
    # a token's result does not depend on the rest of the batch
    alone = ops.attention_decode(dev(qkv[4:5]), dev(pc.kc), dev(pc.vc), dev(pc.table[4:5]), dev(pos[4:5]),
                                 dev(torch.zeros(1, dtype=torch.int32)), nh, nkv, d, page, window, scale, 4096)
    assert torch.equal(alone[0].cpu(), out[4].cpu())


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (2, 2, 128, 64, None), (6, 2, 128, 16, None), (4, 1, 64, 64, None), (3, 3, 64, 8, None),
    (4, 2, 128, 128, None), (2, 1, 64, 16, 70), (2, 2, 128, 64, 64), (2, 1, 128, 32, 1)])
def test_attention_prefill(nh, nkv, d, page, window):
    """The tensor-core prompt kernel: prompts from position 0 (shorter than a tile, exactly a
    tile, several tiles with a ragged end), a chunk that continues a sequence, a single token."""
    lens = [200, 64, 1, 333, 130, 65]
    starts = [0, 0, 0, 100, 129, 0]       # sequence 3 appends 233 tokens to 100 cached ones
    pc = Paged(lens, nkv, d, page, torch.bfloat16, seed=d + nh + page)
    g = torch.Generator().manual_seed(5)
    q_lens = [n - s for n, s in zip(lens, starts)]
    T = sum(q_lens)
    q = torch.randn(T, nh, d, generator=g).bfloat16()
    qkv = torch.cat([q.reshape(T, nh * d), torch.zeros(T, 2 * nkv * d, dtype=torch.bfloat16)], dim=1)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    out = ops.attention_prefill(dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(cu),
                                dev(torch.tensor(lens, dtype=torch.int32)), max(q_lens), nh, nkv, d, page,
                                window, scale)
    got = f64(out)
    assert np.isfinite(got).all()
    for b in range(len(lens)):
        rows = slice(int(cu[b]), int(cu[b + 1]))
        ref = plain_attention_rows(f64(q[rows]), f64(pc.k[b]), f64(pc.v[b]), list(range(starts[b], lens[b])),
                                   nh, nkv, scale, window)
        assert maxrel(got[rows], ref) <= 2 ** -7, f"sequence {b}"
    # the same tokens through the generic kernel agree as well
    seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(q_lens)).int()
    pos = torch.cat([torch.arange(s, n) for s, n in zip(starts, lens)]).int()
    gen = ops.attention_generic(dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(pos), dev(seq),
                                nh, nkv, d, page, window, scale)
    assert maxrel(got, f64(gen)) <= 2 ** -6


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (2, 2, 128, 64, None), (6, 2, 128, 128, None), (4, 1, 64, 64, None), (3, 3, 64, 128, None),
    (2, 1, 64, 64, 70), (2, 2, 128, 64, 64), (2, 1, 128, 64, 1), (4, 2, 128, 64, 200)])
def test_attention_prefill_tc(nh, nkv, d, page, window):
    """The tcgen05 prompt kernel: prompts shorter than a tile, exactly a tile, several tiles with
    a ragged end, a chunk that continues a sequence at an odd position, a single token.  The
    unused places of the cache hold NaN."""
    lens = [200, 128, 1, 333, 130, 65, 600]
    starts = [0, 0, 0, 100, 129, 0, 0]
    pc = Paged(lens, nkv, d, page, torch.bfloat16, seed=d + nh + page)
    g = torch.Generator().manual_seed(5)
    q_lens = [n - s for n, s in zip(lens, starts)]
    T = sum(q_lens)
    q = torch.randn(T, nh, d, generator=g).bfloat16()
    qkv = torch.cat([q.reshape(T, nh * d), torch.zeros(T, 2 * nkv * d, dtype=torch.bfloat16)], dim=1)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    assert ops.attention_prefill_tc_supported(torch.bfloat16, nh, nkv, d, page)
    out = ops.attention_prefill_tc(dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(cu),
                                   dev(torch.tensor(lens, dtype=torch.int32)), max(q_lens), nh, nkv, d, page,
                                   window, scale)
    got = f64(out)
    assert int(ops.tc_error_word(out.device).item()) == 0
    assert np.isfinite(got).all()
    for b in range(len(lens)):
        rows = slice(int(cu[b]), int(cu[b + 1]))
        ref = plain_attention_rows(f64(q[rows]), f64(pc.k[b]), f64(pc.v[b]), list(range(starts[b], lens[b])),
                                   nh, nkv, scale, window)
        assert maxrel(got[rows], ref) <= 2 ** -7, f"sequence {b}"
    # the same inputs evicted from the L2 cache: loads that take long must change nothing (a wait
    # that passes too early only shows when the data is late)
    args = (dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(cu), dev(torch.tensor(lens, dtype=torch.int32)))
    for _ in range(2):
        flush = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
        flush += 1
        torch.cuda.synchronize()
        cold = ops.attention_prefill_tc(*args, max(q_lens), nh, nkv, d, page, window, scale)
        assert torch.equal(cold.cpu(), out.cpu())


def test_attention_prefill_tc_finds_far_keys_and_respects_the_window_edge():
    nh = nkv = 1
    d, page, n = 128, 64, 600
    pc = Paged([n], nkv, d, page, torch.bfloat16, seed=4)
    cu, sl = dev(torch.tensor([0, n], dtype=torch.int32)), dev(torch.tensor([n], dtype=torch.int32))
    for window in (None, 200):
        for qrow, target in ((599, 2), (599, 399), (599, 400), (300, 101), (300, 100), (77, 77), (128, 127)):
            key = torch.randn(d, generator=torch.Generator().manual_seed(target))
            key = (key / key.norm() * 12).bfloat16()
            kc = pc.kc.clone()
            kc[int(pc.table[0, target // page]), 0, target % page] = key
            q = torch.zeros(n, d)
            q[qrow] = key.float() * 2
            qkv = torch.cat([q, torch.zeros(n, 2 * d)], dim=1).bfloat16()
            out = ops.attention_prefill_tc(dev(qkv), dev(kc), dev(pc.vc), dev(pc.table), cu, sl, n, 1, 1, d, page,
                                           window, 1.0)
            hit = maxrel(f64(out[qrow]), f64(pc.v[0][target]).reshape(-1)) <= 1e-2
            inside = target <= qrow and (window is None or target >= qrow - window + 1)
            assert hit == inside, (window, qrow, target)


def test_attention_prefill_finds_far_keys_and_respects_the_window_edge():
    nh = nkv = 1
    d, page, n = 64, 16, 600
    pc = Paged([n], nkv, d, page, torch.bfloat16, seed=4)
    cu, sl = dev(torch.tensor([0, n], dtype=torch.int32)), dev(torch.tensor([n], dtype=torch.int32))
    for window in (None, 200):
        for qrow, target in ((599, 2), (599, 399), (599, 400), (300, 101), (300, 100), (77, 77)):
            key = torch.randn(d, generator=torch.Generator().manual_seed(target))
            key = (key / key.norm() * 12).bfloat16()
            kc = pc.kc.clone()
            kc[int(pc.table[0, target // page]), 0, target % page] = key
            q = torch.zeros(n, d)
            q[qrow] = key.float() * 2
            qkv = torch.cat([q, torch.zeros(n, 2 * d)], dim=1).bfloat16()
            out = ops.attention_prefill(dev(qkv), dev(kc), dev(pc.vc), dev(pc.table), cu, sl, n, 1, 1, d, page,
                                        window, 1.0)
            hit = maxrel(f64(out[qrow]), f64(pc.v[0][target]).reshape(-1)) <= 1e-2
            inside = target <= qrow and (window is None or target >= qrow - window + 1)
            assert hit == inside, (window, qrow, target)


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (8, 2, 128, 64, None), (32, 8, 128, 16, None), (6, 2, 64, 8, None), (10, 2, 128, 64, None),
    (16, 1, 64, 32, None), (4, 2, 128, 4, 300), (12, 4, 64, 64, 5), (14, 2, 128, 64, None)])
def test_attention_decode_gqa(nh, nkv, d, page, window):
    """Grouped heads as rows of an MMA tile: group sizes 2..16 (also ones that are no power of
    two), any page size, sequences around the chunk borders."""
    lens = [1, 127, 128, 129, 700, 1024, 3]
    pc = Paged(lens, nkv, d, page, torch.bfloat16, seed=d + nh)
    g = torch.Generator().manual_seed(3)
    T = len(lens)
    q = torch.randn(T, nh, d, generator=g).bfloat16()
    qkv = torch.cat([q.reshape(T, nh * d), torch.zeros(T, 2 * nkv * d, dtype=torch.bfloat16)], dim=1)
    seq = torch.arange(T, dtype=torch.int32)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    assert ops.attention_decode_gqa_supported(torch.bfloat16, nh, nkv, d)
    for max_len in (1024, 4096):
        out = ops.attention_decode_gqa(dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(pos), dev(seq),
                                       nh, nkv, d, page, window, scale, max_len)
        got = f64(out)
        assert np.isfinite(got).all()
        for b in range(T):
            ref = plain_attention_rows(f64(q[b:b + 1]), f64(pc.k[b]), f64(pc.v[b]), [lens[b] - 1], nh, nkv, scale, window)
            assert maxrel(got[b:b + 1], ref) <= 2 ** -7, f"sequence of {lens[b]} keys"
    alone = ops.attention_decode_gqa(dev(qkv[4:5]), dev(pc.kc), dev(pc.vc), dev(pc.table[4:5]), dev(pos[4:5]),
                                     dev(torch.zeros(1, dtype=torch.int32)), nh, nkv, d, page, window, scale, 4096)
    assert torch.equal(alone[0].cpu(), out[4].cpu())


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (8, 2, 128, 64, None), (32, 8, 128, 128, None), (6, 2, 64, 64, None), (10, 2, 128, 64, None),
    (16, 1, 64, 192, None), (4, 4, 128, 64, 300), (12, 4, 64, 64, 5), (3, 3, 64, 128, None),
    (14, 2, 128, 64, 70)])
def test_attention_decode_ring(nh, nkv, d, page, window):
    """The streaming kernel: group sizes 1..16, sequences around the tile borders, every number of
    splits (blocks without keys, blocks with one tile, one block with all of them)."""
    lens = [1, 63, 64, 65, 700, 1024, 3, 129]
    pc = Paged(lens, nkv, d, page, torch.bfloat16, seed=d + nh)
    g = torch.Generator().manual_seed(3)
    T = len(lens)
    q = torch.randn(T, nh, d, generator=g).bfloat16()
    qkv = torch.cat([q.reshape(T, nh * d), torch.zeros(T, 2 * nkv * d, dtype=torch.bfloat16)], dim=1)
    seq = torch.arange(T, dtype=torch.int32)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    assert ops.attention_decode_ring_supported(torch.bfloat16, nh, nkv, d, page)
    refs = [plain_attention_rows(f64(q[b:b + 1]), f64(pc.k[b]), f64(pc.v[b]), [lens[b] - 1], nh, nkv, scale, window)
            for b in range(T)]
    for splits in (None, 1, 2, 3, 16):
        out = ops.attention_decode_ring(dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(pos), dev(seq),
                                        nh, nkv, d, page, window, scale, 4096, splits=splits)
        got = f64(out)
        assert np.isfinite(got).all()
        for b in range(T):
            assert maxrel(got[b:b + 1], refs[b]) <= 2 ** -7, f"sequence of {lens[b]} keys, {splits} splits"
    assert int(ops.tc_error_word(torch.device("cuda")).item()) == 0
    alone = ops.attention_decode_ring(dev(qkv[4:5]), dev(pc.kc), dev(pc.vc), dev(pc.table[4:5]), dev(pos[4:5]),
                                      dev(torch.zeros(1, dtype=torch.int32)), nh, nkv, d, page, window, scale, 4096,
                                      splits=16)
    assert torch.equal(alone[0].cpu(), out[4].cpu())
    # inputs evicted from the L2 cache: late data must change nothing
    args = (dev(qkv), dev(pc.kc), dev(pc.vc), dev(pc.table), dev(pos), dev(seq))
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
    flush += 1
    torch.cuda.synchronize()
    cold = ops.attention_decode_ring(*args, nh, nkv, d, page, window, scale, 4096, splits=16)
    assert torch.equal(cold.cpu(), out.cpu())


@pytest.mark.parametrize("nh,nkv,d,page,window,rot,slices", [
    (8, 2, 128, 64, None, 128, 3), (4, 4, 128, 64, None, 128, 1), (6, 2, 64, 64, 70, 64, 2), (3, 3, 64, 128, None, 32, 4),
    (16, 1, 64, 64, None, 0, 2), (32, 8, 128, 64, None, 128, 0)])
def test_attention_decode_ring_with_the_position_encoding_inside(nh, nkv, d, page, window, rot, slices):
    """The kernel that also rotates Q and the new K row and writes K and V into the cache, fed with
    the unrotated projection (bfloat16, or K slices of a split product), against the two kernels
    it replaces: the same attention output and the same cache contents, for every number of splits
    (the new row lies in another block's tile each time)."""
    lens = [1, 63, 64, 65, 700, 1024, 3, 129]
    T = len(lens)
    pc = Paged(lens, nkv, d, page, torch.bfloat16, seed=d + nh)
    g = torch.Generator().manual_seed(11)
    width = (nh + 2 * nkv) * d
    if slices:
        ws = torch.randn(slices, T, width, generator=g) * (1.0 / math.sqrt(slices))
        part = ops.SplitKPartials(dev(ws))
        qkv_bf16 = part.materialize(torch.bfloat16)
    else:
        qkv_bf16 = dev(torch.randn(T, width, generator=g).bfloat16())
    seq, pos = dev(torch.arange(T, dtype=torch.int32)), dev(torch.tensor([n - 1 for n in lens], dtype=torch.int32))
    scale = 1.0 / math.sqrt(d)
    table = None
    if rot:
        table = library_rope_table(d, rot, 1e4, 2048)
    # the two kernels: rotation and cache write (from the slices, as the engine would), then attention
    kc1, vc1 = dev(pc.kc), dev(pc.vc)
    src = ops.SplitKPartials(part.ws.clone()) if slices else qkv_bf16.clone()
    q1 = ops.rope_kv_write(src, table, rot, pos, seq, dev(pc.table), kc1, vc1, nh, nkv, d, page, True, err_word())
    want = ops.attention_decode_ring(q1, kc1, vc1, dev(pc.table), pos, seq, nh, nkv, d, page, window, scale, 4096)
    assert np.isfinite(f64(want)).all()
    # the plain implementation of the same: rotation of Q and of the new K row, the new row put behind
    # the sequence's cached keys and values, attention of the one query at the last position
    x = f64(qkv_bf16).reshape(T, nh + 2 * nkv, d)
    rotated = plain.rope_rotate_half(x[:, :nh + nkv], pos.cpu().numpy(), 1e4, rot_dim=rot) if rot else x[:, :nh + nkv]
    plain_rows = []
    for b in range(T):
        k, v = f64(pc.k[b]).copy(), f64(pc.v[b]).copy()
        k[-1], v[-1] = rotated[b, nh:], x[b, nh + nkv:]
        plain_rows.append(plain_attention_rows(rotated[b:b + 1, :nh], k, v, [lens[b] - 1], nh, nkv, scale, window))
    plain_rows = np.concatenate(plain_rows).reshape(T, nh * d)
    for splits in (None, 1, 2, 5, 16):
        kc2, vc2 = dev(pc.kc), dev(pc.vc)
        e = err_word()
        got = ops.attention_decode_ring(part if slices else qkv_bf16, kc2, vc2, dev(pc.table), pos, seq, nh, nkv, d, page,
                                        window, scale, 4096, splits=splits, rope=(table, rot, True, e))
        assert int(e.item()) == 0 and int(ops.tc_error_word(torch.device("cuda")).item()) == 0
        for b in range(T):
            pg, off = int(pc.table[b, (lens[b] - 1) // page]), (lens[b] - 1) % page
            assert torch.equal(kc2[pg, :, off], kc1[pg, :, off]) and torch.equal(vc2[pg, :, off], vc1[pg, :, off]), \
                f"cache row of sequence {b}, {splits} splits"
        assert maxrel(f64(got), f64(want)) <= 2 ** -9, f"{splits} splits"
        assert maxrel(f64(got), plain_rows) <= 2 ** -7, f"{splits} splits, against the plain implementation"
    # a layer that reads another layer's cache entry: nothing is written
    kc3, vc3 = kc1.clone(), vc1.clone()
    got = ops.attention_decode_ring(part if slices else qkv_bf16, kc3, vc3, dev(pc.table), pos, seq, nh, nkv, d, page,
                                    window, scale, 4096, rope=(table, rot, False, err_word()))
    assert torch.equal(kc3.view(torch.int16), kc1.view(torch.int16)) and maxrel(f64(got), f64(want)) <= 2 ** -9


def test_attention_decode_says_what_it_takes():
    assert not ops.attention_decode_supported(torch.float32, 4, 4, 128, 64)
    assert not ops.attention_decode_supported(torch.bfloat16, 4, 4, 24, 64)
    assert not ops.attention_decode_supported(torch.bfloat16, 5, 1, 128, 64)
    assert not ops.attention_decode_supported(torch.bfloat16, 4, 4, 128, 12)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """One key far back (first page) matches the query strongly: the output must be its value.
    A kernel that drops, misplaces or mis-masks far keys fails here although random data would
    average the fault away."""
    nh = nkv = 2
    d, page, n = 64, 16, 900
    pc = Paged([n], nkv, d, page, DT[dtype], seed=1)
    for target in (3, 15, 16, 447, 899):
        q = torch.zeros(1, nh, d)
        kc, vc = pc.kc.clone(), pc.vc.clone()
        key = torch.randn(d, generator=torch.Generator().manual_seed(target))
        key = (key / key.norm() * 12).to(DT[dtype])
        pg = int(pc.table[0, target // page])
        kc[pg, :, target % page] = key
        q[0, :] = key.float() * 2
        qkv = torch.cat([q.reshape(1, nh * d), torch.zeros(1, 2 * nkv * d)], dim=1).to(DT[dtype])
        out = ops.attention_generic(dev(qkv), dev(kc), dev(vc), dev(pc.table),
                                    dev(torch.tensor([n - 1], dtype=torch.int32)),
                                    dev(torch.zeros(1, dtype=torch.int32)), nh, nkv, d, page, None, 1.0)
        want = f64(pc.v[0][target]).reshape(-1)
        assert maxrel(f64(out).reshape(-1), want) <= 1e-2, f"key {target} was not found"
        if dtype == "bfloat16":
            out = ops.attention_decode(dev(qkv), dev(kc), dev(vc), dev(pc.table),
                                       dev(torch.tensor([n - 1], dtype=torch.int32)),
                                       dev(torch.zeros(1, dtype=torch.int32)), nh, nkv, d, page, None, 1.0, 1024)
            assert maxrel(f64(out).reshape(-1), want) <= 1e-2, f"decode kernel: key {target} was not found"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_window_edge(dtype):
    """The oldest key inside the window counts and the one before it does not."""
    nh = nkv = 1
    d, page, n, window = 32, 8, 100, 24
    pc = Paged([n], nkv, d, page, DT[dtype], seed=2)
    p = n - 1
    key = torch.ones(d) * 3
    for target, inside in ((p - window + 1, True), (p - window, False)):
        kc = pc.kc.clone()
        kc[int(pc.table[0, target // page]), 0, target % page] = key.to(DT[dtype])
        qkv = torch.cat([key * 2, torch.zeros(2 * d)]).reshape(1, -1).to(DT[dtype])
        out = f64(ops.attention_generic(dev(qkv), dev(kc), dev(pc.vc), dev(pc.table),
                                        dev(torch.tensor([p], dtype=torch.int32)),
                                        dev(torch.zeros(1, dtype=torch.int32)), 1, 1, d, page, window, 1.0))
        hit = maxrel(out.reshape(-1), f64(pc.v[0][target]).reshape(-1)) <= 1e-2
        assert hit == inside


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,d,rot,page,theta", [(4, 4, 16, 16, 8, 1e4), (6, 2, 24, 24, 16, 5e5),
                                                     (3, 1, 128, 64, 64, 1e6), (2, 2, 64, 0, 32, 1e4)])
def test_rope_and_cache_write(dtype, nh, nkv, d, rot, page, theta):
    lens = [70, 5]
    starts = [64, 0]      # sequence 0 appends positions 64..69, sequence 1 is a new prompt
    pc = Paged(lens, nkv, d, page, DT[dtype], seed=3)
    rows = [(0, p) for p in range(starts[0], lens[0])] + [(1, p) for p in range(lens[1])]
    T = len(rows)
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g).to(DT[dtype])
    seq = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    pos = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    table = None
    if rot:
        table = library_rope_table(d, rot, theta, 128)
    kc, vc, x = dev(pc.kc), dev(pc.vc), dev(qkv)
    err = err_word()
    ops.rope_kv_write(x, table, rot, dev(pos), dev(seq), dev(pc.table), kc, vc, nh, nkv, d, page, True, err)
    assert int(err.item()) == 0
    src = f64(qkv).reshape(T, nh + 2 * nkv, d)
    want = plain.rope_rotate_half(src[:, :nh + nkv], pos.numpy(), theta, rot) if rot else src[:, :nh + nkv]
    tol = 1e-6 if dtype == "float32" else 2 ** -8
    got = f64(x).reshape(T, nh + 2 * nkv, d)
    assert maxrel(got[:, :nh], want[:, :nh]) <= tol
    assert np.array_equal(got[:, nh:], src[:, nh:])          # K and V columns are left alone
    kc, vc = f64(kc), f64(vc)
    for i, (b, p) in enumerate(rows):
        pg = int(pc.table[b, p // page])
        assert maxrel(kc[pg, :, p % page], want[i, nh:]) <= tol
        assert np.array_equal(vc[pg, :, p % page], src[i, nh + nkv:])
    # places that were not written keep what they held
    old_k = f64(pc.kc)
    keep = np.ones(old_k.shape[:3:2], bool)  # [pages, page]
    for b, p in rows:
        keep[int(pc.table[b, p // page]), p % page] = False
    a, b_ = kc.transpose(0, 2, 1, 3)[keep], old_k.transpose(0, 2, 1, 3)[keep]
    assert np.array_equal(np.isnan(a), np.isnan(b_)) and np.array_equal(a[~np.isnan(a)], b_[~np.isnan(b_)])
    # a token whose page is missing raises the error word and writes nothing
    bad = pc.table.clone()
    bad[1, 0] = -1
    ops.rope_kv_write(dev(qkv), table, rot, dev(pos), dev(seq), dev(bad), dev(pc.kc), dev(pc.vc),
                      nh, nkv, d, page, True, err)
    assert int(err.item()) == 2


def test_rope_angles_at_far_positions_match_float64():
    """theta^(-2j/d) * p for p in the thousands: a table computed in float32 arithmetic would be
    off by 1e-4 and more; the kernel's table is float64 rounded once."""
    d = 128
    far_table = library_rope_table(d, d, 1e4, 8192)
    pos = np.array([8191, 4097, 1])
    x = np.zeros((3, 1, d))
    x[:, :, :d // 2] = 1.0
    ref = plain.rope_rotate_half(x, pos, 1e4)
    qkv = torch.zeros(3, 3 * d)
    qkv[:, :d // 2] = 1.0
    kc = torch.zeros(130, 1, 64, d, device="cuda")
    tab = torch.arange(129, dtype=torch.int32).reshape(1, 129).cuda()
    t = dev(qkv)
    ops.rope_kv_write(t, far_table, d, dev(torch.tensor(pos, dtype=torch.int32)),
                      dev(torch.zeros(3, dtype=torch.int32)), tab, kc, kc.clone(), 1, 1, d, 64, True, err_word())
    assert np.abs(f64(t)[:, :d] - ref[:, 0]).max() <= 2e-7


# ---- sampling


@pytest.mark.parametrize("B,V", [(1, 10), (7, 32000), (3, 128256), (64, 513)])
def test_argmax(B, V):
    g = torch.Generator().manual_seed(V)
    lg = torch.randn(B, V, generator=g)
    lg[0, V // 2] = lg[0, V - 1] = 50.0      # equal maxima: the lowest id wins
    out = ops.argmax(dev(lg)).cpu()
    want = lg.argmax(-1)
    want[0] = V // 2
    assert out.tolist() == want.tolist()


@pytest.mark.parametrize("temp,top_k,top_p,pen", [(0.8, 0, 1.0, 1.0), (1.0, 5, 1.0, 1.0), (0.7, 0, 0.9, 1.0),
                                                  (1.3, 40, 0.95, 1.3), (0.5, 3, 0.5, 1.1)])
def test_sample_distribution_matches_the_reference_sampler(temp, top_k, top_p, pen):
    """Draw with a fine grid of uniform numbers and compare the frequencies of the chosen ids
    with the probabilities of the reference's algorithm."""
    V, N = 97, 20000
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(V, generator=g) * 2.5)
    last = [3, 17, 17, 96, -1, 40]
    ids, probs = plain.sample_distribution(logits.numpy(), [t for t in last if t >= 0], pen, top_k, top_p, temp)
    want = np.zeros(V)
    want[ids] = probs
    u = (torch.arange(N, dtype=torch.float32) + 0.5) / N
    lg = logits.repeat(N, 1)
    lt = torch.tensor(last, dtype=torch.int32).repeat(N, 1)
    out = ops.sample(dev(lg), dev(u), temp, top_k, top_p, pen, dev(lt)).cpu().numpy()
    freq = np.bincount(out, minlength=V) / N
    assert set(np.nonzero(freq)[0]) <= set(ids.tolist()), "an id outside the kept set was drawn"
    assert np.abs(freq - want).max() <= 2.0 / N + 1e-4
    # the same uniform number gives the same id whatever else is in the batch
    one = ops.sample(dev(lg[:1]), dev(u[1234:1235]), temp, top_k, top_p, pen, dev(lt[:1])).cpu().numpy()
    assert one[0] == out[1234]


@pytest.mark.parametrize("V", [5000, 32000, 128256])
@pytest.mark.parametrize("temp,top_k,top_p,pen", [(0.9, 0, 1.0, 1.0), (0.1, 40, 0.95, 1.3), (1.0, 64, 1.0, 1.0),
                                                  (0.7, 8, 0.6, 1.2), (0.8, 100, 0.9, 1.0), (1.0, 0, 0.8, 1.0)])
def test_sample_over_a_large_vocabulary(V, temp, top_k, top_p, pen):
    """Vocabularies of several chunks: the two-pass kernels (temperature alone, top_k <= 64) and the
    one-block kernel (the rest) against the reference's algorithm, by the frequencies of the ids
    drawn with a fine grid of uniform numbers."""
    N = 4000
    g = torch.Generator().manual_seed(V + top_k)
    logits = torch.randn(V, generator=g) * 3
    logits[V - 3] = 9.0                       # mass at the end of the last, partial chunk
    logits[2049] = 8.5
    last = [2049, 7, V - 3, 7, -1]
    ids, probs = plain.sample_distribution(logits.numpy(), [t for t in last if t >= 0], pen, top_k, top_p, temp)
    want = np.zeros(V)
    want[ids] = probs
    u = (torch.arange(N, dtype=torch.float32) + 0.5) / N
    lg = dev(logits.repeat(N, 1))
    lt = dev(torch.tensor(last, dtype=torch.int32).repeat(N, 1))
    out = ops.sample(lg, dev(u), temp, top_k, top_p, pen, lt).cpu().numpy()
    freq = np.bincount(out, minlength=V) / N
    assert set(np.nonzero(freq)[0]) <= set(ids.tolist()), "an id outside the kept set was drawn"
    assert np.abs(freq - want).max() <= 2.0 / N + 2e-4
    one = ops.sample(lg[:1], dev(u[1234:1235]), temp, top_k, top_p, pen, lt[:1]).cpu().numpy()
    assert one[0] == out[1234]


def test_sample_with_many_equal_values_takes_the_slow_way_and_stays_right():
    """More equal values at the cut than a chunk hands on: the row is flagged and done by the
    one-block kernel; all equals of the cut are kept, as that kernel keeps them."""
    V, N = 6000, 3000
    logits = torch.full((V,), -5.0)
    logits[100:400] = 2.0                     # 300 equal maxima in one chunk
    logits[4500] = 1.0
    u = (torch.arange(N, dtype=torch.float32) + 0.5) / N
    out = ops.sample(dev(logits.repeat(N, 1)), dev(u), 1.0, 10, 1.0, 1.0, None).cpu().numpy()
    freq = np.bincount(out, minlength=V) / N
    assert set(np.nonzero(freq)[0]) <= set(range(100, 400))
    assert np.abs(freq[100:400] - 1 / 300).max() <= 2.0 / N


def test_sample_large_vocabulary_and_greedy_limit():
    V = 128256
    g = torch.Generator().manual_seed(9)
    lg = torch.randn(4, V, generator=g)
    lg[2, 77777] = 30.0
    u = torch.tensor([0.1, 0.5, 0.9, 0.999])
    out = ops.sample(dev(lg), dev(u), 1.0, 1, 1.0, 1.0, None).cpu()
    assert out.tolist() == lg.argmax(-1).tolist()     # top_k = 1 is greedy
    out = ops.sample(dev(lg), dev(u), 0.05, 0, 0.3, 1.0, None).cpu()
    assert out[2] == 77777


# ---- utilities: random weights, poisoned pages, the bounded wait


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,std,mean", [(1, 0.02, 0.0), (1000, 0.02, 1.0), (300007, 0.5, 0.0)])
def test_fill_random_is_the_numpy_twin_bit_for_bit(dtype, n, std, mean):
    from random_twin import random_key, random_values, to_bfloat16_bits
    key = random_key(7, "model.layers.1.mlp.up_proj.weight")
    out = ops.fill_random(torch.empty(n, dtype=DT[dtype], device="cuda"), key, std, mean).cpu()
    want = random_values(7, "model.layers.1.mlp.up_proj.weight", n, std, mean)
    if dtype == "float32":
        assert np.array_equal(out.numpy().view(np.uint32), want.view(np.uint32))
    else:
        assert np.array_equal(out.view(torch.int16).numpy().view(np.uint16), to_bfloat16_bits(want))
    if n > 1000:
        z = (want.astype(np.float64) - mean) / std
        assert abs(z.mean()) < 0.01 and abs(z.std() - 1) < 0.01 and np.abs(z).max() <= 6.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_poison_pages_fills_exactly_the_named_pages(dtype):
    k = torch.randn(3, 10, 2, 8, 24, device="cuda").to(DT[dtype])
    v = torch.randn(3, 10, 2, 8, 24, device="cuda").to(DT[dtype])
    k0, v0 = k.clone(), v.clone()
    ops.poison_pages(k, v, dev(torch.tensor([7, 0, 3], dtype=torch.int32)))
    for t, t0 in ((k, k0), (v, v0)):
        hit = torch.isnan(t).all(dim=(2, 3, 4))
        assert hit[:, [0, 3, 7]].all() and int(hit.sum()) == 9
        keep = [1, 2, 4, 5, 6, 8, 9]
        assert torch.equal(t[:, keep], t0[:, keep])


def test_a_wait_that_runs_out_sets_the_error_word_and_the_kernel_returns():
    """The tensor-core kernels wait on mbarriers through one bounded wait; here it waits, with a
    short limit, on a barrier at which nothing ever arrives.  The kernel comes back by itself, the
    wait tells its caller that it gave up, the device's error word names the kernel family, and
    the device goes on working."""
    word = ops.tc_error_word()
    word.zero_()
    for code in (4, 5, 7):
        got, gave_up, clocks = ops.selftest_wait_timeout(word, limit_clocks=1 << 18, code=code)
        assert (got, gave_up) == (code, 1)
        assert (1 << 18) <= clocks < (1 << 24)
        word.zero_()
    # the context is as usable as before
    x = torch.arange(8, device="cuda", dtype=torch.float32)
    assert float((x * 2).sum()) == 56.0
