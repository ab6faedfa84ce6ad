"""Each part alone, built through the part registries with sizes of its own, against the plain
implementation (GPU).  The parts are given no model: a sandbox of the library builds one part from a
spec, hands it tensors and runs it on the tokens of a step."""
import math

import numpy as np
import plain_llama as plain
import pytest
import torch
from util import rel_err

from inferllm_b200 import ConfigError
from inferllm_b200.config import PartSpec
from inferllm_b200.parts import PagedKV, PartSandbox, block_norm_roles

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def randn(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def f64(t):
    return t.detach().double().cpu().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part_folds_the_pending_addition(dtype):
    h = PartSandbox({}, dtype)
    norm = h.build("norm", PartSpec("rmsnorm", {"size": 200, "eps": 1e-4}))
    w = randn(200, seed=1, scale=0.1) + 1
    norm.load({"weight": w.to(DT[dtype]).cuda()})
    x, d = randn(6, 200, seed=2), randn(6, 200, seed=3, dtype=DT[dtype])
    stream = h.stream(x.cuda())
    dd = d.cuda()
    stream.add(dd)
    y = norm.forward(stream)
    assert stream.pending is None
    want_x = f64(x) + f64(d)
    assert rel_err(f64(stream.x), want_x) <= 1e-7
    assert rel_err(f64(y), plain.rms_norm(want_x, f64(w.to(DT[dtype])), 1e-4)) <= TOL[dtype]
    # two additions in a row: the first is flushed, the second waits for the next norm
    stream.add(dd)
    stream.add(dd)
    assert rel_err(f64(stream.x), want_x + f64(d)) <= 1e-7 and stream.pending is not None
    # a norm of chosen rows leaves the stream as it is (the final norm of a model)
    rows = torch.tensor([4, 1], dtype=torch.int32, device="cuda")
    y2 = norm.forward(stream, rows=rows)
    assert stream.pending is not None and rel_err(f64(stream.x), want_x + f64(d)) <= 1e-7
    assert rel_err(f64(y2), plain.rms_norm((want_x + 2 * f64(d))[[4, 1]], f64(w.to(DT[dtype])), 1e-4)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    h = PartSandbox({}, dtype)
    H, I = 72, 200
    ffn = h.build("feed_forward", PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I}))
    assert {k: v.shape for k, v in ffn.tensors().items()} == {
        "gate_proj.weight": (I, H), "up_proj.weight": (I, H), "down_proj.weight": (H, I)}
    ws = {k: randn(*v.shape, seed=i, scale=0.1, dtype=torch.bfloat16) for i, (k, v) in enumerate(ffn.tensors().items())}
    ffn.load({k: v.cuda() for k, v in ws.items()})
    x = randn(11, H, seed=9, dtype=DT[dtype])
    out = ffn.forward(x.cuda())
    ref = plain.swiglu_ffn(f64(x), f64(ws["gate_proj.weight"]), f64(ws["up_proj.weight"]), f64(ws["down_proj.weight"]))
    assert rel_err(f64(out), ref) <= TOL[dtype]
    with pytest.raises(ConfigError, match="activation"):
        h.build("feed_forward", PartSpec("gated_mlp", {"hidden_size": 8, "intermediate_size": 8, "activation": "relu"}))


def _attention(h, H, nh, nkv, d, window, theta, rot=None):
    pos = PartSpec("rope_half", {"head_dim": d, "rot_dim": rot or d, "theta": theta, "max_positions": 256})
    spec = PartSpec("attention", {"hidden_size": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d,
                                  "window": window, "position": pos})
    return h.build("mixer", spec)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,nh,nkv,d,window,theta,rot", [(48, 3, 3, 16, None, 1e4, None), (80, 4, 2, 40, None, 5e5, 24),
                                                          (64, 4, 1, 32, 20, 1e6, None)])
def test_attention_part_prompt_then_tokens(dtype, H, nh, nkv, d, window, theta, rot):
    """Two sequences of unequal lengths: prompts in one step, then single tokens, the shorter
    one ending earlier; compared with the plain attention over each whole sequence."""
    req = PagedKV(nkv, d, window)
    h = PartSandbox({0: req}, dtype, page_size=8, num_pages=24)
    att = _attention(h, H, nh, nkv, d, window, theta, rot)
    assert att.cache_request() == req
    ws = {k: randn(*v.shape, seed=i + 1, scale=0.15, dtype=torch.bfloat16) for i, (k, v) in enumerate(att.tensors().items())}
    att.load({k: v.cuda() for k, v in ws.items()})
    lens = [61, 30]
    xs = [randn(n, H, seed=20 + i, dtype=DT[dtype]) for i, n in enumerate(lens)]
    refs = [plain.self_attention(f64(x), f64(ws["q_proj.weight"]), f64(ws["k_proj.weight"]),
                                 f64(ws["v_proj.weight"]), f64(ws["o_proj.weight"]), np.arange(len(x)),
                                 nh, nkv, d, theta, window, rot)[0] for x in xs]
    slots = [h.cache.alloc_slot() for _ in lens]
    pre = [41, 27]
    h.begin_step(slots, pre)
    out = att.forward(torch.cat([x[:p] for x, p in zip(xs, pre)]).cuda())
    h.commit_step()
    got = [[out[:pre[0]]], [out[pre[0]:]]]
    for step in range(lens[0] - pre[0]):
        live = [i for i in range(2) if pre[i] + step < lens[i]]
        h.begin_step([slots[i] for i in live], [1] * len(live))
        out = att.forward(torch.stack([xs[i][pre[i] + step] for i in live]).cuda())
        h.commit_step()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
    for i in range(2):
        assert rel_err(f64(torch.cat(got[i])), refs[i]) <= TOL[dtype]
    h.begin_step([slots[0]], [1])
    assert h.error_word() == 0
    if window:
        # pages that left the window went back to the pool while the sequences were live
        assert len(h.cache.pages_of(0, slots[0])) <= -(-window // 8) + 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_window_and_a_later_portion_after_pages_were_released(dtype):
    """A windowed layer with pages smaller than a key tile of the prompt kernel: after a first
    portion of 100 tokens the pages below the window have gone back to the pool (their table entries
    read -1, and other sequences' data lies in them), then a second portion of 30 tokens arrives in
    one step.  Its first key tile starts below the window, inside the released pages: those keys
    must be skipped, not read."""
    H, nh, nkv, d, window, theta = 128, 2, 1, 64, 40, 1e4
    req = PagedKV(nkv, d, window)
    h = PartSandbox({0: req}, dtype, page_size=16, num_pages=12)
    att = _attention(h, H, nh, nkv, d, window, theta)
    ws = {k: randn(*v.shape, seed=i + 1, scale=0.15, dtype=torch.bfloat16) for i, (k, v) in enumerate(att.tensors().items())}
    att.load({k: v.cuda() for k, v in ws.items()})
    x = randn(130, H, seed=31, dtype=DT[dtype])
    ref = plain.self_attention(f64(x), f64(ws["q_proj.weight"]), f64(ws["k_proj.weight"]), f64(ws["v_proj.weight"]),
                               f64(ws["o_proj.weight"]), np.arange(130), nh, nkv, d, theta, window, None)[0]
    s = h.cache.alloc_slot()
    got = []
    for lo, hi in ((0, 100), (100, 130)):
        h.begin_step([s], [hi - lo])
        got.append(att.forward(x[lo:hi].cuda()))
        if hi == 100:
            kv = h.cache_view(0)
        h.commit_step()
        if hi == 100:
            held = h.cache.pages_of(0, s)
            assert min(held) == 3, "the pages below the window should have been released"
            # what lies in released pages now is somebody else's: make it loud
            free = [p for p in range(12) if p not in held.values()]
            kv.k[free] = float("nan")
            kv.v[free] = float("nan")
    out = f64(torch.cat(got))
    assert np.isfinite(out).all()
    assert rel_err(out, ref) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_reading_another_entrys_cache(dtype):
    """writes=False: the mixer projects only its queries and attends to the keys and values that
    the owner of the cache entry stored in the same step."""
    H, nh, nkv, d = 32, 2, 1, 16
    h = PartSandbox({0: PagedKV(nkv, d)}, dtype, page_size=8)
    owner, reader = _attention(h, H, nh, nkv, d, None, 1e4), _attention(h, H, nh, nkv, d, None, 1e4)
    wo = {k: randn(*v.shape, seed=i + 1, scale=0.2, dtype=torch.bfloat16) for i, (k, v) in enumerate(owner.tensors().items())}
    wr = {k: randn(*v.shape, seed=i + 50, scale=0.2, dtype=torch.bfloat16) for i, (k, v) in enumerate(reader.tensors().items())}
    owner.load({k: v.cuda() for k, v in wo.items()})
    reader.load({k: v.cuda() for k, v in wr.items()})
    x1, x2 = randn(19, H, seed=5, dtype=DT[dtype]), randn(19, H, seed=6, dtype=DT[dtype])
    s = h.cache.alloc_slot()
    h.begin_step([s], [19])
    owner.forward(x1.cuda(), entry=0, writes=True)
    out = reader.forward(x2.cuda(), entry=0, writes=False)
    pos = np.arange(19)
    _, kv = plain.self_attention(f64(x1), *(f64(wo[k + "_proj.weight"]) for k in "qkvo"), pos, nh, nkv, d, 1e4)
    ref, _ = plain.self_attention(f64(x2), *(f64(wr[k + "_proj.weight"]) for k in "qkvo"), pos, nh, nkv, d, 1e4,
                                  kv_override=kv)
    assert rel_err(f64(out), ref) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prenorm_block(dtype):
    H, nh, nkv, d, I, eps = 48, 3, 1, 16, 100, 1e-5
    h = PartSandbox({0: PagedKV(nkv, d)}, dtype, page_size=8)
    att = _attention(h, H, nh, nkv, d, None, 1e4)
    ffn = h.build("feed_forward", PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I}))
    assert block_norm_roles("prenorm") == ("norm1", "norm2")
    # the two norms of a block have specs of their own: here they differ in eps
    eps2 = 1e-2
    norms = {"norm1": h.build("norm", PartSpec("rmsnorm", {"size": H, "eps": eps})),
             "norm2": h.build("norm", PartSpec("rmsnorm", {"size": H, "eps": eps2}))}
    w = {}
    for i, (prefix, part) in enumerate([("a.", att), ("f.", ffn), ("n1.", norms["norm1"]), ("n2.", norms["norm2"])]):
        ts = {k: (randn(*v.shape, seed=7 * i + j, scale=0.15, dtype=torch.bfloat16) + (1 if v.init == "norm" else 0))
              for j, (k, v) in enumerate(part.tensors().items())}
        part.load({k: v.cuda() for k, v in ts.items()})
        w.update({prefix + k: f64(v) for k, v in ts.items()})
    block = h.block("prenorm", att, ffn, norms)
    x = randn(23, H, seed=3)
    s = h.cache.alloc_slot()
    h.begin_step([s], [23])
    stream = h.stream(x.cuda())
    block.forward(stream, entry=0, writes=True)
    got = f64(stream.flush())
    xr = f64(x)
    a, _ = plain.self_attention(plain.rms_norm(xr, w["n1.weight"], eps), w["a.q_proj.weight"], w["a.k_proj.weight"],
                                w["a.v_proj.weight"], w["a.o_proj.weight"], np.arange(23), nh, nkv, d, 1e4)
    xr = xr + a
    xr = xr + plain.swiglu_ffn(plain.rms_norm(xr, w["n2.weight"], eps2), w["f.gate_proj.weight"],
                               w["f.up_proj.weight"], w["f.down_proj.weight"])
    assert rel_err(got, xr) <= TOL[dtype]


def test_position_none_stores_without_rotating():
    H, nh, nkv, d = 32, 2, 2, 16
    h = PartSandbox({0: PagedKV(nkv, d)}, "float32", page_size=8)
    spec = PartSpec("attention", {"hidden_size": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d,
                                  "window": None, "position": PartSpec("none", {})})
    att = h.build("mixer", spec)
    ws = {k: randn(*v.shape, seed=i + 1, scale=0.2) for i, (k, v) in enumerate(att.tensors().items())}
    att.load({k: v.cuda() for k, v in ws.items()})
    x = randn(10, H, seed=4)
    s = h.cache.alloc_slot()
    h.begin_step([s], [10])
    out = att.forward(x.cuda())
    xr = f64(x)
    q = plain.linear(xr, f64(ws["q_proj.weight"])).reshape(10, nh, d)
    k = plain.linear(xr, f64(ws["k_proj.weight"])).reshape(10, nkv, d)
    v = plain.linear(xr, f64(ws["v_proj.weight"])).reshape(10, nkv, d)
    p = plain.softmax_rows(plain.scale_and_mask(plain.attention_scores(q, k, nh, nkv), 1 / math.sqrt(d)))
    ref = plain.linear(plain.weighted_values(p, v, nh, nkv), f64(ws["o_proj.weight"]))
    assert rel_err(f64(out), ref) <= 1e-5
