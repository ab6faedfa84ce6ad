"""The plain implementation against MegEngine/InferLLM's own compiled code, and against itself
(no GPU).  tests/golden/golden_logits.f32 was produced by tests/golden/make_golden.sh, which
builds the reference on the CPU and runs its LLaMA graph (naive kernels) on
tests/golden/golden_model, and calls its grouped-head attention loops directly
(tests/golden/golden_gqa_ops.f32); this test needs neither the reference nor a compiler."""
import os

import numpy as np
import plain_llama as plain
from conftest import TINY, random_prompt

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_matches_the_compiled_reference():
    cfg, w = plain.load_weights(os.path.join(GOLDEN, "golden_model"))
    V = cfg["vocab_size"]
    ref = np.fromfile(os.path.join(GOLDEN, "golden_logits.f32"), dtype="<f4").reshape(-1, V).astype(np.float64)
    row = 0
    for line in open(os.path.join(GOLDEN, "golden_tokens.txt")):
        ids = [int(t) for t in line.split()]
        mine = plain.forward(cfg, w, ids)
        one_by_one, whole_last = ref[row:row + len(ids)], ref[row + len(ids)]
        row += len(ids) + 1
        scale = np.abs(mine).max()
        assert np.abs(mine - one_by_one).max() <= 2e-6 * scale     # the reference computes in float32
        assert np.abs(mine[-1] - whole_last).max() <= 2e-6 * scale
    assert row == ref.shape[0]


def test_plain_grouped_heads_match_the_references_own_loops():
    """golden_gqa_ops.f32 holds what the reference's grouped-head loops give (6 query heads over 2 KV
    heads of size 24, 7 cached positions and 5 new tokens): scores with the K head h / (heads per
    group) (src/kern/naive/naive.cpp:576-604), scale and causal mask (:531-553), softmax (:209-240),
    weighted values with the V head of the group (:634-662).  The plain functions must agree on the
    same inputs."""
    nh, nkv, d, past, n = 6, 2, 24, 7, 5
    total = past + n
    blob = np.fromfile(os.path.join(GOLDEN, "golden_gqa_ops.f32"), dtype="<f4").astype(np.float64)
    sizes = [n * nh * d, total * nkv * d, total * nkv * d, nh * n * total, nh * n * total, nh * n * total, n * nh * d]
    assert blob.size == sum(sizes)
    q, k, v, scores, masked, probs, out = np.split(blob, np.cumsum(sizes)[:-1])
    q, k, v = q.reshape(n, nh, d), k.reshape(total, nkv, d), v.reshape(total, nkv, d)
    s = plain.attention_scores(q, k, nh, nkv)
    assert np.abs(s - scores.reshape(nh, n, total)).max() <= 1e-6 * np.abs(s).max()
    m = plain.scale_and_mask(s, 1.0 / np.sqrt(d), past=past)
    ref_m = masked.reshape(nh, n, total)
    assert np.array_equal(np.isneginf(m), np.isneginf(ref_m))
    assert np.abs(np.where(np.isneginf(m), 0, m) - np.where(np.isneginf(ref_m), 0, ref_m)).max() <= 1e-6
    p = plain.softmax_rows(m)
    assert np.abs(p - probs.reshape(nh, n, total)).max() <= 1e-6
    o = plain.weighted_values(p, v, nh, nkv)
    assert np.abs(o.reshape(n, nh * d) - out.reshape(n, nh * d)).max() <= 1e-6 * np.abs(o).max()
    # and the heads really are grouped: head 2 reads K head 0, head 3 reads K head 1
    assert np.allclose(s[2], q[:, 2] @ k[:, 0].T) and np.allclose(s[3], q[:, 3] @ k[:, 1].T)


def test_plain_is_causal_and_prefix_stable(plain_models):
    """Logits at a position depend on the tokens up to it only."""
    for name in ("A", "B"):
        cfg, w = plain_models[name]
        ids = random_prompt(name, 24, 9)
        full = plain.forward(cfg, w, ids)
        part = plain.forward(cfg, w, ids[:11])
        assert np.abs(full[:11] - part).max() <= 1e-12
        other = ids[:11] + random_prompt(name, 13, 10)
        assert np.abs(plain.forward(cfg, w, other)[:11] - part).max() <= 1e-12


def test_plain_parts():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 12))
    y = plain.rms_norm(x, np.ones(12), 0.0)
    assert np.allclose((y * y).mean(-1), 1.0)
    # rotation keeps norms and composes: position p then the inverse angle gives x back
    q = rng.normal(size=(3, 2, 8))
    r = plain.rope_rotate_half(q, [0, 5, 100], 10000.0)
    assert np.allclose(r[0], q[0]) and np.allclose(np.linalg.norm(r, axis=-1), np.linalg.norm(q, axis=-1))
    # scores between rotated vectors depend on the distance of their positions only
    a = plain.rope_rotate_half(q[:1], [7], 10000.0)[0, 0] @ plain.rope_rotate_half(q[1:2], [3], 10000.0)[0, 0]
    b = plain.rope_rotate_half(q[:1], [107], 10000.0)[0, 0] @ plain.rope_rotate_half(q[1:2], [103], 10000.0)[0, 0]
    assert abs(a - b) <= 1e-9
    # partial rotation leaves the other channels alone
    pr = plain.rope_rotate_half(q, [1, 2, 3], 10000.0, rot_dim=4)
    assert np.array_equal(pr[..., 4:], q[..., 4:]) and not np.allclose(pr[..., :4], q[..., :4])
    s = plain.scale_and_mask(np.zeros((1, 3, 5)), 1.0, past=2)
    assert np.isneginf(s[0, 0, 3]) and s[0, 0, 2] == 0 and s[0, 2, 4] == 0
    s = plain.scale_and_mask(np.zeros((1, 3, 5)), 1.0, past=2, window=2)
    assert np.isneginf(s[0, 0, 0]) and s[0, 0, 1] == 0 and np.isneginf(s[0, 2, 2]) and s[0, 2, 3] == 0
    p = plain.softmax_rows(s)
    assert np.allclose(p.sum(-1), 1.0) and p[0, 0, 0] == 0
    assert abs(plain.silu(0.0)) == 0 and abs(plain.silu(10.0) - 10.0) < 1e-3


def test_plain_sampler_follows_the_reference_order():
    logits = np.array([2.0, 1.0, -1.0, 0.5, 3.0])
    ids, p = plain.sample_distribution(logits, [], 1.0, 0, 1.0, 1.0)
    assert ids.tolist() == [4, 0, 1, 3, 2] and abs(p.sum() - 1) < 1e-12
    ids, p = plain.sample_distribution(logits, [], 1.0, 2, 1.0, 1.0)
    assert ids.tolist() == [4, 0]
    ids, p = plain.sample_distribution(logits, [], 1.0, 0, 0.7, 1.0)       # 0.62 then 0.85 >= 0.7
    assert ids.tolist() == [4, 0] and abs(p.sum() - 1) < 1e-12
    ids, p = plain.sample_distribution(logits, [4, 2], 2.0, 0, 1.0, 1.0)    # 3.0 -> 1.5, -1.0 -> -2.0
    assert ids.tolist()[0] == 0 and ids.tolist()[-1] == 2
    ids, p = plain.sample_distribution(logits, [], 1.0, 0, 1.0, 0.5)        # temperature sharpens
    assert p[0] > 0.8


def test_greedy_generate_stops():
    from conftest import SEEDS  # noqa: F401  (fixtures not needed: a hand-made model)
    cfg = dict(TINY["A"], num_hidden_layers=1)
    rng = np.random.default_rng(1)
    H, I, V = 64, 176, 256
    w = {"model.embed_tokens.weight": rng.normal(size=(V, H)) * 0.1, "lm_head.weight": rng.normal(size=(V, H)) * 0.1,
         "model.norm.weight": np.ones(H)}
    for n, shape in (("self_attn.q_proj", (H, H)), ("self_attn.k_proj", (H, H)), ("self_attn.v_proj", (H, H)),
                     ("self_attn.o_proj", (H, H)), ("mlp.gate_proj", (I, H)), ("mlp.up_proj", (I, H)),
                     ("mlp.down_proj", (H, I))):
        w[f"model.layers.0.{n}.weight"] = rng.normal(size=shape) * 0.1
    w["model.layers.0.input_layernorm.weight"] = w["model.layers.0.post_attention_layernorm.weight"] = np.ones(H)
    free = plain.greedy_generate(cfg, w, [1, 2, 3], 6)
    assert len(free) == 6
    stopped = plain.greedy_generate(cfg, w, [1, 2, 3], 6, stop_ids=[free[2]])
    assert stopped == free[:free.index(free[2]) + 1]
