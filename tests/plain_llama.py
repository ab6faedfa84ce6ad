"""Plain, slow implementation of the LLaMA decoder in float64 numpy.

It is the oracle of the test-suite: whole sequences, no cache, one function for
each part, and no code shared with the `inferllm_b200` package (it reads the raw
`config.json` dictionary and a dictionary of numpy arrays keyed by tensor name).

Every function restates a formula of MegEngine/InferLLM; the citations give the
file and lines of the reference (paths relative to the reference project).  The
reference hard-codes some constants (eps 1e-6 / 1e-5, rope base 10000, MHA only);
here they are arguments, which is the only generalisation.  For the one tiny
configuration that the reference can run (MHA, theta 10000) this file is compared
with the compiled reference itself: see tests/golden/.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


# --------------------------------------------------------------------------- parts


def embed(ids, table):
    """Row gather `x[t,:] = W[id[t],:]` (src/kern/naive/naive.cpp:43-54)."""
    return np.asarray(table, F64)[np.asarray(ids, np.int64)]


def rms_norm(x, weight, eps):
    """`mean = sum(x^2)/H; y = x / sqrt(mean + eps)` then a separate multiply by the
    weight (src/kern/naive/naive.cpp:186-207 and :138-149; op src/core/op.cpp:37-47)."""
    x = np.asarray(x, F64)
    mean = (x * x).sum(-1, keepdims=True) / x.shape[-1]
    return x * (1.0 / np.sqrt(mean + eps)) * np.asarray(weight, F64)


def linear(x, w):
    """`y[m,n] = sum_k W[n,k] x[m,k]`, weight row-major [out, in], no bias
    (src/kern/naive/naive.cpp:363-379)."""
    return np.asarray(x, F64) @ np.asarray(w, F64).T


def rope_rotate_half(x, positions, theta, rot_dim=None):
    """Rotate-half position encoding (RotMode::ModelRotHalf,
    src/kern/naive/naive.cpp:389-414): for pair index j < n_rot/2,
    `angle = p * theta^(-2j/n_rot)`, `out[j] = x[j] cos - x[j+half] sin`,
    `out[j+half] = x[j] sin + x[j+half] cos`, trigonometry in double.
    `x` is [T, heads, d]; `half` is n_rot/2 (the reference rotates the whole head,
    n_rot = d, src/graph/llama_like.cpp:60)."""
    x = np.asarray(x, F64)
    d = x.shape[-1]
    n_rot = d if rot_dim is None else rot_dim
    half = n_rot // 2
    j = np.arange(half, dtype=F64)
    inv = np.power(F64(theta), -2.0 * j / n_rot)
    ang = np.asarray(positions, F64)[:, None] * inv[None, :]  # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:n_rot]
    out[..., :half] = a * c - b * s
    out[..., half:n_rot] = a * s + b * c
    return out


def attention_scores(q, k, n_heads, n_kv_heads):
    """`S[h,i,t] = sum_c Q[i,h,c] K[t,h/g,c]` (src/kern/naive/naive.cpp:606-632; the
    grouped form with key head `h / (heads/groups)` is :576-604)."""
    g = n_heads // n_kv_heads
    T = q.shape[0]
    s = np.empty((n_heads, T, k.shape[0]), F64)
    for h in range(n_heads):
        s[h] = q[:, h, :] @ k[:, h // g, :].T
    return s


def scale_and_mask(s, scale, past=0, window=None):
    """`S = (t > past + i) ? -inf : S * scale` (src/kern/naive/naive.cpp:531-553), the
    scale being 1/sqrt(head size) (src/core/op.cpp:488).  `window` (not in the
    reference) additionally hides keys older than `window` positions."""
    n_q, n_k = s.shape[1], s.shape[2]
    i = np.arange(n_q)[:, None] + past
    t = np.arange(n_k)[None, :]
    hide = t > i
    if window is not None:
        hide = hide | (t < i - window + 1)
    return np.where(hide[None], -np.inf, s * scale)


def softmax_rows(s):
    """Row maximum, `exp(s - max)` (0 where s is -inf), sum, multiply by 1/sum
    (src/kern/naive/naive.cpp:209-240)."""
    m = s.max(-1, keepdims=True)
    e = np.where(np.isneginf(s), 0.0, np.exp(s - m))
    return e * (1.0 / e.sum(-1, keepdims=True))


def weighted_values(p, v, n_heads, n_kv_heads):
    """`O[i,h,c] = sum_t V[t,h/g,c] P[h,i,t]` (src/kern/naive/naive.cpp:664-691,
    grouped form :634-662); the result is already [T, heads*d]."""
    g = n_heads // n_kv_heads
    T, d = p.shape[1], v.shape[-1]
    o = np.empty((T, n_heads, d), F64)
    for h in range(n_heads):
        o[:, h, :] = p[h] @ v[:, h // g, :]
    return o.reshape(T, n_heads * d)


def self_attention(h, wq, wk, wv, wo, positions, n_heads, n_kv_heads, head_dim, theta,
                   window=None, rot_dim=None, kv_override=None):
    """The attention module in the reference's order (src/core/op.cpp:348-500): three
    projections, rotation of Q and of the new K rows, scores, scale + mask, softmax,
    weighted values, then the output projection (src/core/graph.h:106-111).
    `kv_override` = (k, v) lets a layer attend to another layer's rotated keys and
    values (cache sharing; not in the reference).  Returns (out, (k, v))."""
    T = h.shape[0]
    q = linear(h, wq).reshape(T, n_heads, head_dim)
    q = rope_rotate_half(q, positions, theta, rot_dim)
    if kv_override is None:
        k = linear(h, wk).reshape(T, n_kv_heads, head_dim)
        k = rope_rotate_half(k, positions, theta, rot_dim)
        v = linear(h, wv).reshape(T, n_kv_heads, head_dim)
    else:
        k, v = kv_override
    s = attention_scores(q, k, n_heads, n_kv_heads)
    s = scale_and_mask(s, 1.0 / math.sqrt(head_dim), 0, window)
    p = softmax_rows(s)
    o = weighted_values(p, v, n_heads, n_kv_heads)
    return linear(o, wo), (k, v)


def silu(x):
    """`x / (1 + exp(-x))` (src/kern/naive/naive.cpp:80-89)."""
    return x / (1.0 + np.exp(-x))


def swiglu_ffn(h, w_gate, w_up, w_down):
    """`down( silu(gate(h)) * up(h) )` (src/core/graph.cpp:57-79: w3 = up, w1 = gate,
    w2 = down)."""
    return linear(silu(linear(h, w_gate)) * linear(h, w_up), w_down)


# --------------------------------------------------------------------------- model


def forward(config: dict, weights: dict, ids, return_hidden=False):
    """Logits [T, vocab] at every position of one whole sequence.

    Layer stack of src/graph/llama_like.cpp:54-109: embedding; per layer
    norm -> attention -> add, norm -> feed-forward -> add; final norm and output
    matrix (src/core/graph.cpp:117-141), here for every row instead of the last."""
    H = config["hidden_size"]
    nh = config["num_attention_heads"]
    nkv = config.get("num_key_value_heads", nh)
    d = config.get("head_dim") or H // nh
    eps = config.get("rms_norm_eps", 1e-6)
    theta = config.get("rope_theta", 10000.0)
    L = config["num_hidden_layers"]
    pos = np.arange(len(ids))
    x = embed(ids, weights["model.embed_tokens.weight"])
    for i in range(L):
        p = f"model.layers.{i}."
        h = rms_norm(x, weights[p + "input_layernorm.weight"], eps)
        a, _ = self_attention(
            h, weights[p + "self_attn.q_proj.weight"], weights[p + "self_attn.k_proj.weight"],
            weights[p + "self_attn.v_proj.weight"], weights[p + "self_attn.o_proj.weight"],
            pos, nh, nkv, d, theta)
        x = x + a
        h = rms_norm(x, weights[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu_ffn(h, weights[p + "mlp.gate_proj.weight"],
                           weights[p + "mlp.up_proj.weight"], weights[p + "mlp.down_proj.weight"])
    # the reference's head has an eps of its own (1e-5, src/core/graph.h:160-163); a config.json
    # has one eps for all norms, so the extra key exists only for the comparison with the reference
    y = rms_norm(x, weights["model.norm.weight"], config.get("final_norm_eps", eps))
    head = weights["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) \
        else weights["lm_head.weight"]
    logits = linear(y, head)
    return (logits, x) if return_hidden else logits


def greedy_generate(config, weights, prompt, n_new, stop_ids=()):
    """Greedy continuation by re-running the whole sequence for every new token."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        tok = int(np.argmax(forward(config, weights, ids)[-1]))
        out.append(tok)
        ids.append(tok)
        if tok in stop_ids:
            break
    return out


# --------------------------------------------------------------------------- sampling


def sample_distribution(logits, last_tokens, repeat_penalty, top_k, top_p, temp):
    """The reference's sampler up to the random draw (src/utils.cpp:31-115): scale by
    1/temp; for ids among the last tokens multiply negative scores by the penalty and
    divide the others; keep the top_k largest (sorted, :21-29); softmax in double; cut
    after the first prefix whose cumulative probability reaches top_p and renormalise.
    Returns (ids in descending order of score, their probabilities)."""
    logits = np.asarray(logits, F64)
    scaled = logits / temp
    for i in set(int(t) for t in last_tokens):
        if 0 <= i < len(scaled):
            scaled[i] = logits[i] / temp * repeat_penalty if logits[i] < 0 else logits[i] / temp / repeat_penalty
    order = np.argsort(-scaled, kind="stable")
    if top_k and top_k > 0:
        order = order[:top_k]
    vals = scaled[order]
    p = np.exp(vals - vals.max())
    p /= p.sum()
    if top_p < 1.0:
        c = np.cumsum(p)
        n = int(np.searchsorted(c, top_p, side="left")) + 1
        n = min(n, len(p))
        order, p = order[:n], p[:n] / c[n - 1]
    return order, p


def load_weights(folder):
    """Read model.safetensors of a model folder into float64 arrays (independent
    reader: the `safetensors` package, not the product's loader)."""
    import json
    import os

    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    return cfg, {k: v.double().numpy() for k, v in tensors.items()}
