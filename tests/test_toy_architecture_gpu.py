"""A toy architecture defined here, registered, built and stepped without a change to the
library's files (GPU): layers with different mixers, a mixer with fixed-size state of its own,
another position encoding, a feed-forward with routing, two norms of one block that differ, a layer
that runs twice and a layer that reads another layer's cache.  The parts are written in Python over
the library's interface for parts in other languages (the library calls them on every step); the
architecture is a Python class whose spec the library builds its generic decoder from.  It is no model
of anyone's; it shows that the seams hold."""
from dataclasses import dataclass

import numpy as np
import plain_llama as plain
import pytest
import torch
from util import rel_err

from inferllm_b200 import Engine, EngineOptions, StepItem, write_random_model
from inferllm_b200.config import (ArchConfig, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture,
                                  unregister_architecture)
from inferllm_b200.kernels import ops
from inferllm_b200.parts import (FeedForward, FixedState, Mixer, PositionEncoding, TensorDecl, register_feed_forward,
                                 register_mixer, register_position, unregister_part)

pytestmark = pytest.mark.gpu
H, NH, NKV, D, I, V, EPS, EPS2, THETA = 48, 3, 1, 16, 80, 97, 1e-5, 3e-3, 1e4


@register_mixer("toy_running_mean")
class RunningMean(Mixer):
    """out[t] = W . mean(h[0..t]) over the token's own sequence.  The state is the running sum
    and the count, [H + 1] floats per sequence, kept in the cache's fixed-size area.  Written
    with torch operations: a test's part needs no kernel of the package."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.h = int(spec["hidden_size"])

    def tensors(self):
        return {"mix.weight": TensorDecl((self.h, self.h))}

    def load(self, tensors):
        self.w = tensors["mix.weight"].float()

    def cache_request(self):
        return FixedState((self.h + 1,), "float32")

    def forward(self, h, ctx, cache, writes):
        out = torch.empty_like(h)
        off = 0
        slots = ctx.host_slots
        for b, q in enumerate(ctx.q_lens):
            st = cache.state[slots[b]]
            x = h[off:off + q].float()
            sums = st[:self.h] + torch.cumsum(x, 0)
            counts = st[self.h] + torch.arange(1, q + 1, device=h.device, dtype=torch.float32)
            out[off:off + q] = ((sums / counts[:, None]) @ self.w.t()).to(h.dtype)
            st[:self.h] = sums[-1]
            st[self.h] = counts[-1]
            off += q
        return out


@register_position("toy_pairs")
class PairRotation(PositionEncoding):
    """Another position encoding: neighbouring channels (2j, 2j+1) of every Q and K head are
    rotated by p * theta^(-2j/d) (the reference's LLaMA-1 files use this pairing,
    src/kern/naive/naive.cpp:415-440).  The rotation is plain torch; the cache write reuses the
    package's kernel with its own rotation switched off."""

    def encode_and_store(self, qkv, geometry, ctx, kv):
        nh, nkv, d = geometry
        theta = float(self.spec["theta"])
        T = qkv.shape[0]
        x = qkv.view(T, nh + 2 * nkv, d)[:, :nh + nkv].float()
        inv = theta ** (-torch.arange(0, d, 2, device=qkv.device, dtype=torch.float64) / d)
        ang = ctx.token_pos.double()[:, None] * inv[None, :]
        c, s_ = torch.cos(ang).float()[:, None, :], torch.sin(ang).float()[:, None, :]
        a, b = x[..., 0::2], x[..., 1::2]
        rot = torch.stack((a * c - b * s_, a * s_ + b * c), dim=-1).reshape(T, nh + nkv, d)
        qkv.view(T, nh + 2 * nkv, d)[:, :nh + nkv] = rot.to(qkv.dtype)
        if kv.writes:
            ops.rope_kv_write(qkv, None, 0, ctx.token_pos, ctx.token_seq, kv.block_table, kv.k, kv.v, nh, nkv, d,
                              kv.page_size, True, ctx.err)
        return qkv


N_EXPERTS, I_EXPERT = 3, 40


@register_feed_forward("toy_top1_experts")
class Top1Experts(FeedForward):
    """A feed-forward with routing: float32 router logits h . Wr^T, the best expert per token,
    that expert's gated MLP.  Plain torch, token by expert."""

    def tensors(self):
        t = {"router.weight": TensorDecl((N_EXPERTS, H))}
        for e in range(N_EXPERTS):
            t[f"experts.{e}.gate_proj.weight"] = TensorDecl((I_EXPERT, H))
            t[f"experts.{e}.up_proj.weight"] = TensorDecl((I_EXPERT, H))
            t[f"experts.{e}.down_proj.weight"] = TensorDecl((H, I_EXPERT))
        return t

    def load(self, tensors):
        self.w = {k: v.float() for k, v in tensors.items()}

    def forward(self, h, ctx):
        x = h.float()
        choice = (x @ self.w["router.weight"].t()).argmax(-1)
        out = torch.zeros_like(x)
        for e in range(N_EXPERTS):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                xe = x[rows]
                g = xe @ self.w[f"experts.{e}.gate_proj.weight"].t()
                u = xe @ self.w[f"experts.{e}.up_proj.weight"].t()
                out[rows] = (g / (1 + torch.exp(-g)) * u) @ self.w[f"experts.{e}.down_proj.weight"].t()
        return out.to(h.dtype)


@dataclass
class ToyConfig(ArchConfig):
    n_positions: int = 128

    @classmethod
    def from_dict(cls, d):
        return cls(n_positions=d.get("n_positions", 128))

    def to_dict(self):
        return {"architectures": ["ToyMixForCausalLM"], "n_positions": self.n_positions}

    def model_spec(self):
        norm = PartSpec("rmsnorm", {"size": H, "eps": EPS})
        norm_b = PartSpec("rmsnorm", {"size": H, "eps": EPS2})      # the second norm of a block is another one
        att = PartSpec("attention", {"hidden_size": H, "n_heads": NH, "n_kv_heads": NKV, "head_dim": D,
                                     "window": None, "position": PartSpec("rope_half", {
                                         "head_dim": D, "theta": THETA, "max_positions": self.n_positions})})
        mean = PartSpec("toy_running_mean", {"hidden_size": H})
        ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I})
        att_pairs = PartSpec("attention", {"hidden_size": H, "n_heads": NH, "n_kv_heads": NKV, "head_dim": D,
                                           "window": None, "position": PartSpec("toy_pairs", {"theta": THETA})})
        routed = PartSpec("toy_top1_experts", {})
        names = {"mixer": "mixer.", "ffn": "ffn.", "norm1": "ln1.", "norm2": "ln2."}
        layers = [LayerSpec("prenorm", m, f, {"norm1": norm, "norm2": norm_b}, f"blocks.{i}.", dict(names))
                  for i, (m, f) in enumerate([(att, ffn), (mean, ffn), (att, ffn), (att_pairs, routed)])]
        # layer 0, layer 1 (state), layer 0 again (a second cache entry), layer 2 reading entry 0,
        # layer 3 with the other position encoding and the routed feed-forward
        schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                    ScheduleEntry(2, 0, writes=False), ScheduleEntry(3, 3)]
        return ModelSpec(H, V, layers, schedule,
                         PartSpec("embedding", {"name": "emb.", "vocab_size": V, "hidden_size": H}),
                         PartSpec("rmsnorm", {"name": "ln_f.", "size": H, "eps": EPS}),
                         PartSpec("lm_head", {"name": "head.", "tied": True, "vocab_size": V, "hidden_size": H}),
                         self.n_positions, None, [])


def pair_rotation(x, positions, theta):
    d = x.shape[-1]
    ang = np.asarray(positions, np.float64)[:, None] * theta ** (-np.arange(0, d, 2) / d)[None, :]
    c, s_ = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = np.empty_like(x)
    out[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s_
    out[..., 1::2] = x[..., 0::2] * s_ + x[..., 1::2] * c
    return out


def plain_layer3(w, x, pos):
    """Layer 3 of the toy: attention with pair rotation, then the routed feed-forward.  Returns the
    new stream and, per token, the margin between its two best router logits."""
    p = "blocks.3."
    h = plain.rms_norm(x, w[p + "ln1.weight"], EPS)
    T = len(pos)
    q = pair_rotation(plain.linear(h, w[p + "mixer.q_proj.weight"]).reshape(T, NH, D), pos, THETA)
    k = pair_rotation(plain.linear(h, w[p + "mixer.k_proj.weight"]).reshape(T, NKV, D), pos, THETA)
    v = plain.linear(h, w[p + "mixer.v_proj.weight"]).reshape(T, NKV, D)
    sc = plain.scale_and_mask(plain.attention_scores(q, k, NH, NKV), D ** -0.5)
    o = plain.weighted_values(plain.softmax_rows(sc), v, NH, NKV)
    x = x + plain.linear(o, w[p + "mixer.o_proj.weight"])
    h = plain.rms_norm(x, w[p + "ln2.weight"], EPS2)
    logits = plain.linear(h, w[p + "ffn.router.weight"])
    top = np.sort(logits, -1)
    margin = top[:, -1] - top[:, -2]
    f = np.zeros_like(x)
    for t, e in enumerate(logits.argmax(-1)):
        q_ = f"ffn.experts.{e}."
        f[t] = plain.swiglu_ffn(h[t:t + 1], w[p + q_ + "gate_proj.weight"], w[p + q_ + "up_proj.weight"],
                                w[p + q_ + "down_proj.weight"])[0]
    return x + f, margin


def plain_toy(w, ids):
    """The toy model in float64, whole sequence, with the plain implementation's functions.
    Returns the logits and the router margins of the last layer."""
    pos = np.arange(len(ids))
    x = plain.embed(ids, w["emb.weight"])
    kv0 = None
    for layer, entry, writes in [(0, 0, True), (1, 1, True), (0, 2, True), (2, 0, False)]:
        p = f"blocks.{layer}."
        h = plain.rms_norm(x, w[p + "ln1.weight"], EPS)
        if layer == 1:
            mean = np.cumsum(h, 0) / np.arange(1, len(ids) + 1)[:, None]
            a = mean @ w[p + "mixer.mix.weight"].T
        else:
            a, kv = plain.self_attention(h, *(w[p + f"mixer.{n}_proj.weight"] for n in "qkvo"), pos, NH, NKV, D,
                                         THETA, kv_override=None if writes else kv0)
            if entry == 0 and writes:
                kv0 = kv
        x = x + a
        h = plain.rms_norm(x, w[p + "ln2.weight"], EPS2)
        x = x + plain.swiglu_ffn(h, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                                 w[p + "ffn.down_proj.weight"])
    x, margin = plain_layer3(w, x, pos)
    return plain.linear(plain.rms_norm(x, w["ln_f.weight"], EPS), w["emb.weight"]), margin


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    register_architecture("ToyMixForCausalLM", ToyConfig)
    d = str(tmp_path_factory.mktemp("toy"))
    write_random_model(ToyConfig(), d, seed=3, dtype=torch.float32)
    yield d
    unregister_architecture("ToyMixForCausalLM")
    for family, kind in (("mixer", "toy_running_mean"), ("position", "toy_pairs"), ("feed_forward", "toy_top1_experts")):
        unregister_part(family, kind)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_toy_architecture_steps_like_its_plain_twin(toy_folder, dtype, tol):
    _, w = plain.load_weights(toy_folder)
    if dtype == "bfloat16":   # the engine rounds the stored float32 matrices; give the twin the same
        w = {k: (torch.tensor(v).bfloat16().double().numpy() if "ln" not in k else v) for k, v in w.items()}
    eng = Engine.from_folder(toy_folder, EngineOptions(dtype=dtype, max_tokens=512, page_size=16, max_batch=3))
    st = eng.cache.stats()
    assert len(st["paged"]) == 1 and st["paged"][0]["entries"] == [0, 2, 3]
    assert len(st["states"]) == 1 and tuple(eng.state_tensor(0).shape) == (1, 3, H + 1)
    assert eng.info()["graph_safe"] is False        # the toy mixer reads the step's host fields
    rng = np.random.default_rng(0)
    reqs = [rng.integers(0, V, n).tolist() for n in (70, 9, 33, 50)]
    both = [plain_toy(w, r) for r in reqs]
    refs = [b[0] for b in both]
    # a token whose two best router logits are closer than rounding may go to the other expert in
    # the engine: such positions (of the last layer, so nothing downstream is touched) are left out
    sure = [b[1] > (1e-4 if dtype == "float32" else 3e-2) for b in both]
    assert all(s_.mean() > 0.5 for s_ in sure)
    for batch, pre in (([0, 1, 2], [40, 9, 1]), ([3, 1], [17, 5])):     # the second batch reuses slots
        slots = {r: eng.new_sequence() for r in batch}
        lg = eng.step([StepItem(slots[r], reqs[r][:p], list(range(p))) for r, p in zip(batch, pre)]).cpu().numpy()
        off = 0
        for r, p in zip(batch, pre):
            keep = sure[r][:p]
            if keep.any():
                assert rel_err(lg[off:off + p][keep], refs[r][:p][keep]) <= tol
            off += p
        pos = dict(zip(batch, pre))
        live = [r for r in batch if pos[r] < len(reqs[r])]
        while live:
            lg = eng.step([StepItem(slots[r], [reqs[r][pos[r]]], [0]) for r in live]).cpu().numpy()
            for i, r in enumerate(live):
                if sure[r][pos[r]]:
                    assert rel_err(lg[i], refs[r][pos[r]]) <= tol, (r, pos[r])
                pos[r] += 1
            live = [r for r in live if pos[r] < len(reqs[r])]
        for s in slots.values():
            eng.end_sequence(s)
    eng.check_device_errors()
    eng.cache.check()
