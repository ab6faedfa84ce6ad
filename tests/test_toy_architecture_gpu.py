"""A toy architecture defined here, registered, built and stepped without a change to the
package's files (GPU): layers with different mixers, a mixer with fixed-size state of its own,
a layer that runs twice and a layer that reads another layer's cache.  It is no model of
anyone's; it shows that the seams hold."""
from dataclasses import dataclass

import numpy as np
import plain_llama as plain
import pytest
import torch
from util import rel_err

from inferllm_b200 import Engine, EngineOptions, StepItem, write_random_model
from inferllm_b200.config import ArchConfig, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from inferllm_b200.parts import FixedState, Mixer, TensorDecl, register_mixer
from inferllm_b200.registry import register_architecture, unregister_architecture

pytestmark = pytest.mark.gpu
H, NH, NKV, D, I, V, EPS, THETA = 48, 3, 1, 16, 80, 97, 1e-5, 1e4


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
        return FixedState((self.h + 1,), torch.float32)

    def forward(self, h, ctx, cache, writes):
        out = torch.empty_like(h)
        off = 0
        slots = ctx.slots.tolist()
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


@dataclass
class ToyConfig(ArchConfig):
    n_positions: int = 128
    architecture = "ToyMixForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(n_positions=d.get("n_positions", 128))

    def to_dict(self):
        return {"architectures": [self.architecture], "n_positions": self.n_positions}

    def model_spec(self):
        norm = PartSpec("rmsnorm", {"size": H, "eps": EPS})
        att = PartSpec("attention", {"hidden_size": H, "n_heads": NH, "n_kv_heads": NKV, "head_dim": D,
                                     "window": None, "position": PartSpec("rope_half", {
                                         "head_dim": D, "theta": THETA, "max_positions": self.n_positions})})
        mean = PartSpec("toy_running_mean", {"hidden_size": H})
        ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I})
        names = {"mixer": "mixer.", "ffn": "ffn.", "norm1": "ln1.", "norm2": "ln2."}
        layers = [LayerSpec("prenorm", m, ffn, norm, f"blocks.{i}.", dict(names))
                  for i, m in enumerate([att, mean, att])]
        # layer 0, layer 1 (state), layer 0 again (a second cache entry), layer 2 reading entry 0
        schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                    ScheduleEntry(2, 0, writes=False)]
        return ModelSpec(H, V, layers, schedule,
                         PartSpec("embedding", {"name": "emb.", "vocab_size": V, "hidden_size": H}),
                         PartSpec("rmsnorm", {"name": "ln_f.", "size": H, "eps": EPS}),
                         PartSpec("lm_head", {"name": "head.", "tied": True, "vocab_size": V, "hidden_size": H}),
                         self.n_positions, None, [])


def plain_toy(w, ids):
    """The toy model in float64, whole sequence, with the plain implementation's functions."""
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
        h = plain.rms_norm(x, w[p + "ln2.weight"], EPS)
        x = x + plain.swiglu_ffn(h, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                                 w[p + "ffn.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["ln_f.weight"], EPS), w["emb.weight"])


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    register_architecture("ToyMixForCausalLM", ToyConfig)
    d = str(tmp_path_factory.mktemp("toy"))
    write_random_model(ToyConfig(), d, seed=3, dtype=torch.float32)
    yield d
    unregister_architecture("ToyMixForCausalLM")


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_toy_architecture_steps_like_its_plain_twin(toy_folder, dtype, tol):
    _, w = plain.load_weights(toy_folder)
    if dtype == "bfloat16":   # the engine rounds the stored float32 matrices; give the twin the same
        w = {k: (torch.tensor(v).bfloat16().double().numpy() if "ln" not in k else v) for k, v in w.items()}
    eng = Engine.from_folder(toy_folder, EngineOptions(dtype=dtype, max_tokens=512, page_size=16, max_batch=3))
    assert len(eng.cache.paged) == 1 and len(eng.cache.paged[0].entries) == 2   # entries 0 and 2
    assert len(eng.cache.states) == 1 and eng.cache.states[0].state.shape == (1, 3, H + 1)
    rng = np.random.default_rng(0)
    reqs = [rng.integers(0, V, n).tolist() for n in (70, 9, 33, 50)]
    refs = [plain_toy(w, r) for r in reqs]
    for batch, pre in (([0, 1, 2], [40, 9, 1]), ([3, 1], [17, 5])):     # the second batch reuses slots
        slots = {r: eng.new_sequence() for r in batch}
        lg = eng.step([StepItem(slots[r], reqs[r][:p], list(range(p))) for r, p in zip(batch, pre)]).cpu().numpy()
        off = 0
        for r, p in zip(batch, pre):
            assert rel_err(lg[off:off + p], refs[r][:p]) <= tol
            off += p
        pos = dict(zip(batch, pre))
        live = [r for r in batch if pos[r] < len(reqs[r])]
        while live:
            lg = eng.step([StepItem(slots[r], [reqs[r][pos[r]]], [0]) for r in live]).cpu().numpy()
            for i, r in enumerate(live):
                assert rel_err(lg[i], refs[r][pos[r]]) <= tol, (r, pos[r])
                pos[r] += 1
            live = [r for r in live if pos[r] < len(reqs[r])]
        for s in slots.values():
            eng.end_sequence(s)
    eng.check_device_errors()
    eng.cache.check()
