"""Helpers of the GPU tests: tolerances and engine construction."""
import numpy as np

# Bounds on max |difference| relative to max |reference| of the compared block.  float32: a few
# ulps of accumulated rounding against the float64 plain implementation.  bfloat16: activations
# and matrices carry 8 bits of mantissa.  They are fixed; a failure is a fault, not a reason to
# widen them.
F32_TOL = 2e-5
BF16_TOL = 4e-2
TOL = {"float32": F32_TOL, "bfloat16": BF16_TOL}
# Beside the largest difference, the mean of |difference| and the mean of the signed difference, both
# relative to max |reference| (the three figures of the reference's own checker, test/checker.cpp:46-99):
# a wrong rounding point or a bias shows in the means long before it reaches the bound on the maximum.
MEAN_TOL = {"float32": 2e-6, "bfloat16": 8e-3}
BIAS_TOL = {"float32": 5e-7, "bfloat16": 2e-3}


def rel_err(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), "non-finite values in the engine's output"
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def assert_close(got, ref, dtype, what=""):
    e = rel_err(got, ref)
    assert e <= TOL[dtype], f"{what}: relative error {e:.3e} exceeds {TOL[dtype]:.1e} ({dtype})"
    diff = np.asarray(got, np.float64) - np.asarray(ref, np.float64)
    top = max(np.abs(np.asarray(ref, np.float64)).max(), 1e-30)
    mean, bias = float(np.abs(diff).mean() / top), float(abs(diff.mean()) / top)
    assert mean <= MEAN_TOL[dtype], f"{what}: mean |difference| {mean:.3e} exceeds {MEAN_TOL[dtype]:.1e} ({dtype})"
    if diff.size >= 4096:       # the mean of few numbers is no evidence of a bias
        assert bias <= BIAS_TOL[dtype], f"{what}: mean difference {bias:.3e} exceeds {BIAS_TOL[dtype]:.1e} ({dtype})"
    return e


def make_engine(folder, dtype, max_tokens=1024, page_size=64, max_batch=None, max_seq_len=None, poison=False):
    from inferllm_b200 import Engine, EngineOptions
    return Engine.from_folder(folder, EngineOptions(
        dtype=dtype, max_tokens=max_tokens, page_size=page_size, max_batch=max_batch,
        max_seq_len=max_seq_len, poison_freed_pages=poison))


class PartHarness:
    """The minimum an engine gives a part under test: a runtime, a cache for the part's request
    and step contexts made the way the engine makes them."""

    def __init__(self, requests, dtype, num_slots=4, num_pages=16, page_size=16, max_seq_len=256):
        import torch

        from inferllm_b200.cache import SequenceCache
        from inferllm_b200.parts import Runtime
        self.rt = Runtime(torch.device("cuda"), {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype],
                          page_size)
        self.cache = SequenceCache(requests, num_slots, num_pages, page_size, max_seq_len, self.rt)
        self.err = torch.zeros(1, dtype=torch.int32, device="cuda")
        self._stages = [(None, None, None)] * 4
        self._stage_next = 0

    def _upload(self, parts, offs, total, into=None):
        from inferllm_b200.engine import Engine
        return Engine._upload(self, parts, offs, total, into)

    def context(self, slots, q_lens, ids=None, want=()):
        from inferllm_b200.engine import StepContext
        plan = self.cache.plan_step(slots, q_lens)
        ctx = StepContext(self, plan, ids if ids is not None else [0] * sum(q_lens), list(want))
        return ctx, plan
