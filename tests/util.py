"""Helpers of the tests: tolerances, engine construction, and a plain generation loop (the oracle of
the library's loop: it looks at every token before it takes the next step and hands the chooser the
whole history every time)."""
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


def _ints(toks):
    return [int(t) for t in (toks.tolist() if hasattr(toks, "tolist") else toks)]


def plain_generate(backend, prompts, choose, max_new_tokens, stop_ids=()):
    """The same decisions without any overlap: step, choose, look, then step again."""
    from inferllm_b200.engine import StepItem, plan_batches
    limits, stop = backend.limits(), set(stop_ids)
    tokens, finish = [[] for _ in prompts], [""] * len(prompts)
    batches = plan_batches([len(p) for p in prompts], max_new_tokens, limits)
    for batch in batches:
        slots = {r: backend.new_sequence() for r in batch}
        hist = {r: list(prompts[r]) for r in batch}
        live = sorted(batch, key=lambda r: -len(prompts[r]))
        toks = _ints(choose(backend.step([StepItem(slots[r], list(prompts[r]), [len(prompts[r]) - 1]) for r in live]), live,
                            [0] * len(live), [hist[r] for r in live]))
        while True:
            nxt = []
            for r, tok in zip(live, toks):
                tokens[r].append(tok)
                hist[r].append(tok)
                if tok in stop:
                    finish[r] = "stop"
                elif len(tokens[r]) >= max_new_tokens:
                    finish[r] = "length"
                elif len(hist[r]) > limits.max_seq_len:
                    finish[r] = "context"
                else:
                    nxt.append(r)
                    continue
                backend.end_sequence(slots.pop(r))
            live = nxt
            if not live:
                break
            toks = _ints(choose(backend.step([StepItem(slots[r], [hist[r][-1]], [0]) for r in live]), live,
                                [len(tokens[r]) for r in live], [hist[r] for r in live]))
    return tokens, finish, batches
