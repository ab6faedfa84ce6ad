#!/usr/bin/env python3
"""Benchmark of inferllm_b200 on one B200: decode tokens per second of a LLaMA-2-7B-sized
model with random weights (the headline: batch 8 at the end of a 4096-token context), the same
through the Python entry point with host tokens in and out, a 2,048-token prefill, and decode
at batch 1 and 64 at the start, the middle and the end of the context.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Timing is by CUDA events on the launching
stream after the warm-up steps; every step reads all weights (13 GB, far larger than the L2),
so nothing is served from cache between steps.  The reference (MegEngine/InferLLM) publishes
only CPU int4 numbers for this architecture (docs/profile.md: 3.2-12.7 tok/s) and no GPU number,
so `vs_baseline` is null.  `--impl reference` builds the unmodified reference with its own CMake
files and times its public `Model` API (baseline/reference_arm.py): float32, one sequence, a
model of the same layer sizes with 4 of the 32 layers; `points.ref_like_*` of this program's own
line are measured at exactly that configuration.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# LLaMA-2-7B size (32 layers of width 4096, 32 heads of 128, feed-forward 11008, 32000 words), context 4096
CONFIG_7B = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=32, head_dim=128,
                 intermediate_size=11008, vocab_size=32000, rope_theta=10000.0, rms_norm_eps=1e-5,
                 max_position_embeddings=4096, tie_word_embeddings=False)
# Llama-3-8B size (8 KV heads, feed-forward 14336, 128256 words) and LLaMA-2-13B size (40 layers of
# width 5120), for runs beside the default one (--model 8b / 13b)
CONFIG_8B = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
                 vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=8192,
                 tie_word_embeddings=False)
CONFIG_13B = dict(architectures=["LlamaForCausalLM"], hidden_size=5120, num_hidden_layers=40,
                  num_attention_heads=40, num_key_value_heads=40, head_dim=128, intermediate_size=13824,
                  vocab_size=32000, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=4096,
                  tie_word_embeddings=False)
MODELS = {"7b": ("LLaMA-2-7B size", CONFIG_7B), "8b": ("Llama-3-8B size", CONFIG_8B),
          "13b": ("LLaMA-2-13B size", CONFIG_13B)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device=0):
        self.samples, self.times, self.proc, self.device = [], [], None, device

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)
                self.times.append(time.time())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, begin=None, end=None):
        """Median SM clock and the throttle reasons seen; `begin`, `end` (wall-clock seconds): only
        the samples taken between them, if there are at least two (a sample is up to a period late)."""
        samples = self.samples
        if begin is not None and end is not None:
            inside = [s for s, t in zip(self.samples, self.times) if begin <= t <= end + 0.1]
            if len(inside) >= 2:
                samples = inside
        if not samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(s[0]) for s in samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(samples[0][1]), "reasons": reasons,
                "samples": len(mhz)}


def _has(program):
    import shutil
    return shutil.which(program) is not None


def model_figures(cfg, n_layers):
    """Bytes and flops of one step, from the configuration."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * d * H + H * nh * d + 3 * H * I          # matrix elements
    matrix = n_layers * per_layer + V * H                                # + the output matrix
    norms = (2 * n_layers + 1) * H
    weight_bytes = 2 * (matrix + norms)
    kv_bytes_per_token = 2 * nkv * d * 2 * n_layers
    return {"matrix_elems": matrix, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token,
            "layer_matrix_elems": per_layer}


def prefill_flops(cfg, n_layers, T, fig):
    nh, d = cfg["num_attention_heads"], cfg["head_dim"]
    linear = 2 * T * (n_layers * fig["layer_matrix_elems"]) + 2 * 1 * cfg["vocab_size"] * cfg["hidden_size"]
    attn = n_layers * nh * 4 * d * (T * (T + 1) // 2)                     # QK^T and PV over the causal half
    return linear + attn


SCENARIOS = {"8b": "16:64:2048:256", "13b": "32:128:1024:to4096", "7b": "8:512:512:256"}
REF_LIKE_LAYERS = 4            # layers of the model that the reference arm runs (baseline/reference_arm.py)


def run_kernels(pk, pk_src, only=None):
    """The hot kernels one by one at several sizes (beside the contract): each is replayed from a
    CUDA graph of several launches on different buffers (so that nothing is served from L2 by the
    launch before), timed with events, and printed as one JSON line with its algorithmic bytes or
    flops against the peaks."""
    import math

    import torch

    from inferllm_b200.kernels import ops

    dev = torch.device("cuda")
    torch.manual_seed(0)

    side = torch.cuda.Stream()

    def graph_us(fns, reps=10):
        # warm-up and capture on one stream: the library keeps a context (working memory, error word)
        # per stream for calls outside an engine, which has to exist before the capture begins
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for f in fns:
                f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps / len(fns) * 1e3

    def emit(kernel, size, us, nbytes=None, flops=None):
        line = {"kernel": kernel, "size": size, "us": round(us, 1)}
        if nbytes is not None:
            line["GB_per_s"] = round(nbytes / us / 1e3, 0)
            line["frac_of_hbm"] = round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)
        if flops is not None:
            line["TF_per_s"] = round(flops / us / 1e6, 0)
            line["frac_of_bf16"] = round(flops / us / 1e6 / pk["bf16_tflops"], 3)
        line["peaks"] = pk_src
        print(json.dumps(line), flush=True)

    def want(section):
        return only is None or only in section

    d, page = 128, 64
    # ---- decode attention (the position encoding and the cache write inside)
    for B, nh, nkv, ctx in () if not want("attention_decode_ring") else ((1, 32, 32, 512), (1, 32, 32, 4096), (8, 32, 32, 512), (8, 32, 32, 4096), (64, 32, 32, 512),
                            (64, 32, 32, 4096), (8, 32, 8, 4096), (1, 32, 8, 32768), (16, 32, 8, 16384), (8, 40, 40, 4096)):
        per = -(-ctx // page)
        n_l = max(2, min(8, int(2e9 // (B * per * page * nkv * d * 4)) or 2))
        kc = torch.randn(n_l, B * per, nkv, page, d, device=dev).bfloat16()
        vc = torch.randn_like(kc)
        table = torch.arange(B * per, dtype=torch.int32, device=dev).view(B, per)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        seq = torch.arange(B, dtype=torch.int32, device=dev)
        qkv = torch.randn(B, (nh + 2 * nkv) * d, device=dev).bfloat16()
        cs = torch.randn(ctx, d // 2, 2, device=dev)
        err = torch.zeros(1, dtype=torch.int32, device=dev)
        us = graph_us([lambda i=i: ops.attention_decode_ring(qkv, kc[i], vc[i], table, pos, seq, nh, nkv, d, page, None,
                                                             0.088, ctx, rope=(cs, d, True, err)) for i in range(n_l)])
        emit("attention_decode_ring (fused)", f"batch {B}, {nh} heads over {nkv}, context {ctx}", us,
             nbytes=B * ctx * nkv * d * 4)
        del kc, vc
    # ---- decode-sized products (weights of the three model sizes)
    shapes = {"7B qkv": (12288, 4096), "7B o": (4096, 4096), "7B gate/up+act": (22016, 4096), "7B down": (4096, 11008),
              "7B head": (32000, 4096), "8B qkv": (6144, 4096), "8B gate/up+act": (28672, 4096), "8B down": (4096, 14336),
              "8B head": (128256, 4096), "13B qkv": (15360, 5120), "13B gate/up+act": (27648, 5120), "13B down": (5120, 13824)}
    for name, (N, K) in shapes.items() if want("gemm_tc (decode)") else ():
        n_w = max(2, min(6, int(1.5e9 // (N * K * 2))))
        ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(n_w)]
        for M in (1, 8, 16):
            x = torch.randn(M, K, device=dev).bfloat16()
            # the kernels themselves with the engine's choice of K slices (the slices stay unreduced, as in a step)
            if "act" in name and ops.gemm_tc_splits(M, N, K) == 1:
                us = graph_us([lambda w=w: ops.gemm_bf16_tc_gated(x, w) for w in ws])
            else:
                us = graph_us([lambda w=w: ops.gemm_bf16_tc(x, w, torch.float32, defer_reduce=True) for w in ws])
            emit("gemm_tc (decode)", f"{name}, {M} tokens", us, nbytes=N * K * 2)
        del ws
    # ---- the float32 mode's product of a few rows (true float32: no tensor cores, one chain of FMAs per output)
    for name, (N, K) in shapes.items() if want("gemm_f32 (decode)") else ():
        if not name.startswith("7B"):
            continue
        n_w = max(2, min(4, int(1.5e9 // (N * K * 4))))
        ws = [torch.randn(N, K, device=dev) * 0.02 for _ in range(n_w)]
        for M in (1, 4, 8):
            x = torch.randn(M, K, device=dev)
            us = graph_us([lambda w=w: ops.gemm_f32(x, w) for w in ws])
            emit("gemm_f32 (decode)", f"{name.replace('+act', '')}, {M} tokens", us, nbytes=N * K * 4)
        del ws
    # ---- prompt attention
    for T, nh, nkv in () if not want("attention_prefill_tc") else ((512, 32, 32), (2048, 32, 32), (2048, 32, 8), (8192, 32, 32), (16384, 32, 32), (16384, 32, 8)):
        n_pages = T // page
        kc = torch.randn(n_pages, nkv, page, d, device=dev).bfloat16()
        vc = torch.randn_like(kc)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
        qkv = torch.randn(T, (nh + 2 * nkv) * d, device=dev).bfloat16()
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        sl = torch.tensor([T], dtype=torch.int32, device=dev)
        us = graph_us([lambda: ops.attention_prefill_tc(qkv, kc, vc, table, cu, sl, T, nh, nkv, d, page, None, 0.088)] * 3)
        emit("attention_prefill_tc", f"prompt of {T}, {nh} heads over {nkv}", us, flops=4 * nh * d * T * (T + 1) / 2)
        del kc, vc, qkv
    # ---- prompt-sized products on the SM-pair kernel, and the library beside them
    x = torch.randn(2048, 4096, device=dev).bfloat16()
    for name, (N, K) in () if not want("gemm_tc2") else (("7B qkv", (12288, 4096)), ("7B gate/up+act", (22016, 4096)), ("7B down", (4096, 11008))):
        xx = x if K == 4096 else torch.randn(2048, K, device=dev).bfloat16()
        ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(3)]
        gated = "act" in name
        us = graph_us([lambda w=w: ops.gemm_bf16_tc2(xx, w, torch.bfloat16, gated=gated) for w in ws])
        emit("gemm_tc2", f"{name}, 2048 tokens", us, flops=2 * 2048 * N * K)
        if gated:
            us = graph_us([lambda w=w: ops.swiglu(torch.mm(xx, w.t())) for w in ws])
        else:
            us = graph_us([lambda w=w: torch.mm(xx, w.t()) for w in ws])
        emit("library (cuBLAS)" + (" + swiglu" if gated else ""), f"{name}, 2048 tokens", us, flops=2 * 2048 * N * K)
        del ws
    # ---- the memory-bound kernels of a prompt step (2,048 tokens of a 7B layer)
    if not want("add_rmsnorm, rope_kv_write"):
        return 0
    T, H, I, nh, nkv = 2048, 4096, 11008, 32, 32
    resid = [torch.randn(T, H, device=dev) for _ in range(4)]
    delta = [torch.randn(T, H, device=dev).bfloat16() for _ in range(4)]
    wn = torch.ones(H, device=dev).bfloat16()
    us = graph_us([lambda i=i: ops.add_rmsnorm(resid[i], delta[i], wn, 1e-5, torch.bfloat16) for i in range(4)])
    emit("add_rmsnorm", "2048 tokens x 4096", us, nbytes=T * H * 12)
    qs = [torch.randn(T, (nh + 2 * nkv) * d, device=dev).bfloat16() for _ in range(4)]
    kcs = [torch.zeros(T // page, nkv, page, d, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    vcs = [torch.zeros_like(k) for k in kcs]
    cs = torch.randn(4096, d // 2, 2, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    table = torch.arange(T // page, dtype=torch.int32, device=dev).view(1, -1)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    us = graph_us([lambda i=i: ops.rope_kv_write(qs[i], cs, d, pos, seq, table, kcs[i], vcs[i], nh, nkv, d, page, True, err)
                   for i in range(4)])
    emit("rope_kv_write", "2048 tokens, 32 + 2 x 32 heads of 128", us, nbytes=T * (nh + 2 * nkv) * d * 4)
    gu = [torch.randn(T, 2 * I, device=dev).bfloat16() for _ in range(4)]
    us = graph_us([lambda i=i: ops.swiglu(gu[i]) for i in range(4)])
    emit("swiglu", "2048 tokens x 11008", us, nbytes=T * I * 6)
    return 0


def run_scenario(args, cfg, cfgd, model_name, L, fig, pk, pk_src):
    """An unequal batch through `Model.generate`: one prompt step, then one token per sequence and
    step, host token ids in and out.  Prints one JSON line with prompt and decode tokens per second
    and the fraction of the memory rate the decode steps reach (weights once per step plus the live
    cache at the mean context)."""
    import torch

    from inferllm_b200 import Model, ModelConfig
    from inferllm_b200.kernels import ops

    spec = SCENARIOS[args.model] if args.scenario == "config" else args.scenario
    B, lo, hi = (int(x) for x in spec.split(":")[:3])
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(lo, hi + 1, (B,), generator=g).tolist()
    new = spec.split(":")[3]
    # "toN": every sequence decodes until the longest prompt's sequence stands at position N
    new = int(new[2:]) - max(lens) - 1 if new.startswith("to") else int(new)
    prompts = [torch.randint(0, cfgd["vocab_size"], (n,), generator=g).tolist() for n in lens]
    ctx = max(lens) + new + 1
    max_tokens = sum(-(-(n + new + 1) // 64) * 64 for n in lens) + 64
    model = Model(ModelConfig(compt_type="bfloat16", nr_ctx=ctx, max_tokens=max_tokens, max_batch=B, gemm=args.gemm))
    model.load_random(cfg, seed=0)
    model.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=0, end_token=-1)
    # warm-up with the same prompts: the step's working memory has grown to this step's size, the
    # library has chosen its kernels for these shapes, the decode graph of this batch is captured
    model.generate(prompts, max_new_tokens=4, stop_ids=[])
    with ClockSampler() as cs:
        res = model.generate(prompts, max_new_tokens=new, stop_ids=[])
    steps = res.step_s[max(3, args.warmup):]
    dec_ms = sum(steps) / len(steps) * 1e3
    mean_ctx = sum(lens) / B + new - len(steps) / 2
    step_bytes = fig["weight_bytes"] + B * mean_ctx * fig["kv_bytes_per_token"]
    pf_flops = sum(prefill_flops(cfgd, L, n, fig) for n in lens)
    print(json.dumps({
        "scenario": spec, "model": model_name, "layers": L, "batch": B, "prompt_lengths": [min(lens), max(lens)],
        "prompt_tokens": sum(lens), "new_tokens_each": new, "last_position": max(lens) + new,
        "prefill": {"tokens_per_s": round(res.prefill_tokens / res.prefill_s, 1), "ms": round(res.prefill_s * 1e3, 2),
                    "frac": round(pf_flops / res.prefill_s / (pk["bf16_tflops"] * 1e12), 4)},
        "decode": {"tokens_per_s": round(B / dec_ms * 1e3, 1), "ms_per_step": round(dec_ms, 4),
                   "steps_timed": len(steps), "hbm_frac": round(step_bytes / (dec_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)},
        "peaks": pk_src, "clocks": cs.summary(), "gpu_launches": ops.launch_count()}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--only", choices=["decode", "prefill"], help="run one scenario (for profiling); "
                    "prints a short JSON line of that scenario only")
    ap.add_argument("--model", default="7b", choices=sorted(MODELS), help="LLaMA-2-7B (default), Llama-3-8B or LLaMA-2-13B sizes")
    ap.add_argument("--gemm", default="auto", choices=["auto", "tc", "library"])
    ap.add_argument("--no-pdl", action="store_true", help="launch kernels without programmatic dependent launch")
    ap.add_argument("--context", type=int, default=CONTEXT, help="position at which the timed decode steps end")
    ap.add_argument("--timeline", action="store_true", help="with --only decode: print when every kernel of one "
                    "step starts and ends inside the captured graph")
    ap.add_argument("--kernels", action="store_true", help="beside the contract: the hot kernels one by one at "
                    "several sizes, one JSON line each")
    ap.add_argument("--kernel", metavar="NAME", help="with --kernels: only the section whose name holds NAME "
                    "(attention_decode_ring, gemm_tc (decode), gemm_f32 (decode), attention_prefill_tc, gemm_tc2, add_rmsnorm)")
    ap.add_argument("--scenario", metavar="B:MIN:MAX:NEW", help="beside the contract: B prompts of random ids with "
                    "lengths uniform in [MIN, MAX] (seeded) prefilled in one step of unequal lengths, then NEW tokens "
                    "each (or 'toN': until position N), through the Python entry point; 'config' = the workload of --model "
                    "(8b: 16:64:2048:256, 13b: 32:128:1024:to4096)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: inferllm_b200 is a single-GPU library; --gpus {args.gpus} is not supported (N=1 only)")
        return 2
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
        gpu = subprocess.run(["nvidia-smi", "-L"], capture_output=True).returncode == 0 if _has("nvidia-smi") else False
        with ClockSampler() as cs:
            line = reference_arm.run(args.steps, args.warmup, layers=REF_LIKE_LAYERS, gpu_visible=gpu)
        if "unavailable" not in line:
            # the clocks of the timed calls alone (the run also writes and loads a model file)
            line["clocks"] = cs.summary(*line.pop("timed_window_unix", (None, None)))
            line["gpu_launches"] = 0        # none of this repository's kernels run in the reference arm
        print(json.dumps(line))
        return 0
    K, W = args.steps, max(3, args.warmup)

    import torch

    from inferllm_b200 import Model, ModelConfig, StepItem, config_from_dict
    from inferllm_b200.kernels import ops

    model_name, base_cfg = MODELS[args.model]
    cfgd = dict(base_cfg)
    full_layers = cfgd["num_hidden_layers"]
    if args.layers:
        cfgd["num_hidden_layers"] = args.layers
    L = cfgd["num_hidden_layers"]
    cfg = config_from_dict(cfgd)
    fig = model_figures(cfgd, L)
    pk, pk_src = peaks()
    B = args.batch

    if args.kernels:
        return run_kernels(pk, pk_src, args.kernel)
    if args.scenario:
        return run_scenario(args, cfg, cfgd, model_name, L, fig, pk, pk_src)

    # one engine for every scenario: cache for 64 sequences at the full context (137 GB at 7B size),
    # or for the batch alone where only that is run
    decode_room = K + W + 8
    if args.only == "decode":           # one scenario: room for the batch at the context asked for
        max_tokens = B * (-(-(args.context + 8) // 64) * 64) + 64
    elif args.skip_points:
        max_tokens = max(B * CONTEXT, PREFILL_TOKENS) + 64
    else:
        max_tokens = max(B, 64) * CONTEXT + 64
    model = Model(ModelConfig(compt_type="bfloat16", nr_ctx=CONTEXT, max_tokens=max_tokens, max_batch=max(B, 64), gemm=args.gemm))
    model.load_random(cfg, seed=0)
    if args.no_pdl:
        ops.set_pdl(False)
    model.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=0, end_token=-1)
    eng = model.engine
    g = torch.Generator().manual_seed(0)

    def rand_ids(n, vocab=cfgd["vocab_size"]):
        return torch.randint(0, vocab, (n,), generator=g).tolist()

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    # ---- decode: `batch` sequences, timed steps end at position `ctx_end`
    def decode_run(engine, batch, ctx_end, steps, warm, timeline=False):
        start = ctx_end - steps - warm - (3 if timeline else 0)     # the timeline takes three steps of its own
        slots = [engine.new_sequence() for _ in range(batch)]
        per_step = max(1, 8192 // start)                  # prompts go in steps of about 8k tokens
        for i in range(0, batch, per_step):
            engine.step([StepItem(s, rand_ids(start), []) for s in slots[i:i + per_step]])
        toks = [[t] for t in rand_ids(batch)]

        def one():
            engine.step([StepItem(s, t, [0]) for s, t in zip(slots, toks)])

        for _ in range(warm):
            one()
        if timeline:
            print_timeline(one)
        before = ops.launch_count()
        ms = timed(one, steps)
        launches = ops.launch_count() - before
        for s in slots:
            engine.end_sequence(s)
        return ms, launches

    def print_timeline(one):
        """Start and duration of every kernel of one step inside its captured graph, from the driver's
        activity records (torch.profiler over CUPTI; no replay, no serialisation: the kernels overlap as
        they do in a timed run, each some microseconds slower for the tracing)."""
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                one()
            torch.cuda.synchronize()
        ev = sorted((e for e in prof.events() if e.device_type.name == "CUDA"), key=lambda e: e.time_range.start)
        last = ev[-(len(ev) // 3):]                 # the third step
        t0, latest = last[0].time_range.start, last[0].time_range.start
        print("   start     ends  since the latest end before it   kernel")
        for e in last:
            start, end = e.time_range.start - t0, e.time_range.end - t0
            print(f"{start:8.1f} {end:8.1f}   {e.time_range.end - max(latest, e.time_range.start):+7.1f} us   {e.name[:64]}")
            latest = max(latest, e.time_range.end)
        print(f"step: {latest - t0:.1f} us")

    def hbm_frac(figures, batch, ctx_end, steps, ms):
        nbytes = figures["weight_bytes"] + batch * (ctx_end - steps // 2) * figures["kv_bytes_per_token"]
        return nbytes, nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]

    if args.only == "decode":
        ms, launches = decode_run(eng, B, args.context, K, W, timeline=args.timeline)
        print(json.dumps({"only": "decode", "batch": B, "layers": L, "context": args.context,
                          "ms_per_step": round(ms, 4), "gpu_launches": launches}))
        return 0

    # the clocks are sampled over all timed regions together (one region alone is a tenth of a second)
    sampler = ClockSampler()
    sampler.__enter__()

    # ---- prefill of one 2,048-token prompt
    prompt = rand_ids(PREFILL_TOKENS)

    def prefill_once():
        s = eng.new_sequence()
        eng.step([StepItem(s, prompt, [PREFILL_TOKENS - 1])])
        eng.end_sequence(s)

    for _ in range(3):
        prefill_once()
    pf_ms = timed(prefill_once, 3)
    if args.only == "prefill":
        sampler.__exit__()
        print(json.dumps({"only": "prefill", "layers": L, "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3)}))
        return 0
    pf_flops = prefill_flops(cfgd, L, PREFILL_TOKENS, fig)
    prefill = {"value": round(PREFILL_TOKENS / pf_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
               "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "frac_of_sustained": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
               "tflops": round(pf_flops / (pf_ms * 1e-3) / 1e12, 1)}

    ms, launches = decode_run(eng, B, CONTEXT, K, W)
    value = B / ms * 1e3
    step_bytes, frac = hbm_frac(fig, B, CONTEXT, K, ms)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(frac, 4), "peak_source": pk_src, "bytes_per_step": step_bytes}

    # ---- the same through the Python entry point: host token ids in, host token ids out, every
    # step; W warm-up steps after the prompt, then K timed steps that end at the same position
    # (the first few dozen steps after a batch of long prompts run slower while the GPU comes back from
    # the power cap the prompts drove it into; they are warm-up here as the separate prompt phase is above)
    We = max(W, 48)
    plen = CONTEXT - K - We - 1
    model.generate([rand_ids(64) for _ in range(B)], max_new_tokens=4, stop_ids=[])      # compile/capture
    res = model.generate([rand_ids(plen) for _ in range(B)], max_new_tokens=K + We + 1, stop_ids=[])
    timed_steps = res.step_s[-K:]
    e2e_val = B * len(timed_steps) / sum(timed_steps)
    h2d = eng.last_upload_bytes          # token ids, positions, slots and page table of the last step
    e2e = {"value": round(e2e_val, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B,
           "steps": len(timed_steps), "warmup": res.decode_steps - len(timed_steps)}

    # ---- batch 1 and 64 at the start (prompts of 512 tokens), the middle and the end of the context,
    # each with the fraction of the memory rate it reaches
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            for ctx_end, name in ((512 + K + W, f"decode_b{b}"), (CONTEXT // 2, f"decode_b{b}_ctx{CONTEXT // 2}"),
                                  (CONTEXT, f"decode_b{b}_ctx{CONTEXT}")):
                pms, _ = decode_run(eng, b, ctx_end, K, W)
                points[name] = round(b / pms * 1e3, 1)
                points[name + "_hbm_frac"] = round(hbm_frac(fig, b, ctx_end, K, pms)[1], 4)
        pms, _ = decode_run(eng, B, 512 + K + W, K, W)
        points[f"decode_b{B}_ctx512"] = round(B / pms * 1e3, 1)
        points[f"decode_b{B}_ctx512_hbm_frac"] = round(hbm_frac(fig, B, 512 + K + W, K, pms)[1], 4)
        points["ctx_of_b1_b64"] = 512
        # ---- what the reference arm measures (`--impl reference`): one sequence at context 512 of a model
        # with the same layer sizes and REF_LIKE_LAYERS layers, in bfloat16 and in float32
        del model, eng
        torch.cuda.empty_cache()
        like = dict(cfgd, num_hidden_layers=REF_LIKE_LAYERS)
        like_fig = model_figures(like, REF_LIKE_LAYERS)
        for dtype, tag in (("bfloat16", "bf16"), ("float32", "f32")):
            m2 = Model(ModelConfig(compt_type=dtype, nr_ctx=1024, max_tokens=1024, max_batch=1))
            m2.load_random(config_from_dict(like), seed=0)
            pms, _ = decode_run(m2.engine, 1, 512 + K + W, K, W)
            points[f"ref_like_b1_ctx512_{tag}"] = round(1 / pms * 1e3, 1)
            del m2
            torch.cuda.empty_cache()
        points["ref_like_layers"] = REF_LIKE_LAYERS
    sampler.__exit__()
    clocks = sampler.summary()

    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048-token prompt",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": {"model": model_name, "global_batch": B, "seq_len": CONTEXT, "parallelism": "none (1 GPU)",
                   "layers": L, "layers_of_config": full_layers, "hidden": cfgd["hidden_size"],
                   "heads": cfgd["num_attention_heads"], "kv_heads": cfgd["num_key_value_heads"],
                   "head_dim": cfgd["head_dim"], "intermediate": cfgd["intermediate_size"],
                   "vocab": cfgd["vocab_size"], "context_len": CONTEXT,
                   "decode_positions": f"{CONTEXT - K}..{CONTEXT}", "prefill_tokens": PREFILL_TOKENS,
                   "l2": "inputs larger than L2 (13 GB of weights read per step)", "page_size": 64,
                   "peaks": pk_src},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill, "roofline": roofline,
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
