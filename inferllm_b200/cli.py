"""Command line in the manner of the reference's `llama` program.

Options keep the reference's names and meanings where it has them
(`app_params_parse`, application/llama/llama.cpp:88-128; defaults :20-41):
  -m/--model, -g, -d/--dtype, -c/--ctx_size, -s/--seed, -t/--threads, --top_k, --top_p,
  --temp, --repeat_penalty, --repeat_last_n, --mmap, -v/--version.
What differs: `-m` names a model folder (config.json + safetensors) instead of a .bin file;
`-g` takes "GPU" or a GPU ordinal ("CPU" is refused: there is no CPU path); `-d` takes
bfloat16 or float32; prompts are token ids, since tokenisation is outside this library:
`--prompt-ids "1,5,9"` (repeatable), `--prompt-file FILE` (one request per line) or
`--random-prompts "5,9,16"` (lengths); `-n` is the reference's n_predict field (128, never
parsed there).  `--random-weights SEED` with `--config FILE` writes nothing and runs a model
with random weights; `--write-random-model DIR` writes such a model folder and exits.
"""
from __future__ import annotations

import argparse
import json
import random
import sys


def build_parser():
    ap = argparse.ArgumentParser(prog="llama", description=__doc__.split("\n\n")[0])
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("-g", dest="device", default="GPU", help="GPU, or a GPU ordinal (default GPU = 0)")
    ap.add_argument("-d", "--dtype", default="bfloat16", help="compute dtype: bfloat16 | float32")
    ap.add_argument("-c", "--ctx_size", type=int, default=2048, help="longest sequence (default 2048)")
    ap.add_argument("-s", "--seed", type=int, default=-1, help="RNG seed (default -1: from the clock)")
    ap.add_argument("-t", "--threads", type=int, default=4, help="accepted for compatibility; no effect")
    ap.add_argument("-n", "--n_predict", type=int, default=128, help="new tokens per request")
    ap.add_argument("--top_k", type=int, default=40)
    ap.add_argument("--top_p", type=float, default=0.95)
    ap.add_argument("--temp", type=float, default=0.10, help="temperature; 0 = greedy")
    ap.add_argument("--repeat_last_n", type=int, default=64)
    ap.add_argument("--repeat_penalty", type=float, default=1.30)
    ap.add_argument("--mmap", action="store_true", help="accepted; weight files are always mapped")
    ap.add_argument("--color", action="store_true", help="accepted; no effect")
    ap.add_argument("-v", "--version", type=int, default=2, help="accepted; the model class comes from config.json")
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids")
    ap.add_argument("--prompt-file", help="file with one request (comma- or space-separated ids) per line")
    ap.add_argument("--random-prompts", help="comma-separated prompt lengths of random ids")
    ap.add_argument("--max-tokens", type=int, help="tokens the cache holds (default: fits all requests at once, up to 64 Ki)")
    ap.add_argument("--config", help="config.json for --random-weights / --write-random-model")
    ap.add_argument("--random-weights", type=int, metavar="SEED")
    ap.add_argument("--write-random-model", metavar="DIR")
    ap.add_argument("--no-stop", action="store_true", help="ignore the end token")
    return ap


def _ids(text):
    return [int(x) for x in text.replace(",", " ").split()]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from . import Model, ModelConfig, config_from_dict, write_random_model

    if args.device.upper() == "CPU":
        print("llama: -g CPU is not supported: this library runs on one CUDA GPU only", file=sys.stderr)
        return 2
    device_id = 0 if args.device.upper() == "GPU" else int(args.device)
    dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype)

    cfg = None
    if args.config:
        with open(args.config) as f:
            cfg = config_from_dict(json.load(f))
    if args.write_random_model:
        if cfg is None:
            print("llama: --write-random-model needs --config", file=sys.stderr)
            return 2
        import torch
        write_random_model(cfg, args.write_random_model, args.random_weights or 0,
                           torch.float32 if dtype == "float32" else torch.bfloat16)
        print(f"wrote {args.write_random_model}")
        return 0

    prompts = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    vocab_hint = cfg.vocab_size if cfg is not None else None
    if args.random_prompts:
        if vocab_hint is None:
            with open(f"{args.model}/config.json") as f:
                vocab_hint = json.load(f)["vocab_size"]
        rng = random.Random(args.seed if args.seed >= 0 else None)
        prompts += [[rng.randrange(vocab_hint) for _ in range(n)] for n in _ids(args.random_prompts)]
    if not prompts:
        print("llama: no prompt given (--prompt-ids, --prompt-file or --random-prompts)", file=sys.stderr)
        return 2

    need = sum(-(-min(len(p) + args.n_predict, args.ctx_size) // 64) * 64 for p in prompts)
    max_tokens = args.max_tokens or min(need, 65536)
    model = Model(ModelConfig(compt_type=dtype, device_type="gpu", nr_thread=args.threads,
                              nr_ctx=args.ctx_size, device_id=device_id, enable_mmap=args.mmap,
                              max_tokens=max_tokens))
    if args.random_weights is not None and cfg is not None:
        model.load_random(cfg, args.random_weights)
    elif args.model:
        model.load(args.model)
    else:
        print("llama: give -m DIR, or --config FILE with --random-weights SEED", file=sys.stderr)
        return 2
    end_token = model.end_token if model.end_token is not None else 2
    model.init(args.top_k, args.top_p, args.temp, args.repeat_penalty, args.repeat_last_n,
               args.seed, end_token)
    res = model.generate(prompts, args.n_predict, stop_ids=[] if args.no_stop else None)
    for i, (toks, why) in enumerate(zip(res.tokens, res.finish)):
        print(f"[{i}] {why}: " + ",".join(str(t) for t in toks))
    print(res.summary(), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
