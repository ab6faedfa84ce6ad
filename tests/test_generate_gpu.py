"""Generation through the entry point and the command line against the plain implementation's
greedy continuation, and the sampling options end to end (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import plain_llama as plain
import pytest
from conftest import ROOT, TINY, random_prompt

from inferllm_b200 import Model, ModelConfig
from inferllm_b200.sampling import Sampler, SamplingParams, uniform_for

pytestmark = pytest.mark.gpu


def load(folder, dtype, **kw):
    m = Model(ModelConfig(compt_type=dtype, nr_ctx=kw.pop("nr_ctx", 256), **kw))
    m.load(folder)
    return m


@pytest.mark.parametrize("name,lens,n_new", [("A", [5, 9, 16], 8), ("B", [1, 7, 23, 40], 12)])
def test_greedy_generation_matches_plain(name, lens, n_new, model_folders, plain_models):
    cfg, w = plain_models[name]
    prompts = [random_prompt(name, n, 40 + n) for n in lens]
    want = [plain.greedy_generate(cfg, w, p, n_new) for p in prompts]
    m = load(model_folders[name], "float32", nr_ctx=TINY[name]["max_position_embeddings"], max_tokens=512)
    m.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=0, seed=0, end_token=-1)
    res = m.generate(prompts, max_new_tokens=n_new, stop_ids=[])
    assert res.tokens == want and res.finish == ["length"] * len(lens)
    # bfloat16 may turn a near-tie the other way; the first tokens of every request must agree
    mb = load(model_folders[name], "bfloat16", nr_ctx=TINY[name]["max_position_embeddings"], max_tokens=512)
    mb.init(0, 1.0, 0.0, 1.0, 0, 0, -1)
    got = mb.generate(prompts, max_new_tokens=n_new, stop_ids=[]).tokens
    assert sum(g == w_ for g, w_ in zip(got, want)) >= len(lens) - 1
    assert all(g[0] == w_[0] for g, w_ in zip(got, want))


def test_warm_up_changes_nothing_and_gives_everything_back(model_folders, plain_models):
    """`Model.warm_up` runs prompt steps of every bucket and captures the graphs of the batch sizes
    asked for; afterwards all slots and pages are free and generation gives the same tokens."""
    name = "C"
    cfg, w = plain_models[name]
    prompts = [random_prompt(name, n, 70 + n) for n in (130, 9)]
    want = [plain.greedy_generate(cfg, w, p, 6) for p in prompts]
    m = load(model_folders[name], "float32", nr_ctx=TINY[name]["max_position_embeddings"], max_tokens=1024)
    m.init(0, 1.0, 0.0, 1.0, 0, 0, -1)
    m.warm_up(prompt_tokens=300, batch_sizes=(1, 2, 5000))
    cache = m.engine.cache
    cache.check()
    assert cache.slots_free == cache.num_slots and cache.pages_free() == [cache.num_pages]
    assert m.engine.info()["graphs_captured"] >= 3, "no graph was captured"
    assert m.generate(prompts, max_new_tokens=6, stop_ids=[]).tokens == want


def test_stop_token_ends_early_and_batches_follow_each_other(model_folders, plain_models):
    name = "A"
    cfg, w = plain_models[name]
    prompts = [random_prompt(name, n, 70 + n) for n in (30, 4, 11, 19, 2)]
    free_run = [plain.greedy_generate(cfg, w, p, 10) for p in prompts]
    stop = free_run[1][3]                       # request 1 stops at its 4th token
    want = [plain.greedy_generate(cfg, w, p, 10, stop_ids=[stop]) for p in prompts]
    m = load(model_folders[name], "float32", nr_ctx=128, max_tokens=64 * 2, max_batch=2)   # 2 at a time
    m.init(0, 1.0, 0.0, 1.0, 0, 0, end_token=stop)
    res = m.generate(prompts, max_new_tokens=10)
    assert res.tokens == want
    assert res.batches == [[0, 1], [2, 3], [4]]
    assert res.finish[1] == "stop" and len(res.tokens[1]) <= 4
    m.engine.cache.check()
    assert m.engine.cache.slots_free == 2


def test_single_conversation_api_of_the_reference(model_folders, plain_models):
    """load / init / prefill / decode / decode_iter / get_remain_token / reset_token."""
    name = "B"
    cfg, w = plain_models[name]
    system, user = random_prompt(name, 12, 1), random_prompt(name, 5, 2)
    want = plain.greedy_generate(cfg, w, system + user, 6)
    m = load(model_folders[name], "float32", nr_ctx=64)
    m.init(0, 1.0, 0.0, 1.0, 0, 0, end_token=-1)
    assert m.get_remain_token() == 64
    m.prefill(system)
    assert m.get_remain_token() == 64 - 12
    got = [m.decode(user)]
    for _ in range(5):
        got.append(m.decode_iter())
    assert got == want
    assert m.get_remain_token() == 64 - 12 - 5 - 5
    assert "Total Model Compute Token:  5" in m.decode_summary()
    m.reset_token()
    assert m.get_remain_token() == 64
    assert m.decode(system + user) == want[0]


def test_temperature_sampling_is_reproducible_and_batch_independent(model_folders):
    name = "B"
    prompts = [random_prompt(name, n, 90 + n) for n in (1, 7, 23, 40)]
    m = load(model_folders[name], "float32", nr_ctx=256, max_tokens=1024)
    m.init(top_k=0, top_p=1.0, temp=0.8, repeat_penalty=1.0, repeat_last_n=0, seed=123, end_token=-1)
    a = m.generate(prompts, max_new_tokens=12, stop_ids=[]).tokens
    b = m.generate(prompts, max_new_tokens=12, stop_ids=[]).tokens
    assert a == b
    assert len({tuple(t) for t in a}) == 4
    m.init(0, 1.0, 0.8, 1.0, 0, seed=124, end_token=-1)
    assert m.generate(prompts, max_new_tokens=12, stop_ids=[]).tokens != a
    # request 0 alone draws what it drew in the batch: its random numbers are keyed by
    # (seed, request, step) and its logits do not depend on the batch
    m.init(0, 1.0, 0.8, 1.0, 0, seed=123, end_token=-1)
    assert m.generate(prompts[:1], max_new_tokens=12, stop_ids=[]).tokens[0] == a[0]
    assert 0.0 <= uniform_for(1, 2, 3) < 1.0 and uniform_for(1, 2, 3) != uniform_for(1, 2, 4)


def test_repeat_penalty_changes_greedy_choice(model_folders, plain_models):
    """Greedy with a repetition penalty picks what the reference's sampler ranks first: the
    penalised maximum.  The prompt ends with the model's own favourite, which the penalty demotes."""
    name = "A"
    cfg, w = plain_models[name]
    p = random_prompt(name, 20, 5)
    top = int(np.argmax(plain.forward(cfg, w, p)[-1]))
    prompt = p + [top]
    logits = plain.forward(cfg, w, prompt)[-1]
    ids, _ = plain.sample_distribution(logits, prompt, 1.5, 1, 1.0, 1.0)
    m = load(model_folders[name], "float32", nr_ctx=128)
    m.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.5, repeat_last_n=64, seed=0, end_token=-1)
    tok = m.generate([prompt], max_new_tokens=1, stop_ids=[]).tokens[0][0]
    assert tok == int(ids[0])
    m.init(top_k=0, top_p=1.0, temp=0.0, repeat_penalty=1.0, repeat_last_n=64, seed=0, end_token=-1)
    assert m.generate([prompt], max_new_tokens=1, stop_ids=[]).tokens[0][0] == int(np.argmax(logits))


@pytest.mark.parametrize("temp", [0.0, 0.9])
def test_repeat_penalty_with_the_windows_on_the_device(temp, model_folders):
    """The library's loop keeps the host a step behind and lets the sampler keep the last tokens on the
    device; it must choose what a plain loop chooses that passes the histories from the host at every
    step (unequal prompts, a window shorter than some prompts, sequences ending early).  The plain loop
    is the tests' own (tests/util.py) over the same engine and the same sampling kernels."""
    from util import plain_generate
    name = "B"
    prompts = [random_prompt(name, n, 70 + n) for n in (1, 9, 30, 17)]
    m = load(model_folders[name], "float32", nr_ctx=256, max_tokens=1024)
    params = SamplingParams(temp=temp, top_k=20, top_p=0.9, repeat_penalty=1.4, repeat_last_n=12, seed=5)
    m.init(top_k=20, top_p=0.9, temp=temp, repeat_penalty=1.4, repeat_last_n=12, seed=5, end_token=-1)
    want_tokens, _, _ = plain_generate(m.engine, prompts, Sampler(m.engine, params).choose, 25, [])
    stop = [want_tokens[2][6]]                       # a token request 2 really samples: it ends early
    want_tokens, want_finish, _ = plain_generate(m.engine, prompts, Sampler(m.engine, params).choose, 25, stop)
    got = m.generate(prompts, max_new_tokens=25, stop_ids=stop)
    assert got.tokens == want_tokens and got.finish == want_finish
    assert "stop" in got.finish and "length" in got.finish
    # the library's loop driven from Python over the same engine and sampler agrees as well
    from inferllm_b200.engine import generate
    again = generate(m.engine, prompts, Sampler(m.engine, params).choose, 25, stop)
    assert again.tokens == want_tokens and again.finish == want_finish


def test_command_line(model_folders, plain_models, tmp_path):
    name = "A"
    cfg, w = plain_models[name]
    prompts = [random_prompt(name, n, 60 + n) for n in (6, 13)]
    want = [plain.greedy_generate(cfg, w, p, 5) for p in prompts]
    args = [os.path.join(ROOT, "bin", "llama"), "-m", model_folders[name], "-g", "GPU", "-d", "float32",
            "-c", "128", "-n", "5", "--temp", "0", "--top_k", "0", "--top_p", "1", "--repeat_penalty", "1",
            "--no-stop", "-s", "1"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(args, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("[")]
    got = [[int(t) for t in ln.split(": ")[1].split(",")] for ln in lines]
    assert got == want and "decode:" in r.stderr
    r = subprocess.run([os.path.join(ROOT, "bin", "llama"), "-m", model_folders[name], "-g", "CPU",
                        "--prompt-ids", "1"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "CPU" in r.stderr
    # random weights from a config file, no model folder
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(TINY["B"]))
    r = subprocess.run([os.path.join(ROOT, "bin", "llama"), "--config", str(cfg_file),
                        "--random-weights", "4", "--random-prompts", "3,8", "-n", "4", "-c", "64", "-s", "2"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert len([ln for ln in r.stdout.splitlines() if ln.startswith("[")]) == 2


def test_every_end_token_of_the_configuration_stops_by_default(model_folders, plain_models, tmp_path):
    """config.json may list several end tokens (tiny B has two); without `stop_ids` generation
    stops at any of them, through `Model.generate` and through the command line.  The second of two
    end tokens is made the one that the greedy continuation meets."""
    import shutil
    name = "B"
    cfg, w = plain_models[name]
    prompt = random_prompt(name, 9, 5)
    free = plain.greedy_generate(cfg, w, prompt, 10)
    stop_at = max(i for i in range(10) if free[i] not in free[:i])      # the last token that appears for the first time
    unused = next(t for t in range(TINY[name]["vocab_size"]) if t not in free)
    folder = str(tmp_path / "model")
    shutil.copytree(model_folders[name], folder)
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    c["eos_token_id"] = [unused, free[stop_at]]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(c, f)
    m = load(folder, "float32", nr_ctx=128, max_tokens=256)
    assert m.end_token == unused and m.end_tokens == [unused, free[stop_at]]
    m.init(0, 1.0, 0.0, 1.0, 0, 0, m.end_token)
    res = m.generate([prompt], max_new_tokens=10)
    assert res.tokens == [free[:stop_at + 1]] and res.finish == ["stop"]
    r = subprocess.run([os.path.join(ROOT, "bin", "llama"), "-m", folder, "-d", "float32", "-c", "128",
                        "-n", "10", "--temp", "0", "--top_k", "0", "--top_p", "1", "--repeat_penalty", "1", "-s", "1",
                        "--prompt-ids", ",".join(map(str, prompt))], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("[0]")][0]
    assert line == "[0] stop: " + ",".join(map(str, free[:stop_at + 1]))
