"""bin/trace_run replays the same requests whole, with the last 32 tokens decoded one by one,
and in batches of unequal lengths, in float32 and in bfloat16; all are compared with the plain
implementation (GPU).  The program is run as a user runs it: a child process, steps on standard
input, logits in files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
from conftest import ROOT, TINY, random_prompt
from util import assert_close

pytestmark = pytest.mark.gpu
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(folder, dtype, steps, out_dir, max_tokens):
    """Feed the steps one at a time, waiting for `done <step>` after each."""
    proc = subprocess.Popen([TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
                             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                            text=True)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    vocab = json.load(open(os.path.join(folder, "config.json")))["vocab_size"]
    out = {}
    for st in steps:
        p = os.path.join(out_dir, f"{st['step']}.f32")
        n_want = sum(len(e.get("want", [])) for e in st["entries"])
        assert os.path.exists(p) == (n_want > 0)
        if n_want:
            out[st["step"]] = np.fromfile(p, dtype="<f4").reshape(n_want, vocab)
    return out


def collect(steps, logits):
    """(request id) -> {position: logits row}, from the steps and the files they produced."""
    pos, got = {}, {}
    for st in steps:
        row = 0
        for e in st["entries"]:
            start = pos.get(e["id"], 0)
            for w in e.get("want", []):
                got.setdefault(e["id"], {})[start + w] = logits[st["step"]][row]
                row += 1
            pos[e["id"]] = start + len(e["tokens"])
    return got


def check(name, dtype, reqs, got, plain_logits):
    for rid, ids in reqs.items():
        ref = plain_logits(name, ids)
        have = got[rid]
        assert sorted(have) == list(range(len(ids))), f"request {rid}: positions missing"
        assert_close(np.stack([have[p] for p in range(len(ids))]), ref, dtype, f"{name} {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_three_ways(name, dtype, model_folders, plain_logits, tmp_path):
    maxpos = TINY[name]["max_position_embeddings"]
    lens = {"a": maxpos, "b": 70, "c": 33, "d": 100, "e": 65}
    reqs = {rid: random_prompt(name, n, 500 + i) for i, (rid, n) in enumerate(lens.items())}
    folder = model_folders[name]

    # 1. each request alone and whole
    steps = [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
             for i, (rid, ids) in enumerate(reqs.items())]
    whole = collect(steps, replay(folder, dtype, steps, str(tmp_path / "whole"), 64 * -(-maxpos // 64)))
    check(name, dtype, reqs, whole, plain_logits)

    # 2. the last 32 tokens one by one
    steps, k = [], 0
    for rid, ids in reqs.items():
        n = len(ids) - 32
        steps.append({"step": k, "entries": [{"id": rid, "tokens": ids[:n], "want": list(range(n))}], "end": []})
        k += 1
        for j in range(n, len(ids)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [ids[j]], "want": [0]}],
                          "end": [rid] if j == len(ids) - 1 else []})
            k += 1
    tail = collect(steps, replay(folder, dtype, steps, str(tmp_path / "tail"), 64 * -(-maxpos // 64)))
    check(name, dtype, reqs, tail, plain_logits)

    # 3. batches of unequal lengths, shorter requests ending earlier, one batch after another in a
    #    cache that holds only one batch: slots and pages are used again
    batches, pre = [["a", "b", "c"], ["d", "e"]], {"a": maxpos - 40, "b": 64, "c": 1, "d": 65, "e": 3}
    need = max(sum(-(-lens[r] // 64) * 64 for r in b) for b in batches)
    steps, k = [], 0
    for batch in batches:
        pos = {r: pre[r] for r in batch}
        steps.append({"step": k, "entries": [{"id": r, "tokens": reqs[r][:pre[r]], "want": list(range(pre[r]))}
                                             for r in batch], "end": []})
        k += 1
        live = list(batch)
        while live:
            ending = [r for r in live if pos[r] + 1 == lens[r]]
            steps.append({"step": k, "entries": [{"id": r, "tokens": [reqs[r][pos[r]]], "want": [0]} for r in live],
                          "end": ending})
            k += 1
            for r in live:
                pos[r] += 1
            live = [r for r in live if pos[r] < lens[r]]
    batched = collect(steps, replay(folder, dtype, steps, str(tmp_path / "batched"), need))
    check(name, dtype, reqs, batched, plain_logits)

    # the three cuttings agree with each other: in float32 bit for bit
    for rid, ids in reqs.items():
        for p in range(len(ids)):
            if dtype == "float32":
                assert np.array_equal(whole[rid][p], tail[rid][p]) and np.array_equal(whole[rid][p], batched[rid][p])
            else:
                assert_close(tail[rid][p], whole[rid][p], dtype)
                assert_close(batched[rid][p], whole[rid][p], dtype)


def test_steps_without_wanted_logits_write_no_file(model_folders, tmp_path):
    steps = [{"step": 7, "entries": [{"id": "x", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 9, "entries": [{"id": "x", "tokens": [4], "want": [0]}], "end": ["x"]}]
    out = replay(model_folders["A"], "float32", steps, str(tmp_path), 64)
    assert list(out) == [9] and out[9].shape == (1, 256)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wanted_places_in_any_order_many_requests_and_two_batches_alive(dtype, model_folders, plain_logits, tmp_path):
    """What a trace may also hold: wanted places out of order and named twice (the rows follow `want`),
    an entry without `want` and a line without `end`, a hundred requests alive at once (the cache has a
    slot per page), and a second batch that starts while the first is still decoding."""
    name = "A"
    n_req = 100
    lens = [3 + (7 * i) % 29 for i in range(n_req)]
    reqs = {f"r{i}": random_prompt(name, lens[i] + 2, 900 + i) for i in range(n_req)}
    first, second = [f"r{i}" for i in range(60)], [f"r{i}" for i in range(60, n_req)]

    def prompt_entry(rid, i):
        n = len(reqs[rid]) - 2
        want = [n - 1, 0, n - 1] if i % 3 == 0 else ([n - 1] if i % 3 == 1 else None)
        e = {"id": rid, "tokens": reqs[rid][:n]}
        if want is not None:
            e["want"] = want
        return e

    steps = [{"step": 0, "entries": [prompt_entry(r, i) for i, r in enumerate(first)]},              # no "end"
             {"step": 1, "entries": [{"id": r, "tokens": [reqs[r][-2]], "want": [0]} for r in first], "end": []},
             {"step": 2, "entries": [prompt_entry(r, i) for i, r in enumerate(second)], "end": []},  # the first batch still lives
             {"step": 3, "entries": [{"id": r, "tokens": [reqs[r][-1]], "want": [0]} for r in first], "end": first},
             {"step": 4, "entries": [{"id": r, "tokens": [reqs[r][-2]], "want": [0]} for r in second], "end": second[:5]},
             {"step": 5, "entries": [{"id": r, "tokens": [reqs[r][-1]], "want": [0]} for r in second[5:]], "end": second[5:]}]
    out = replay(model_folders[name], dtype, steps, str(tmp_path), 64 * n_req)
    for st in steps:
        row = 0
        for e in st["entries"]:
            rid = e["id"]
            ref = plain_logits(name, reqs[rid])
            start = {0: 0, 2: 0, 1: len(reqs[rid]) - 2, 4: len(reqs[rid]) - 2, 3: len(reqs[rid]) - 1, 5: len(reqs[rid]) - 1}[st["step"]]
            for w in e.get("want", []):
                assert_close(out[st["step"]][row][None], ref[start + w][None], dtype, f"step {st['step']} {rid} place {w}")
                row += 1
        assert row == out[st["step"]].shape[0]
