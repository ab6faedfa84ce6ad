"""The engine against the plain implementation, in every way of cutting the work (GPU).

For each tiny model, in float32 and in bfloat16: each request alone and whole; the last 32
tokens one by one; batches of unequal lengths whose shorter requests end earlier, one batch
after another on a cache so small that slots and pages are used again; long decoding; the
first tokens of a sequence.  In float32 the engine's own results must also be bit-identical
across the cuttings: its kernels fix the order of every sum per row.
"""
import numpy as np
import pytest
import torch
from conftest import TINY, random_prompt
from util import assert_close, make_engine

from inferllm_b200 import EngineError, StepItem
from inferllm_b200.cache import CacheError, CacheFull

pytestmark = pytest.mark.gpu

MODELS = ["A", "B", "C", "D"]
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [128, 97, 40], "B": [256, 131, 33], "C": [300, 77, 513], "D": [200, 65, 130]}


def whole(eng, ids):
    s = eng.new_sequence()
    lg = eng.step([StepItem(s, ids, list(range(len(ids))))])
    eng.end_sequence(s)
    return lg.cpu().numpy()


def tail_one_by_one(eng, ids, tail=32):
    s = eng.new_sequence()
    n = len(ids) - tail
    out = [eng.step([StepItem(s, ids[:n], list(range(n)))])]
    for t in ids[n:]:
        out.append(eng.step([StepItem(s, [t], [0])]))
    eng.end_sequence(s)
    return torch.cat(out).cpu().numpy()


def in_batches(eng, requests, prefill_lens, batches):
    """Teacher-forced replay: each batch starts together (prompts of unequal lengths in one
    step), then one token per live request and step; a request leaves when its tokens are used
    up.  Returns per request the logits at all its positions."""
    got = {}
    for batch in batches:
        slots = {r: eng.new_sequence() for r in batch}
        lg = eng.step([StepItem(slots[r], requests[r][:prefill_lens[r]], list(range(prefill_lens[r])))
                       for r in batch]).cpu().numpy()
        off = 0
        for r in batch:
            got[r] = [lg[off:off + prefill_lens[r]]]
            off += prefill_lens[r]
        pos = {r: prefill_lens[r] for r in batch}
        live = [r for r in batch if pos[r] < len(requests[r])]
        for r in batch:
            if r not in live:
                eng.end_sequence(slots[r])
        while live:
            lg = eng.step([StepItem(slots[r], [requests[r][pos[r]]], [0]) for r in live]).cpu().numpy()
            nxt = []
            for i, r in enumerate(live):
                got[r].append(lg[i:i + 1])
                pos[r] += 1
                if pos[r] < len(requests[r]):
                    nxt.append(r)
                else:
                    eng.end_sequence(slots[r])
            live = nxt
    return {r: np.concatenate(v) for r, v in got.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_whole_and_tail_one_by_one(name, dtype, model_folders, plain_logits):
    eng = make_engine(model_folders[name], dtype, max_tokens=1024)
    for i, n in enumerate(LENGTHS[name]):
        ids = random_prompt(name, n, 100 + i)
        ref = plain_logits(name, ids)
        w = whole(eng, ids)
        assert_close(w, ref, dtype, f"{name} whole n={n}")
        if n > 40:
            t = tail_one_by_one(eng, ids)
            assert_close(t, ref, dtype, f"{name} last 32 one by one n={n}")
            if dtype == "float32":
                assert np.array_equal(w, t), "float32: whole and one-by-one logits differ in bits"
            else:
                assert_close(t, w, dtype, "whole vs one by one")
    eng.check_device_errors()
    eng.cache.check()
    assert eng.cache.slots_free == eng.cache.num_slots


@pytest.mark.parametrize("page_size", [8, 16])
@pytest.mark.parametrize("name", ["C", "D"])
def test_small_pages_take_the_other_attention_kernels(name, page_size, model_folders, plain_logits):
    """With pages of fewer than 64 positions the bfloat16 engine cannot use the TMA-fed attention
    kernels and runs the warp-level ones instead: the same logits in every cutting."""
    from inferllm_b200.kernels import ops
    cfg = TINY[name]
    assert not ops.attention_decode_ring_supported(torch.bfloat16, cfg["num_attention_heads"],
                                                   cfg.get("num_key_value_heads", cfg["num_attention_heads"]),
                                                   cfg["head_dim"], page_size)
    eng = make_engine(model_folders[name], "bfloat16", max_tokens=1024, page_size=page_size)
    ids = random_prompt(name, LENGTHS[name][0], 300)
    ref = plain_logits(name, ids)
    w = whole(eng, ids)
    assert_close(w, ref, "bfloat16", f"{name} whole, pages of {page_size}")
    t = tail_one_by_one(eng, ids)
    assert_close(t, ref, "bfloat16", f"{name} last 32 one by one, pages of {page_size}")
    reqs = [random_prompt(name, n, 310 + i) for i, n in enumerate([90, 33, 70])]
    got = in_batches(eng, reqs, [60, 1, 33], [[0, 1, 2]])
    for r, q in enumerate(reqs):
        assert_close(got[r], plain_logits(name, q), "bfloat16", f"{name} request {r}, pages of {page_size}")
    eng.check_device_errors()
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_unequal_batches_with_slot_reuse(name, dtype, model_folders, plain_logits):
    maxpos = TINY[name]["max_position_embeddings"]
    total = [maxpos, 70, 33, 129 if maxpos > 129 else 90, 64, 1, 65, 100]
    prefill = [maxpos - 20, 65, 1, 64, 63, 1, 33, 90]
    reqs = [random_prompt(name, n, 200 + i) for i, n in enumerate(total)]
    # three slots and few pages: the second and third batch must reuse what the first gave back
    need = max(sum(-(-total[r] // 64) for r in b) for b in ([0, 1, 2], [3, 4, 5], [6, 7]))
    eng = make_engine(model_folders[name], dtype, max_tokens=64 * need, max_batch=3)
    got = in_batches(eng, reqs, prefill, [[0, 1, 2], [3, 4, 5], [6, 7]])
    for r, ids in enumerate(reqs):
        assert_close(got[r], plain_logits(name, ids), dtype, f"{name} request {r} in batches")
    if dtype == "float32":
        for r in (0, 3, 7):
            assert np.array_equal(got[r], whole(eng, reqs[r])), \
                f"float32: request {r} differs between a batch and alone"
    eng.check_device_errors()
    eng.cache.check()
    assert eng.cache.pages_free() == [need]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "D"])
def test_slot_reuse_with_poisoned_pages(name, dtype, model_folders, plain_logits):
    """The same batches on an engine that fills every page that goes back to the pool (and every
    page nobody has held yet) with NaN: a kernel that reads a page its sequence does not hold, or
    a place of its last page behind its length, gives NaN instead of a plausible number."""
    maxpos = TINY[name]["max_position_embeddings"]
    total = [maxpos, 70, 33, 129, 64, 1, 65, 100]
    prefill = [maxpos - 20, 65, 1, 64, 63, 1, 33, 90]
    reqs = [random_prompt(name, n, 500 + i) for i, n in enumerate(total)]
    need = max(sum(-(-total[r] // 64) for r in b) for b in ([0, 1, 2], [3, 4, 5], [6, 7]))
    eng = make_engine(model_folders[name], dtype, max_tokens=64 * need, max_batch=3, poison=True)
    got = in_batches(eng, reqs, prefill, [[0, 1, 2], [3, 4, 5], [6, 7]])
    for r, ids in enumerate(reqs):
        assert_close(got[r], plain_logits(name, ids), dtype, f"{name} request {r} in batches, poisoned pages")
    eng.check_device_errors()
    eng.cache.check()
    free = [p for p in range(need)]
    k, v = eng.cache_tensors(0)
    assert bool(torch.isnan(k[:, free].float()).all()) and bool(torch.isnan(v[:, free].float()).all()), "all pages are free again and must be poisoned"


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_weights_are_the_same_from_a_folder_and_on_the_device(dtype, tmp_path):
    """One seed gives one model: written to a folder by `write_random_model` (host generator) and read
    back, or filled on the device by `Engine.from_config` (fill kernel), the tensors are the same
    bits and so are the logits."""
    from inferllm_b200 import Engine, EngineOptions, config_from_dict, write_random_model
    cfg = config_from_dict(TINY["A"])
    folder = str(tmp_path)
    write_random_model(cfg, folder, 1234, torch.float32 if dtype == "float32" else torch.bfloat16)
    a = Engine.from_folder(folder, EngineOptions(dtype=dtype, max_tokens=256))
    b = Engine.from_config(cfg, EngineOptions(dtype=dtype, max_tokens=256), 1234)
    ids = random_prompt("A", 50, 3)
    assert np.array_equal(whole(a, ids), whole(b, ids))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(dtype, model_folders, plain_logits):
    """A one-token prompt decoded for hundreds of steps across page borders, next to a second
    sequence that starts at the same time and ends early."""
    name = "D"
    ids = random_prompt(name, 400, 7)
    other = random_prompt(name, 9, 8)
    eng = make_engine(model_folders[name], dtype, max_tokens=64 * 8, max_batch=2)
    got = in_batches(eng, [ids, other], [1, 2], [[0, 1]])
    ref = plain_logits(name, ids)
    assert_close(got[0][:8], ref[:8], dtype, "first tokens")
    assert_close(got[0], ref, dtype, "long decoding")
    assert_close(got[1], plain_logits(name, other), dtype, "short neighbour")
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_wanted_places_and_padding_free_batches(dtype, model_folders, plain_logits):
    name = "B"
    a, b, c = (random_prompt(name, n, 300 + n) for n in (50, 3, 17))
    eng = make_engine(model_folders[name], dtype, max_tokens=512)
    sa, sb, sc = (eng.new_sequence() for _ in range(3))
    lg = eng.step([StepItem(sa, a, [49, 0]), StepItem(sb, b, []), StepItem(sc, c, [16])]).cpu().numpy()
    assert lg.shape == (3, TINY[name]["vocab_size"])
    assert_close(lg[0], plain_logits(name, a)[49], dtype)
    assert_close(lg[1], plain_logits(name, a)[0], dtype)
    assert_close(lg[2], plain_logits(name, c)[16], dtype)
    none = eng.step([StepItem(sb, [7], [])])
    assert tuple(none.shape) == (0, TINY[name]["vocab_size"])
    # the request that asked for nothing still advanced: its next logits see all four tokens
    lg = eng.step([StepItem(sb, [9], [0])]).cpu().numpy()
    assert_close(lg[0], plain_logits(name, b + [7, 9])[-1], dtype)
    for s in (sa, sb, sc):
        eng.end_sequence(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_single_prompts_padded_and_replayed_from_graphs(dtype, model_folders, plain_logits):
    """A single prompt is padded to whole buckets of 64 tokens behind its real ones and, from the
    second time a bucket is seen, captured and replayed.  Three rounds (issued, captured, replayed)
    of: a prompt of 100 tokens, a second piece of 100 tokens behind 128 (padded to 128: its padding
    leaves keys behind the sequence's length, in pages the sequence holds anyway), then single
    tokens that overwrite them.  Every logit matches the plain implementation, and in float32 the
    three rounds agree bit for bit."""
    name = "C"
    ids = random_prompt(name, 300, 9)
    ref = plain_logits(name, ids)
    eng = make_engine(model_folders[name], dtype, max_tokens=1024, max_batch=2)
    rounds = []
    for _ in range(3):
        s = eng.new_sequence()
        out = [eng.step([StepItem(s, ids[:100], list(range(100)))]),
               eng.step([StepItem(s, ids[100:128], list(range(28)))]),
               eng.step([StepItem(s, ids[128:228], list(range(100)))])]
        assert eng.sequence_length(s) == 228
        for t in ids[228:]:
            out.append(eng.step([StepItem(s, [t], [0])]))
        eng.end_sequence(s)
        rounds.append(torch.cat(out).cpu().numpy())
        assert_close(rounds[-1], ref, dtype, f"round {len(rounds)}")
    if dtype == "float32":
        assert np.array_equal(rounds[0], rounds[1]) and np.array_equal(rounds[0], rounds[2])
    assert eng.info()["graphs_captured"] >= 2, "the buckets of 128 tokens (100 and 28 wanted rows) should be captured"
    eng.check_device_errors()
    eng.cache.check()
    assert eng.cache.slots_free == eng.cache.num_slots


def test_result_does_not_depend_on_the_slot_or_on_old_cache_contents(model_folders):
    """float32, bit for bit: a request gives the same logits in a fresh cache, in another slot,
    and in pages that other requests have filled before."""
    name = "A"
    ids = random_prompt(name, 100, 1)
    eng = make_engine(model_folders[name], "float32", max_tokens=64 * 6, max_batch=3)
    first = tail_one_by_one(eng, ids)
    junk = [eng.new_sequence() for _ in range(2)]
    eng.step([StepItem(junk[0], random_prompt(name, 128, 2), []),
              StepItem(junk[1], random_prompt(name, 90, 3), [])])
    eng.end_sequence(junk[0])          # slot 0 and its pages go back, slot 1 stays live
    s = eng.new_sequence()
    lg = [eng.step([StepItem(s, ids[:68], list(range(68)))])]
    for t in ids[68:]:
        lg.append(eng.step([StepItem(s, [t], [0]), StepItem(junk[1], [5], [])])[:1])
    again = torch.cat(lg).cpu().numpy()
    assert np.array_equal(first, again)
    eng.check_device_errors()


@pytest.mark.parametrize("name", ["C", "D"])
def test_bfloat16_steps_give_the_same_bits_every_time(name, model_folders):
    """No sum of the bfloat16 kernels depends on timing (split products and split attention are added
    up in a fixed order, nothing is accumulated with atomics): the same batch, replayed in the same
    engine and in a second engine, gives the same logits bit for bit, through prompts of unequal
    lengths, eager first steps, captured graphs and their replays."""
    lens = [LENGTHS[name][0], 70, 33]
    reqs = [random_prompt(name, n, 40 + i) for i, n in enumerate(lens)]
    pre = [lens[0] - 20, 40, 5]
    runs = []
    for _ in range(2):
        eng = make_engine(model_folders[name], "bfloat16", max_tokens=64 * 16, max_batch=3)
        for _ in range(2):
            runs.append(in_batches(eng, reqs, pre, [[0, 1, 2]]))
        eng.check_device_errors()
        del eng
    for other in runs[1:]:
        for r in range(3):
            assert np.array_equal(runs[0][r], other[r]), f"request {r} differs between two runs of the same batch"


def test_refusals(model_folders):
    eng = make_engine(model_folders["A"], "float32", max_tokens=128, max_batch=2)
    s = eng.new_sequence()
    with pytest.raises(EngineError, match="vocabulary"):
        eng.step([StepItem(s, [256], [])])
    with pytest.raises(EngineError, match="wanted place"):
        eng.step([StepItem(s, [1, 2], [2])])
    with pytest.raises(EngineError, match="at least one token"):
        eng.step([StepItem(s, [], [])])
    with pytest.raises(CacheError, match="maximum sequence length"):
        eng.step([StepItem(s, [1] * 129, [])])
    t = eng.new_sequence()
    eng.step([StepItem(s, [1] * 100, [])])
    with pytest.raises(CacheFull):
        eng.step([StepItem(t, [1] * 10, [])])     # two pages are taken, the cache has two
    assert eng.sequence_length(t) == 0
    with pytest.raises(CacheFull):
        eng.new_sequence()
    eng.end_sequence(s)
    eng.step([StepItem(t, [1] * 10, [9])])
    eng.check_device_errors()


@pytest.mark.parametrize("name", ["C", "D"])
def test_all_products_on_the_package_kernels(name, model_folders, plain_logits):
    """gemm="tc": prompts and single tokens both go through the tcgen05 kernels (no library
    product anywhere in the step) and still match the plain implementation."""
    from inferllm_b200 import Engine, EngineOptions
    eng = Engine.from_folder(model_folders[name], EngineOptions(dtype="bfloat16", max_tokens=1024, gemm="tc"))
    assert eng.info()["gemm"] == "tc"
    for i, n in enumerate(LENGTHS[name]):
        ids = random_prompt(name, n, 100 + i)
        assert_close(whole(eng, ids), plain_logits(name, ids), "bfloat16", f"{name} whole n={n}")
        if n > 40:
            assert_close(tail_one_by_one(eng, ids), plain_logits(name, ids), "bfloat16", f"{name} tail n={n}")
    eng.check_device_errors()
    # the choice belongs to the engine: another engine beside it keeps its own
    other = Engine.from_folder(model_folders[name], EngineOptions(dtype="bfloat16", max_tokens=256))
    assert other.info()["gemm"] == "auto" and eng.info()["gemm"] == "tc"


def _drawn_configurations():
    """Seeded configurations off the beaten sizes: head sizes in steps of 16 up to 256 (those of the
    tensor-core kernels and others), 1..5 KV heads with 1..7 query heads each, widths that are no
    multiple of 8, odd intermediate sizes and vocabularies."""
    rng = np.random.default_rng(20240229)
    out = []
    for d in (16, 32, 48, 64, 80, 96, 128, 160, 256):
        nkv = int(rng.integers(1, 6))
        group = int(rng.choice([1, 2, 3, 4, 7]))
        out.append(dict(
            architectures=["LlamaForCausalLM"], hidden_size=int(rng.choice([36, 72, 100, 136, 200, 264, 90, 54])),
            num_hidden_layers=int(rng.integers(1, 4)), num_attention_heads=nkv * group, num_key_value_heads=nkv,
            head_dim=d, intermediate_size=int(rng.integers(40, 400)), vocab_size=int(rng.integers(50, 1500)),
            rope_theta=float(rng.choice([1e4, 5e5, 1e6, 777.0])), rms_norm_eps=float(rng.choice([1e-5, 1e-6, 2e-4])),
            max_position_embeddings=int(rng.choice([160, 192, 333])), tie_word_embeddings=bool(rng.integers(0, 2)),
            eos_token_id=2))
    return out


@pytest.mark.parametrize("index", range(9))
def test_drawn_configurations(index, tmp_path):
    """The engine takes every size a configuration may have: whole, with its last tokens one by one
    and in a batch of two, in both precisions against the plain implementation."""
    import plain_llama

    from inferllm_b200 import config_from_dict, write_random_model
    cfg = _drawn_configurations()[index]
    folder = str(tmp_path)
    write_random_model(config_from_dict(cfg), folder, 900 + index, torch.bfloat16)
    pcfg, pw = plain_llama.load_weights(folder)
    rng = np.random.default_rng(index)
    maxpos = cfg["max_position_embeddings"]
    reqs = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (maxpos, 67, 5)]
    refs = [plain_llama.forward(pcfg, pw, ids) for ids in reqs]
    what = f"configuration {index}: " + ", ".join(f"{k}={cfg[k]}" for k in (
        "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size"))
    for dtype in DTYPES:
        eng = make_engine(folder, dtype, max_tokens=64 * 12, max_batch=3)
        w = whole(eng, reqs[0])
        assert_close(w, refs[0], dtype, what + " whole")
        t = tail_one_by_one(eng, reqs[0], tail=9)
        assert_close(t, refs[0], dtype, what + " last 9 one by one")
        got = in_batches(eng, reqs, [maxpos - 30, 60, 5], [[0, 1, 2]])
        for r in range(3):
            assert_close(got[r], refs[r], dtype, what + f" request {r} of a batch")
        if dtype == "float32":
            assert np.array_equal(w, t) and np.array_equal(w, got[0]), what + ": float32 logits differ between cuttings"
        eng.check_device_errors()
        eng.cache.check()
        del eng


@pytest.mark.parametrize("seed", range(10))
def test_drawn_configurations_pages_and_batches(seed, tmp_path):
    """Ten more draws in which everything varies together: the sizes as above, the page size (16 to 128),
    the number of requests (3 to 7, or 17 to 40 so that single-token steps take the library's products),
    their lengths, how much of each is its prompt, how the requests are cut into batches that follow one
    another in the same slots, the length of the tail decoded one by one, and whether freed pages are
    poisoned; both precisions against the plain implementation, float32 bit for bit between cuttings."""
    import plain_llama

    from inferllm_b200 import config_from_dict, write_random_model
    rng = np.random.default_rng(77000 + seed)
    d = int(rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 144, 192, 256]))
    nkv, group = int(rng.integers(1, 6)), int(rng.choice([1, 1, 2, 3, 4, 5, 8]))
    maxpos = int(rng.choice([96, 160, 257, 400]))
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=int(rng.choice([24, 36, 72, 100, 136, 200, 264, 90, 54, 256, 512])),
               num_hidden_layers=int(rng.integers(1, 4)), num_attention_heads=nkv * group, num_key_value_heads=nkv, head_dim=d,
               intermediate_size=int(rng.integers(17, 600)), vocab_size=int(rng.integers(33, 3000)),
               rope_theta=float(rng.choice([1e4, 5e5, 1e6, 777.0, 123456.7])),
               rms_norm_eps=float(rng.choice([1e-5, 1e-6, 2e-4, 1e-3])), max_position_embeddings=maxpos,
               tie_word_embeddings=bool(rng.integers(0, 2)), eos_token_id=2)
    page = int(rng.choice([16, 32, 64, 64, 128]))
    what = f"draw {seed}, pages of {page}: " + ", ".join(f"{k}={cfg[k]}" for k in (
        "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size",
        "vocab_size", "max_position_embeddings", "tie_word_embeddings"))
    folder = str(tmp_path)
    write_random_model(config_from_dict(cfg), folder, 7000 + seed, torch.bfloat16)
    pcfg, pw = plain_llama.load_weights(folder)
    n_req = int(rng.integers(3, 8)) if seed % 3 else int(rng.integers(17, 41))
    lens = [int(rng.integers(1, (maxpos if n_req < 10 else min(maxpos, 120)) + 1)) for _ in range(n_req)]
    lens[0] = maxpos
    reqs = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lens]
    refs = [plain_llama.forward(pcfg, pw, ids) for ids in reqs]
    pre = [int(rng.integers(1, n + 1)) for n in lens]
    pre[0] = max(1, maxpos - int(rng.integers(1, 40)))
    order = list(range(n_req))
    rng.shuffle(order)
    cut = sorted(set([0, n_req] + [int(x) for x in rng.integers(1, n_req, size=2)]))
    batches = [order[a:b] for a, b in zip(cut[:-1], cut[1:])]
    for dtype in DTYPES:
        eng = make_engine(folder, dtype, max_tokens=sum(-(-n // page) * page for n in lens) + 2 * page, page_size=page,
                          max_batch=max(len(b) for b in batches), poison=bool(rng.integers(0, 2)))
        w = whole(eng, reqs[0])
        assert_close(w, refs[0], dtype, what + " whole")
        tail = int(rng.integers(1, min(33, maxpos)))
        t = tail_one_by_one(eng, reqs[0], tail=tail)
        assert_close(t, refs[0], dtype, what + f" last {tail} one by one")
        got = in_batches(eng, reqs, pre, batches)
        for r in range(n_req):
            assert_close(got[r], refs[r], dtype, what + f" request {r} ({lens[r]} tokens, prompt of {pre[r]}) in {batches}")
        if dtype == "float32":
            assert np.array_equal(w, t) and np.array_equal(w, got[0]), what + ": float32 logits differ between cuttings"
        eng.check_device_errors()
        eng.cache.check()
        del eng


def test_layers_of_real_width_bfloat16_against_float32():
    """Two layers with the widths of an 8B model (4096 wide, 32 heads over 8 KV heads of 128, a
    14336-wide feed-forward, 128256 words): the bfloat16 engine with its tensor-core kernels at the
    sizes they were written for, against the true float32 engine on the same random weights, whole,
    token by token and in an unequal batch."""
    from inferllm_b200 import Engine, EngineOptions, config_from_dict
    cfg = config_from_dict(dict(architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=2,
                                num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                                intermediate_size=14336, vocab_size=128256, rope_theta=500000.0,
                                rms_norm_eps=1e-5, max_position_embeddings=1024))
    g = torch.Generator().manual_seed(17)
    reqs = [torch.randint(0, 128256, (n,), generator=g).tolist() for n in (200, 70, 129)]
    got = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_config(cfg, EngineOptions(dtype=dtype, max_tokens=1024, max_batch=3), 3)
        w = whole(eng, reqs[0])
        t = tail_one_by_one(eng, reqs[0])
        b = in_batches(eng, reqs, [150, 70, 1], [[0, 1, 2]])
        got[dtype] = (w, t, b)
        eng.check_device_errors()
        eng.cache.check()
        del eng
        torch.cuda.empty_cache()
    w32, t32, b32 = got["float32"]
    w16, t16, b16 = got["bfloat16"]
    assert np.array_equal(w32, t32) and np.array_equal(w32, b32[0])
    assert_close(w16, w32, "bfloat16", "whole, real widths")
    assert_close(t16, w32, "bfloat16", "last 32 one by one, real widths")
    for r in range(3):
        assert_close(b16[r], b32[r], "bfloat16", f"request {r} in a batch, real widths")


def test_long_context(tmp_path):
    """A prompt of 4,200 tokens in one step (33 tiles of the prompt attention kernel per head), then
    40 tokens one by one over 66 and 67 key tiles per head, which a single sequence reads in as many
    splits as the decode attention kernel has, against the plain implementation (the kernels' own
    tests make single far keys stand out; here the whole path runs at that length)."""
    import plain_llama

    from inferllm_b200 import config_from_dict, write_random_model
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=128, num_hidden_layers=1, num_attention_heads=2,
               num_key_value_heads=1, head_dim=64, intermediate_size=256, vocab_size=300, rope_theta=10000.0,
               rms_norm_eps=1e-5, max_position_embeddings=4352, tie_word_embeddings=False, eos_token_id=2)
    folder = str(tmp_path)
    write_random_model(config_from_dict(cfg), folder, 77, torch.bfloat16)
    pcfg, pw = plain_llama.load_weights(folder)
    rng = np.random.default_rng(5)
    ids = rng.integers(3, 300, 4240).tolist()
    ref = plain_llama.forward(pcfg, pw, ids)[4199:]
    for dtype in DTYPES:
        eng = make_engine(folder, dtype, max_tokens=4352, max_batch=1)
        s = eng.new_sequence()
        out = [eng.step([StepItem(s, ids[:4200], [4199])])]
        for t in ids[4200:]:
            out.append(eng.step([StepItem(s, [t], [0])]))
        eng.end_sequence(s)
        got = torch.cat(out).cpu().numpy()
        assert_close(got[:1], ref[:1], dtype, "end of a 4,200-token prompt")
        assert_close(got[1:], ref[1:], dtype, "40 tokens one by one behind it")
        eng.check_device_errors()
        del eng


def test_random_batches_against_float32():
    """Forty batches of random size (1..12), random prompt lengths (2..3000), random numbers of
    single-token steps and sequences that end at different times, on a mid-sized model with grouped
    heads: one request of every batch is replayed alone on the float32 engine and must agree; the
    kernels' error words stay clear and the cache keeps its invariants."""
    from inferllm_b200 import Engine, EngineOptions, config_from_dict
    cfg = config_from_dict(dict(architectures=["LlamaForCausalLM"], hidden_size=1024, num_hidden_layers=3,
                                num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=2816,
                                vocab_size=5000, max_position_embeddings=4096))
    eng = Engine.from_config(cfg, EngineOptions(dtype="bfloat16", max_tokens=40000, max_batch=12), 5)
    ref = Engine.from_config(cfg, EngineOptions(dtype="float32", max_tokens=8192, max_batch=2), 5)
    rng = np.random.default_rng(1)
    for _ in range(40):
        B = int(rng.integers(1, 13))
        lens = [int(rng.integers(2, 3000)) for _ in range(B)]
        n_dec = int(rng.integers(1, 40))
        pre = [max(1, n - int(rng.integers(0, n_dec + 1))) for n in lens]
        reqs = [rng.integers(0, 5000, size=n).tolist() for n in lens]
        i = int(rng.integers(0, B))
        got = in_batches(eng, reqs, pre, [list(range(B))])[i]
        want = in_batches(ref, [reqs[i]], [pre[i]], [[0]])[0]
        assert_close(got[pre[i] - 1:], want[pre[i] - 1:], "bfloat16", f"request {i} of a batch of {B} (lengths {lens})")
        eng.check_device_errors()
        eng.cache.check()


@pytest.mark.parametrize("B", [17, 33, 64, 80])
def test_decode_steps_of_many_sequences(B, tmp_path):
    """One-token steps of 17, 33, 64 and 80 sequences: from 17 tokens on a decode step takes the
    library's products (finished tensors instead of K slices into the norms and into the fused
    attention kernel), and each batch size captures a graph of its own.  Every sequence has another
    length; all of them are checked against the float32 engine at every decoded position, and two
    of them (the shortest and the longest) against the plain implementation."""
    import plain_llama

    from inferllm_b200 import config_from_dict, write_random_model
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=64, intermediate_size=704, vocab_size=640, rope_theta=10000.0,
               rms_norm_eps=1e-5, max_position_embeddings=512, tie_word_embeddings=False, eos_token_id=2)
    folder = str(tmp_path)
    write_random_model(config_from_dict(cfg), folder, 5, torch.bfloat16)
    rng = np.random.default_rng(B)
    lens = [int(rng.integers(3, 200)) for _ in range(B)]
    lens[0], lens[1] = 3, 260
    n_dec = 6
    reqs = [rng.integers(0, 640, size=n + n_dec).tolist() for n in lens]
    eng = make_engine(folder, "bfloat16", max_tokens=B * 320 + 64, max_batch=B)
    ref = make_engine(folder, "float32", max_tokens=B * 320 + 64, max_batch=B)
    got = in_batches(eng, reqs, lens, [list(range(B))])
    want = in_batches(ref, reqs, lens, [list(range(B))])
    for r in range(B):
        assert_close(got[r][lens[r] - 1:], want[r][lens[r] - 1:], "bfloat16", f"request {r} of {B}")
    pcfg, pw = plain_llama.load_weights(folder)
    for r in (0, 1):
        plain = plain_llama.forward(pcfg, pw, reqs[r])
        assert_close(want[r], plain, "float32", f"request {r} of {B}, float32")
        assert_close(got[r], plain, "bfloat16", f"request {r} of {B}, bfloat16")
    eng.check_device_errors()
    eng.cache.check()


def test_batch_that_shrinks_across_the_kernel_switch(tmp_path):
    """Twenty sequences of which eight end early, one per step, so that the live count falls from 20
    to 12 while decoding: the step changes from the library's products to the package's split
    product at 16 tokens, and every count replays or captures another graph.  All positions against
    the float32 engine, the last request to end against the plain implementation."""
    import plain_llama

    from inferllm_b200 import config_from_dict, write_random_model
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=4, head_dim=64, intermediate_size=704, vocab_size=640, rope_theta=10000.0,
               rms_norm_eps=1e-5, max_position_embeddings=512, tie_word_embeddings=True, eos_token_id=2)
    folder = str(tmp_path)
    write_random_model(config_from_dict(cfg), folder, 6, torch.bfloat16)
    rng = np.random.default_rng(3)
    B = 20
    lens = [int(rng.integers(5, 150)) for _ in range(B)]
    extra = [2 + i for i in range(8)] + [14] * (B - 8)   # requests 0..7 end after 2..9 single-token steps
    reqs = [rng.integers(0, 640, size=n + e).tolist() for n, e in zip(lens, extra)]
    eng = make_engine(folder, "bfloat16", max_tokens=B * 192 + 64, max_batch=B)
    ref = make_engine(folder, "float32", max_tokens=B * 192 + 64, max_batch=B)
    for _ in range(2):                                   # the second round replays the graphs the first captured
        got = in_batches(eng, reqs, lens, [list(range(B))])
        want = in_batches(ref, reqs, lens, [list(range(B))])
        for r in range(B):
            assert_close(got[r][lens[r] - 1:], want[r][lens[r] - 1:], "bfloat16", f"request {r}")
    pcfg, pw = plain_llama.load_weights(folder)
    plain = plain_llama.forward(pcfg, pw, reqs[B - 1])
    assert_close(want[B - 1], plain, "float32", "the last request, float32")
    assert_close(got[B - 1], plain, "bfloat16", "the last request, bfloat16")
    eng.check_device_errors()
    eng.cache.check()


def test_cache_sized_from_the_memory_that_is_left(model_folders):
    """max_tokens=None: the cache takes `mem_fraction` of what the device has free beside the weights."""
    import gc

    from inferllm_b200 import Engine, EngineOptions
    gc.collect()
    torch.cuda.empty_cache()
    free, total = torch.cuda.mem_get_info()
    eng = Engine.from_folder(model_folders["A"], EngineOptions(dtype="bfloat16", max_tokens=None, mem_fraction=0.05,
                                                               max_batch=4, page_size=64))
    cfg = TINY["A"]
    per_token = 2 * cfg["num_hidden_layers"] * cfg.get("num_key_value_heads", cfg["num_attention_heads"]) \
        * (cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]) * 2
    held = eng.cache.pages_free()[0] * 64 * per_token
    assert 0.03 * free <= held <= 0.05 * total
    ids = random_prompt("A", 40, 1)
    assert whole(eng, ids).shape[0] == 40


def test_device_errors_name_the_kernel_family(model_folders):
    """A wait that runs out inside a kernel leaves a code in the device's error word;
    `check_device_errors` turns it into an error that says which family of kernels gave up, and
    clears it."""
    from inferllm_b200.engine import device_view
    from inferllm_b200.kernels import ops
    eng = make_engine(model_folders["A"], "bfloat16")
    word = device_view(eng.info()["tc_error_word"], (1,), torch.int32)
    for code, words in ((4, "matrix product"), (5, "prompt attention"), (7, "decode attention")):
        assert ops.selftest_wait_timeout(word, 1 << 18, code)[:2] == (code, 1)
        with pytest.raises(EngineError, match=words):
            eng.check_device_errors()
        eng.check_device_errors()
