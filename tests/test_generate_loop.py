"""Decisions of the library's generation loop, with stand-ins for the engine and the sampler (no
GPU).  The loop (engine/generate.cpp) keeps the host one step behind the device: sampled tokens feed
the next step without being looked at, and a sequence that turns out to have sampled a stop token has
been run one step too far.  Its decisions (which tokens come out, why each request ended, which
requests ran together) are compared with a plain loop written out below, which looks at every token
before it takes the next step."""
import pytest

from util import plain_generate

from inferllm_b200.engine import Limits, RequestTooLong, generate, plan_batches


class FakeBackend:
    """Keeps the bookkeeping a real engine would and returns 'logits' that simply name, for each
    wanted place, (slot, position) so that a scripted chooser can answer."""

    def __init__(self, max_batch=2, num_pages=8, page_size=4, max_seq_len=16):
        self.lim = Limits(max_batch, num_pages, page_size, max_seq_len)
        self.free = list(range(max_batch))[::-1]
        self.len = {}
        self.log = []
        self.fed = []
        self.peak_pages = 0

    def limits(self):
        return self.lim

    def new_sequence(self):
        s = self.free.pop()
        self.len[s] = 0
        return s

    def end_sequence(self, slot):
        assert slot in self.len, "slot freed twice"
        del self.len[slot]
        self.free.append(slot)

    def step(self, items, device_ids=None):
        assert len({it.slot for it in items}) == len(items)
        if device_ids is not None:
            assert len(device_ids) == len(items) and all(len(it.tokens) == 1 for it in items)
            self.fed.append([int(t) for t in device_ids])
        out = []
        for it in items:
            assert it.slot in self.len and len(it.tokens) >= 1
            assert (self.len[it.slot] == 0) or len(it.tokens) == 1, "prompts only at the start"
            self.len[it.slot] += len(it.tokens)
            assert self.len[it.slot] <= self.lim.max_seq_len
            for w in it.want:
                out.append((it.slot, self.len[it.slot] - len(it.tokens) + w, tuple(it.tokens)))
        pages = sum(-(-n // self.lim.page_size) for n in self.len.values())
        assert pages <= self.lim.num_pages
        self.peak_pages = max(self.peak_pages, pages)
        self.log.append([(it.slot, len(it.tokens)) for it in items])
        return out


def scripted(script):
    """chooser: request r's k-th generated token is script[r][k]."""
    def choose(logits, requests, steps, histories):
        assert len(logits) == len(requests)
        return [script[r][s] for r, s in zip(requests, steps)]
    return choose


def test_plan_batches_by_slots_and_pages():
    lim = Limits(max_batch=3, num_pages=6, page_size=4, max_seq_len=16)
    assert plan_batches([3, 3, 3, 3], 1, lim) == [[0, 1, 2], [3]]
    assert plan_batches([8, 8, 8], 4, lim) == [[0, 1], [2]]          # 3 pages each
    with pytest.raises(RequestTooLong, match="longest sequence"):
        plan_batches([17], 1, lim)
    with pytest.raises(RequestTooLong, match="empty"):
        plan_batches([0], 1, lim)
    with pytest.raises(RequestTooLong, match="pages"):
        plan_batches([12], 8, Limits(3, 3, 4, 32))


def test_stop_tokens_end_sequences_early_and_are_kept():
    be = FakeBackend()
    script = {0: [7, 9, 8, 8, 8], 1: [4, 4, 4, 9, 8]}
    res = generate(be, [[1, 2, 3], [1]], scripted(script), max_new_tokens=5, stop_ids=[9])
    assert res.tokens == [[7, 9], [4, 4, 4, 9]]
    assert res.finish == ["stop", "stop"]
    # the prompts, then steps of both requests; request 0 (slot 0) sampled its stop token in the second
    # step and is seen one step late, so it is stepped once more and then dropped; request 1 likewise
    assert be.log[0] == [(0, 3), (1, 1)] and be.log[1] == [(0, 1), (1, 1)] and be.log[2] == [(0, 1), (1, 1)]
    assert all(step == [(1, 1)] for step in be.log[3:]) and len(be.log) == 5
    assert be.len == {} and sorted(be.free) == [0, 1]
    assert res.prefill_tokens == 4 and res.decode_tokens == 4 and res.decode_steps == 3
    # what was fed back is what was sampled, in the order of the step's sequences
    assert be.fed[0] == [7, 4] and be.fed[1] == [9, 4]


def test_max_new_tokens_and_no_step_after_the_last_token():
    be = FakeBackend()
    res = generate(be, [[1, 2]], scripted({0: [5, 6, 7, 8]}), max_new_tokens=3)
    assert res.tokens == [[5, 6, 7]] and res.finish == ["length"]
    assert len(be.log) == 3  # prefill + 2 decode steps; the third token is never fed back


def test_context_limit():
    be = FakeBackend(max_seq_len=6, num_pages=8)
    res = generate(be, [[1, 2, 3, 4]], scripted({0: [5] * 10}), max_new_tokens=10)
    # positions 0..5 hold 4 prompt + 2 generated tokens; the third generated token has no place
    assert res.tokens == [[5, 5, 5]] and res.finish == ["context"]
    assert be.len == {}


def test_batches_run_one_after_another_and_reuse_slots():
    be = FakeBackend(max_batch=2, num_pages=4, page_size=4, max_seq_len=8)
    prompts = [[1] * 3, [2] * 2, [3] * 4, [4], [5] * 2]
    script = {r: [10 + r] * 4 for r in range(5)}
    seen = []
    res = generate(be, prompts, scripted(script), max_new_tokens=2, on_token=lambda r, t: seen.append((r, t)))
    assert res.batches == [[0, 1], [2, 3], [4]]
    assert res.tokens == [[10 + r] * 2 for r in range(5)]
    assert [n for _, n in be.log[0]] == [3, 2] and [n for _, n in be.log[2]] == [4, 1]
    assert {s for s, _ in be.log[2]} == {0, 1} and len(be.log[4]) == 1   # the same two slots again
    assert sorted(seen) == sorted((r, 10 + r) for r in range(5) for _ in range(2))
    assert be.peak_pages <= 4 and be.len == {}


def test_the_chooser_gets_the_prompts_once_and_keeps_the_history_itself():
    be = FakeBackend()
    got = []

    def choose(logits, requests, steps, histories):
        got.append((list(requests), list(steps), None if histories is None else [list(h) for h in histories]))
        return [9 for _ in requests]

    generate(be, [[1, 2], [3]], choose, max_new_tokens=3)
    assert got == [([0, 1], [0, 0], [[1, 2], [3]]), ([0, 1], [1, 1], None), ([0, 1], [2, 2], None)]


def test_slots_are_returned_when_a_step_raises():
    class Boom(FakeBackend):
        def step(self, items, device_ids=None):
            if len(self.log) == 1:
                raise RuntimeError("boom")
            return super().step(items, device_ids)

    be = Boom()
    with pytest.raises(RuntimeError, match="boom"):
        generate(be, [[1], [2]], scripted({0: [5] * 3, 1: [5] * 3}), max_new_tokens=3)
    assert be.len == {} and sorted(be.free) == [0, 1]


def test_zero_new_tokens():
    be = FakeBackend()
    res = generate(be, [[1]], scripted({0: []}), max_new_tokens=0)
    assert res.tokens == [[]] and be.log == [] and res.finish == ["length"]


@pytest.mark.parametrize("max_new,stop,max_seq", [(5, [9], 16), (3, [], 16), (10, [9], 6), (1, [9], 16), (4, [7, 4], 16)])
def test_the_loop_decides_like_the_plain_loop(max_new, stop, max_seq):
    """The library's loop returns what the plain loop returns, feeds the tokens it sampled, and gives
    every slot back, although sequences that hit a stop token have been run one step too far."""
    prompts = [[1, 2, 3], [1], [5, 5], [2, 2, 2, 2], [8]]
    script = {0: [7, 9, 8, 8, 8, 1, 1, 1, 1, 1], 1: [4, 4, 4, 9, 8, 1, 1, 1, 1, 1], 2: [9] * 10, 3: [3] * 10,
              4: [6, 6, 6, 6, 6, 6, 6, 9, 9, 9]}
    a = FakeBackend(max_batch=3, num_pages=12, page_size=4, max_seq_len=max_seq)
    b = FakeBackend(max_batch=3, num_pages=12, page_size=4, max_seq_len=max_seq)
    want_tokens, want_finish, want_batches = plain_generate(a, prompts, scripted(script), max_new, stop)
    got = generate(b, prompts, scripted(script), max_new, stop)
    assert got.tokens == want_tokens and got.finish == want_finish and got.batches == want_batches
    assert b.len == {} and sorted(b.free) == [0, 1, 2]
    # every token fed back is one that was sampled for that step
    flat = [t for step in b.fed for t in step]
    assert all(t in {x for v in script.values() for x in v} for t in flat)
    assert got.decode_tokens + len(prompts) == sum(len(t) for t in got.tokens)
    # a backend that hands the sampled tokens to the host by a copy of its own (started right after
    # the sampling, read one step later, possibly after some of its sequences were dropped)
    c = FakeBackend(max_batch=3, num_pages=12, page_size=4, max_seq_len=max_seq)
    c.reads = 0

    def read_tokens_async(toks):
        snapshot = [int(t) for t in toks]

        def result():
            c.reads += 1
            return snapshot
        return result
    c.read_tokens_async = read_tokens_async
    again = generate(c, prompts, scripted(script), max_new, stop)
    assert again.tokens == want_tokens and again.finish == want_finish and c.len == {}
    assert c.reads >= 1


def test_a_batch_is_stepped_longest_prompt_first():
    """The loop puts a batch's sequences into every step longest first (the attention kernels hand
    out their blocks in that order) and keeps the results by request."""
    prompts = [[1], [1, 2, 3, 4, 5], [1, 2], [1, 2, 3]]
    script = {r: [10 + r] * 3 for r in range(4)}
    be = FakeBackend(max_batch=4, num_pages=16, page_size=4, max_seq_len=16)
    res = generate(be, prompts, scripted(script), 3, [])
    assert res.tokens == [[10 + r] * 3 for r in range(4)]
    assert [n for _, n in be.log[0]] == [5, 3, 2, 1]               # the prompts, longest first
    first = [slot for slot, _ in be.log[0]]
    assert all([slot for slot, _ in step] == first for step in be.log[1:3])   # and so in the steps after


def test_timing_uses_the_callers_clock():
    t = [0.0]

    def clock():
        t[0] += 1.0
        return t[0]

    res = generate(FakeBackend(), [[1, 2]], scripted({0: [5, 6, 7]}), max_new_tokens=3, clock=clock)
    assert res.decode_steps == 2 and res.prefill_s > 0 and res.decode_s > 0 and len(res.step_s) == 2
