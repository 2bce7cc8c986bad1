"""The generation loop's decisions, with a scripted stepper instead of a GPU: batching by cache
size, prompts in one step or in pieces, stop tokens, early enders, errors, slot reuse."""
from typing import List

import pytest

from xpu_serve_b200.engine.generate import generate, max_new_for, plan_batches
from xpu_serve_b200.sampling import GenerateRequest, SamplingParams


class FakeStepper:
    """Next token = (sum of the sequence's tokens so far) % 50, so the whole history matters.
    Checks what a real cache would: slots held once, steps only for live sequences."""

    def __init__(self, capacity_tokens=4096, max_context=512, max_slots=8, fail_at_step=None):
        self.capacity_tokens, self.max_context, self.max_slots = capacity_tokens, max_context, max_slots
        self.page_size = 64
        self.free = list(range(max_slots))
        self.hist = {}
        self.log = []
        self.peak_tokens = 0
        self.fail_at_step = fail_at_step

    def open(self, requests):
        assert len(requests) <= len(self.free), "more sequences than slots"
        hs = [self.free.pop(0) for _ in requests]
        for h in hs:
            self.hist[h] = []
        self.log.append(("open", list(hs)))
        return hs

    def close(self, handles):
        for h in handles:
            assert h in self.hist, "slot freed twice"
            del self.hist[h]
            self.free.append(h)
        self.free.sort()
        self.log.append(("close", list(handles)))

    def step(self, handles, token_lists, want):
        if self.fail_at_step is not None and sum(1 for e in self.log if e[0] == "step") == self.fail_at_step:
            self.fail_at_step = None
            raise RuntimeError("device fault (scripted)")
        out = []
        for h, toks, w in zip(handles, token_lists, want):
            assert h in self.hist and len(toks) >= 1
            self.hist[h] += list(toks)
            assert len(self.hist[h]) <= self.max_context
            out.append(sum(self.hist[h]) % 50 if w else None)
        held = sum(-(-len(v) // 64) * 64 for v in self.hist.values())
        assert held <= self.capacity_tokens
        self.peak_tokens = max(self.peak_tokens, held)
        self.log.append(("step", list(handles), [len(t) for t in token_lists], list(want)))
        return out


def expected(prompt: List[int], max_new: int, stops=()):
    hist, out = list(prompt), []
    while len(out) < max_new:
        t = sum(hist) % 50
        if t in stops:
            return out, "stop"
        out.append(t)
        hist.append(t)
    return out, "length"


GREEDY = SamplingParams(temperature=0.0)


def test_single_request_matches_the_scripted_model():
    st = FakeStepper()
    r = generate(st, [GenerateRequest([3, 4, 5], GREEDY, 6)])[0]
    assert (r.tokens, r.finish) == expected([3, 4, 5], 6)
    assert r.stats.prompt_tokens == 3 and r.stats.generated_tokens == 6
    steps = [e for e in st.log if e[0] == "step"]
    assert steps[0][2] == [3] and all(s[2] == [1] for s in steps[1:]) and len(steps) == 6   # 1 prompt + 5 decode
    assert st.hist == {} and st.free == list(range(8))


def test_unequal_batch_shorter_requests_leave_early():
    st = FakeStepper()
    prompts = [[1] * 5, [2] * 9, [3] * 13]
    news = [2, 7, 4]
    res = generate(st, [GenerateRequest(p, GREEDY, n) for p, n in zip(prompts, news)])
    for r, p, n in zip(res, prompts, news):
        assert (r.tokens, r.finish) == expected(p, n)
        assert r.stats.batch_size == 3
    steps = [e for e in st.log if e[0] == "step"]
    assert steps[0][2] == [5, 9, 13]                                  # the prompts run in ONE step
    assert [len(s[1]) for s in steps[1:]] == [3, 2, 2, 1, 1, 1]        # 2, then 4, then 7 tokens reached
    closes = [e[1] for e in st.log if e[0] == "close"]
    assert closes == [[0], [2], [1]]                                  # each slot is given back when its sequence ends


def test_stop_token_is_not_returned():
    p = [7, 7, 7]
    full, _ = expected(p, 10)
    stop = full[3]
    want, finish = expected(p, 10, stops=(stop,))
    r = generate(FakeStepper(), [GenerateRequest(p, GREEDY, 10, [stop])])[0]
    assert r.finish == "stop" and r.tokens == want and stop not in r.tokens
    first = generate(FakeStepper(), [GenerateRequest(p, GREEDY, 10, [full[0]])])[0]
    assert first.finish == "stop" and first.tokens == []


def test_errors_do_not_touch_the_other_requests():
    st = FakeStepper(max_context=32)
    res = generate(st, [GenerateRequest([], GREEDY, 4), GenerateRequest([1] * 32, GREEDY, 4),
                        GenerateRequest([2, 3], GREEDY, 4),
                        GenerateRequest([5], SamplingParams(top_p=0.0), 4)])
    assert res[0].finish == "error" and res[0].error == "empty prompt"
    assert res[1].finish == "error" and "does not fit the context limit of 32" in res[1].error
    assert res[3].finish == "error" and "top_p" in res[3].error
    assert (res[2].tokens, res[2].finish) == expected([2, 3], 4)


def test_max_new_is_clamped_to_the_context():
    st = FakeStepper(max_context=10)
    r = generate(st, [GenerateRequest([1] * 7, GREEDY, 100)])[0]
    assert r.finish == "length" and len(r.tokens) == 3
    assert max_new_for(GenerateRequest([1] * 7, GREEDY, 100), 10) == 3
    z = generate(st, [GenerateRequest([1, 2], GREEDY, 0)])[0]
    assert z.finish == "length" and z.tokens == []
    assert all(e[3] == [False] for e in st.log if e[0] == "step" and e[2] == [2])   # nothing wanted, nothing sampled


def test_batches_follow_one_another_and_slots_are_reused():
    st = FakeStepper(capacity_tokens=64 * 5, max_slots=8)
    reqs = [GenerateRequest([i + 1] * (10 + 30 * i), GREEDY, 5) for i in range(5)]    # 64,64,128,128,192 tokens held
    plan = plan_batches(reqs, range(5), 8, 64 * 5, 64, st.max_context)
    assert plan == [[0, 1, 2], [3, 4]]
    res = generate(st, reqs)
    for r, q in zip(res, reqs):
        assert (r.tokens, r.finish) == expected(q.prompt, 5)
    opens = [e[1] for e in st.log if e[0] == "open"]
    assert opens == [[0, 1, 2], [0, 1]]                      # the second batch gets the first batch's slots
    assert st.peak_tokens <= 64 * 5
    assert plan_batches(reqs, range(5), 2, 10 ** 9, 64, 512) == [[0, 1], [2, 3], [4]]


def test_request_larger_than_the_cache_is_an_error():
    st = FakeStepper(capacity_tokens=128)
    r = generate(st, [GenerateRequest([1] * 100, GREEDY, 100)])[0]
    assert r.finish == "error" and "does not fit the cache" in r.error


def test_prompts_in_pieces():
    st = FakeStepper()
    prompts = [[1] * 20, [2] * 3, [3] * 11]
    res = generate(st, [GenerateRequest(p, GREEDY, 3) for p in prompts], prefill_chunk=8)
    for r, p in zip(res, prompts):
        assert (r.tokens, r.finish) == expected(p, 3)
    steps = [e for e in st.log if e[0] == "step"]
    assert [s[2] for s in steps[:5]] == [[8], [8], [4, 3, 1], [8], [2]]
    assert [s[3] for s in steps[:5]] == [[False], [False], [True, True, False], [False], [True]]


def test_callback_cancels_one_request():
    seen = []

    def on_token(i, t):
        seen.append((i, t))
        return not (i == 1 and len([1 for j, _ in seen if j == 1]) == 2)

    res = generate(FakeStepper(), [GenerateRequest([1, 2], GREEDY, 5), GenerateRequest([3, 4], GREEDY, 5)], on_token)
    assert res[0].finish == "length" and len(res[0].tokens) == 5
    assert res[1].finish == "cancelled" and len(res[1].tokens) == 2


def test_a_failing_step_fails_the_batch_and_frees_its_slots():
    st = FakeStepper(fail_at_step=2)
    res = generate(st, [GenerateRequest([1, 2], GREEDY, 1), GenerateRequest([3, 4], GREEDY, 5),
                        GenerateRequest([5, 6], GREEDY, 5)], max_batch=2)
    assert res[0].finish == "length" and len(res[0].tokens) == 1      # had ended before the fault
    assert res[1].finish == "error" and "scripted" in res[1].error and len(res[1].tokens) == 2
    assert st.hist == {} and st.free == list(range(8))
    assert res[2].finish == "length" and len(res[2].tokens) == 5      # the next batch runs


def test_sampling_params_meaning():
    assert SamplingParams(temperature=0).greedy() and SamplingParams(top_k=1).greedy()
    assert not SamplingParams().greedy()
    assert not SamplingParams(temperature=0).needs_logits()
    assert SamplingParams(temperature=0, repetition_penalty=1.1).needs_logits()
