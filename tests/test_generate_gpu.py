"""Generation through the Python entry point, and the sampling kernels, against the plain
implementation."""
import numpy as np
import pytest
import torch

import plain_lfm3 as plain
import tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen_models")
    return {(n, d): tiny.make_folder(root, n, d) for n in ("A", "B", "W") for d in ("float32", "bfloat16")}


def plain_greedy(cfg, W, prompt, n, stops=()):
    seq, out, margins = list(prompt), [], []
    for _ in range(n):
        logits = plain.forward(cfg, W, seq)[-1]
        order = np.argsort(-logits)
        t = int(order[0])
        if t in stops:
            break
        margins.append(float(logits[order[0]] - logits[order[1]]) / float(np.abs(logits).max()))
        out.append(t)
        seq.append(t)
    return out, margins


@pytest.mark.parametrize("name,lengths,steps", [("A", (5, 9, 13), 8), ("B", (1, 4, 7, 16, 23), 12), ("W", (3, 50, 41), 10)])
def test_greedy_float32_matches_plain(folders, name, lengths, steps):
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    folder = folders[(name, "float32")]
    cfg, W = plain.load_folder(folder)
    engine = Engine(folder, precision="f32", ctx=256, max_batch=8)
    prompts = [tiny.prompt(name, n, salt=i) for i, n in enumerate(lengths)]
    res = engine.generate([GenerateRequest(p, SamplingParams(temperature=0.0), steps, []) for p in prompts])
    for p, r in zip(prompts, res):
        want, margins = plain_greedy(cfg, W, p, steps)
        assert min(margins) > 1e-4, "the test's own tokens are near ties; pick another prompt"
        assert r.finish == "length" and r.tokens == want
    engine.stepper.cache.check()
    assert engine.stepper.cache.slots.held_count == 0


def test_greedy_bfloat16_follows_plain_until_a_near_tie(folders):
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    folder = folders[("A", "bfloat16")]
    cfg, W = plain.load_folder(folder)
    engine = Engine(folder, precision="bf16", ctx=256, max_batch=8)
    prompts = [tiny.prompt("A", n, salt=i) for i, n in enumerate((5, 9, 13))]
    res = engine.generate([GenerateRequest(p, SamplingParams(temperature=0.0), 8, []) for p in prompts])
    for p, r in zip(prompts, res):
        seq = list(p)
        for t in r.tokens:
            logits = plain.forward(cfg, W, seq)[-1]
            best = int(np.argmax(logits))
            assert t == best or (logits[best] - logits[t]) / np.abs(logits).max() < 2e-2
            seq.append(t)


@pytest.mark.parametrize("name,precision", [("W", "f32"), ("B", "f32"), ("W", "bf16")])
def test_prompts_in_pieces_of_16_tokens(folders, name, precision):
    """`prefill_chunk=16`: a batch's prompts go through the step function 16 tokens a step (a piece may end
    in the middle of one prompt and the next step go on from there; src/engine/engine.cpp:296-313 cuts a
    single prompt the same way). The tokens are the plain greedy run's."""
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    dtype = {"f32": "float32", "bf16": "bfloat16"}[precision]
    folder = folders[(name, dtype)]
    cfg, W = plain.load_folder(folder)
    engine = Engine(folder, precision=precision, ctx=256, max_batch=8, prefill_chunk=16)
    steps = []
    real = engine.stepper.step
    engine.stepper.step = lambda h, t, w: (steps.append([len(x) for x in t]), real(h, t, w))[1]
    prompts = [tiny.prompt(name, n, salt=60 + i) for i, n in enumerate((5, 50, 41, 23))]
    res = engine.generate([GenerateRequest(p, SamplingParams(temperature=0.0), 6, []) for p in prompts])
    prompt_steps = [s for s in steps if max(s) > 1]
    assert len(prompt_steps) == 8 and all(sum(s) <= 16 for s in prompt_steps)        # 119 tokens, 16 a step
    assert [5, 11] in prompt_steps                # a step that ends one prompt and starts the next one
    for p, r in zip(prompts, res):
        assert r.finish == "length"
        if precision == "f32":
            want, margins = plain_greedy(cfg, W, p, 6)
            assert min(margins) > 1e-4, "the test's own tokens are near ties; pick another prompt"
            assert r.tokens == want
        else:
            seq = list(p)
            for t in r.tokens:
                logits = plain.forward(cfg, W, seq)[-1]
                best = int(np.argmax(logits))
                assert t == best or (logits[best] - logits[t]) / np.abs(logits).max() < min(2e-2, 2 * tiny.bound(name, dtype))
                seq.append(t)
    engine.stepper.cache.check()
    assert engine.stepper.cache.slots.held_count == 0


def test_stop_tokens_and_early_enders(folders):
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    folder = folders[("B", "float32")]
    cfg, W = plain.load_folder(folder)
    engine = Engine(folder, precision="f32", ctx=128, max_tokens=64 * 4, max_batch=3)
    prompts = [tiny.prompt("B", n, salt=i) for i, n in enumerate((4, 7, 16, 23, 2))]
    free_run = [plain_greedy(cfg, W, p, 10)[0] for p in prompts]
    stops = [[free_run[0][3]], [], [free_run[2][0]], [free_run[3][9]], []]
    news = [10, 3, 10, 10, 6]
    res = engine.generate([GenerateRequest(p, SamplingParams(temperature=0.0), n, s)
                           for p, n, s in zip(prompts, news, stops)])
    for p, r, n, s in zip(prompts, res, news, stops):
        want, _ = plain_greedy(cfg, W, p, n, s)
        assert r.tokens == want
        assert r.finish == ("stop" if len(want) < n else "length")
    assert [r.stats.batch_size for r in res] == [3, 3, 3, 2, 2]      # two batches, one after the other
    engine.stepper.cache.check()


def test_seeded_sampling_matches_plain_sampler(folders):
    """Temperature 0.8 with a seed: the kernel's choice equals the plain sampler's given the same
    uniform, step after step (configuration B's workload: prompts 1/4/7/16/23, 12 steps)."""
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    folder = folders[("B", "float32")]
    cfg, W = plain.load_folder(folder)
    engine = Engine(folder, precision="f32", ctx=128, max_batch=8)
    prompts = [tiny.prompt("B", n, salt=i) for i, n in enumerate((1, 4, 7, 16, 23))]
    params = [SamplingParams(temperature=0.8, seed=11 + i) for i in range(3)] + \
             [SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=5),
              SamplingParams(temperature=1.3, min_p=0.05, top_p=0.95, seed=2 ** 63 + 9)]
    res = engine.generate([GenerateRequest(p, sp, 12, []) for p, sp in zip(prompts, params)])
    again = engine.generate([GenerateRequest(p, sp, 12, []) for p, sp in zip(prompts, params)])
    for p, sp, r, r2 in zip(prompts, params, res, again):
        assert r.tokens == r2.tokens, "the same seed gives the same tokens"
        seq = list(p)
        for step, t in enumerate(r.tokens):
            logits = plain.forward(cfg, W, seq)[-1]
            u = plain.uniform(sp.seed, step)
            want = plain.sample(logits, sp.temperature, sp.top_k, sp.top_p, sp.min_p, u)
            if t != want:    # only a uniform that lands within rounding of a boundary may differ
                w = plain.kept_weights(logits, sp.temperature, sp.top_k, sp.top_p, sp.min_p)
                c = np.cumsum(w) / w.sum()
                assert min(abs(c[t] - u), abs(c[want] - u), abs(c[t - 1] - u)) < 1e-5, (step, t, want)
            seq.append(t)


def test_sampling_kernel_distribution_and_cuts():
    """The kernel's kept set and draw against the plain sampler over many uniforms, on logits with
    ties, a wide vocabulary that is no power of two, and every combination of cuts."""
    from xpu_serve_b200.ops import lib as ops
    rng = np.random.default_rng(0)
    # 5,003: one CTA a row; 16,384 and 20,011: a row shared by a cluster of CTAs, with and without 16-byte loads
    for V, n in ((5003, 256), (16384, 16), (20011, 9)):
        base = rng.normal(0, 2.5, size=V).astype(np.float32)
        base[100:110] = base[100]                     # ties inside the likely region
        base[V - 3] = base[V // 2] = base[100]        # and across the parts of the row that different CTAs read
        base[7] = base.max() + 0.5
        cases = [(1.0, 0, 1.0, 0.0), (0.7, 50, 1.0, 0.0), (1.0, 0, 0.9, 0.0), (1.5, 0, 1.0, 0.02),
                 (0.9, 200, 0.8, 0.01), (1.0, 3, 0.5, 0.0), (2.0, V, 0.999, 0.0), (1.0, 12, 1.0, 0.5)]
        for temp, k, p, mp in cases:
            logits = torch.tensor(np.tile(base, (n, 1)), device="cuda")
            seeds = torch.arange(n, dtype=torch.int64, device="cuda") * 7919 + 3
            counters = torch.arange(n, dtype=torch.int64, device="cuda") % 5
            out = torch.empty(n, dtype=torch.int32, device="cuda")
            f = lambda v, dt=torch.float32: torch.full((n,), v, dtype=dt, device="cuda")   # noqa: E731
            ops.sample(logits, f(temp), f(k, torch.int32), f(p), f(mp), seeds, counters, out)
            got = out.cpu().numpy()
            w = plain.kept_weights(base, temp, k, p, mp)
            assert (w[got] > 0).all(), f"a dropped token was drawn with cuts {temp, k, p, mp} of {V}"
            miss = 0
            for i in range(n):
                u = plain.uniform(int(seeds[i]), int(counters[i]))
                assert ops.uniform(int(seeds[i]), int(counters[i])) == u
                miss += int(plain.sample(base, temp, k, p, mp, u) != got[i])
            assert miss <= 1, f"{miss} draws differ with cuts {temp, k, p, mp} of {V}"
    # greedy rows: temperature 0 or top_k 1 pick the first largest (the last, wide row: a cluster of CTAs)
    logits = torch.tensor(np.tile(base, (4, 1)), device="cuda")
    logits[1, 3] = logits[1, 7]                                  # a tie: the lower index wins
    logits[2, V - 5] = logits[2, 7]                              # also when another CTA holds the other one
    out = torch.empty(4, dtype=torch.int32, device="cuda")
    ops.sample(logits, torch.tensor([0.0, 0.0, 1.0, 1.0], device="cuda"),
               torch.tensor([0, 0, 1, 1], dtype=torch.int32, device="cuda"), torch.ones(4, device="cuda"),
               torch.zeros(4, device="cuda"), torch.zeros(4, dtype=torch.int64, device="cuda"),
               torch.zeros(4, dtype=torch.int64, device="cuda"), out)
    assert out.tolist() == [7, 3, 7, 7]
    ops.argmax(logits, out)
    assert out.tolist() == [7, 3, 7, 7]


def test_penalties_match_plain(folders):
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    folder = folders[("A", "float32")]
    cfg, W = plain.load_folder(folder)
    engine = Engine(folder, precision="f32", ctx=128, max_batch=4)
    prompts = [tiny.prompt("A", n, salt=i) for i, n in enumerate((6, 11))]
    sp = [SamplingParams(temperature=0.0, repetition_penalty=1.3, presence_penalty=0.2, frequency_penalty=0.1),
          SamplingParams(temperature=0.0, repetition_penalty=1.0, presence_penalty=0.0, frequency_penalty=0.7)]
    res = engine.generate([GenerateRequest(p, s, 10, []) for p, s in zip(prompts, sp)])
    for p, s, r in zip(prompts, sp, res):
        seq, gen = list(p), []
        for t in r.tokens:
            logits = plain.apply_penalties(plain.forward(cfg, W, seq)[-1], p, gen, s.repetition_penalty,
                                           s.presence_penalty, s.frequency_penalty)
            best = int(np.argmax(logits))
            assert t == best or abs(logits[best] - logits[t]) < 1e-5 * np.abs(logits).max()
            seq.append(t)
            gen.append(t)


@pytest.mark.parametrize("kind", ["greedy", "sampled", "penalties", "mixed"])
def test_running_ahead_changes_no_token(folders, monkeypatch, kind):
    """Batches decode with the next step already started on the device, fed there with the tokens that the
    graph's argmax or the sampling kernels chose. Stop tokens that end one sequence in the middle, unequal
    lengths, a page boundary (64) crossed while running ahead, a sequence that reaches the context's end, a
    callback that cancels: the same tokens as without running ahead, for greedy sequences, seeded draws,
    penalties (whose token counts the step that runs ahead updates too) and a batch that mixes them."""
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    folder = folders[("A", "float32")]
    how = {
        "greedy": lambda i: SamplingParams(temperature=0.0),
        "sampled": lambda i: SamplingParams(temperature=0.9, top_p=0.95, top_k=60, seed=100 + i),
        "penalties": lambda i: SamplingParams(temperature=0.0 if i % 2 else 0.8, repetition_penalty=1.3,
                                              frequency_penalty=0.2, presence_penalty=0.1, seed=7 + i),
        "mixed": lambda i: SamplingParams(temperature=0.0) if i % 2 else SamplingParams(temperature=1.1, min_p=0.02, seed=i),
    }[kind]
    prompts = [tiny.prompt("A", n, salt=40 + i) for i, n in enumerate((60, 3, 17, 100))]

    def run(ahead, stops, cancel_at=None):
        monkeypatch.setenv("XS_NO_RUN_AHEAD", "0" if ahead else "1")
        engine = Engine(folder, precision="f32", ctx=128, max_batch=8)
        assert engine.stepper.run_ahead == ahead
        seen = []
        ran_ahead = [0]
        take = engine.stepper._take_ahead

        def counting_take(*a):
            ran_ahead[0] += 1
            return take(*a)

        engine.stepper._take_ahead = counting_take

        def on_token(i, t):
            seen.append((i, t))
            return not (cancel_at is not None and i == 2 and sum(1 for j, _ in seen if j == 2) >= cancel_at)

        reqs = [GenerateRequest(p, how(i), n, list(stops)) for i, (p, n) in enumerate(zip(prompts, (40, 30, 25, 60)))]
        res = engine.generate(reqs, on_token)
        if ahead:
            assert ran_ahead[0] > 20, "the steps did not run ahead"
        engine.stepper.cache.check()
        assert engine.stepper.cache.slots.held_count == 0
        return [(r.finish, r.tokens) for r in res]

    plain_run = run(False, [])
    assert plain_run[3][0] == "length" and len(plain_run[3][1]) == 28        # 100 + 28 = the context of 128
    assert run(True, []) == plain_run
    # a stop token that sequence 1 meets in the middle of its run
    stop = plain_run[1][1][7]
    with_stop = run(False, [stop])
    assert any(f == "stop" for f, _ in with_stop)
    assert run(True, [stop]) == with_stop
    assert run(True, [], cancel_at=5) == run(False, [], cancel_at=5)


def test_running_ahead_refuses_another_token(folders):
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    engine = Engine(folders[("A", "float32")], precision="f32", ctx=128, max_batch=4)
    st = engine.stepper
    reqs = [GenerateRequest(tiny.prompt("A", 5, salt=1), SamplingParams(temperature=0.0), 8, [])]
    hs = st.open(reqs)
    (t0,) = st.step(hs, [reqs[0].prompt], [True])
    (t1,) = st.step(hs, [[t0]], [True])           # from here on the next step is already running
    with pytest.raises(RuntimeError, match="one decode step ahead"):
        st.step(hs, [[(t1 + 1) % 512]], [True])
    st.close(hs)


def test_a_tcgen05_wait_that_gave_up_fails_the_step(folders, tmp_path):
    """The tcgen05 kernels bound their waits and set a status word when one runs out; what they computed is
    then partial. No wait is made to run out here: the word is set by hand, as a kernel would have left it.
    The generation loop reads it with the tokens it waits for anyway and fails the batch; replay reads it
    with the logits; the word is cleared, and the next call works."""
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    from xpu_serve_b200.engine.replay import Replayer
    from xpu_serve_b200.ops import lib as ops
    folder = folders[("A", "bfloat16")]
    engine = Engine(folder, precision="bf16", ctx=128, max_batch=4)
    dev = engine.model.rt.device
    reqs = [GenerateRequest(tiny.prompt("A", n, salt=80 + i), SamplingParams(temperature=0.0), 5, []) for i, n in enumerate((9, 4))]
    good = engine.generate(reqs)
    assert all(r.finish == "length" for r in good)

    def as_a_kernel_would():
        ops.gemm_tc_status(dev).fill_(3)
        ops._tc_unread.add(ops.gemm_tc_status(dev).device)

    as_a_kernel_would()
    bad = engine.generate(reqs)
    assert all(r.finish == "error" and "tcgen05" in r.error and r.tokens == [] for r in bad)
    assert ops.gemm_tc_status(dev).item() == 0 and not ops.tc_status_unread(dev)
    engine.stepper.cache.check()
    assert engine.stepper.cache.slots.held_count == 0
    assert [r.tokens for r in engine.generate(reqs)] == [r.tokens for r in good]
    rp = Replayer(engine.model, 256, None)
    as_a_kernel_would()
    step = {"step": 0, "entries": [{"id": "a", "tokens": reqs[0].prompt, "want": [0]}], "end": []}
    with pytest.raises(ops.KernelError, match="tcgen05"):
        rp.run_step(step)
    assert rp.cache.slots.held_count == 0 and ops.gemm_tc_status(dev).item() == 0
    assert rp.run_step(dict(step, end=["a"])) is not None
