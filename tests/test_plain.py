"""The plain implementation against the reference project's own LFM3 code (golden logits made by
tests/golden/make_golden.py with the reference's CPU backend), and against hand-made cases that a
mistaken reading of a formula would fail."""
import json
import os

import numpy as np
import pytest

import plain_lfm3 as plain
import tiny

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_matches_the_reference_cpu_backend(tmp_path):
    with open(os.path.join(GOLDEN, "lfm3_R_last_logits.json")) as f:
        meta = json.load(f)
    ref = np.fromfile(os.path.join(GOLDEN, "lfm3_R_last_logits.f32"), dtype="<f4").reshape(len(meta["lengths"]), meta["vocab"])
    folder = tiny.make_folder(tmp_path, meta["config"], meta["dtype"])
    cfg, W = plain.load_folder(folder)
    for row, n in zip(ref, meta["lengths"]):
        got = plain.forward(cfg, W, tiny.prompt(meta["config"], n))[-1]
        gap = np.abs(got - row).max() / np.abs(row).max()
        assert gap < 2e-6, f"length {n}: gap {gap:.3e}"       # the reference keeps float32 values between ops
        assert int(got.argmax()) == int(row.argmax())


def test_rms_norm_no_offset():
    x = np.array([[3.0, 4.0]])
    w = np.array([0.5, 2.0])
    want = x / np.sqrt(12.5 + 1e-6) * w
    assert np.allclose(plain.rms_norm(x, w, 1e-6), want, rtol=1e-12)
    assert not np.allclose(plain.rms_norm(x, w, 1e-6), x / np.sqrt(12.5 + 1e-6) * (1 + w))


def test_rope_pairs_are_half_apart_and_tail_is_untouched():
    D, pairs = 8, 2
    inv = plain.rope_inv_freq(100.0, D, pairs)
    assert inv[2] == 0 and inv[3] == 0 and inv[0] == 1.0 and abs(inv[1] - 100.0 ** (-2 / 8)) < 1e-7
    x = np.arange(1.0, 9.0).reshape(1, 1, D)
    y = plain.rope(x, np.array([3]), inv)
    a = 3 * inv[1]
    assert np.isclose(y[0, 0, 1], x[0, 0, 1] * np.cos(a) - x[0, 0, 5] * np.sin(a))    # channel 1 pairs with 5
    assert np.isclose(y[0, 0, 5], x[0, 0, 5] * np.cos(a) + x[0, 0, 1] * np.sin(a))
    assert y[0, 0, 2] == x[0, 0, 2] and y[0, 0, 7] == x[0, 0, 7]                       # beyond the rotated pairs
    assert np.allclose(plain.rope(x, np.array([0]), inv), x)


def test_causal_conv_last_tap_multiplies_the_current_token():
    g = np.array([[1.0], [10.0], [100.0]])
    w = np.array([[2.0, 3.0, 5.0]])      # taps j = 0, 1, 2
    out = plain.causal_conv(g, w)
    assert out[:, 0].tolist() == [5.0, 3.0 + 50.0, 2.0 + 30.0 + 500.0]


def test_attention_masks_window_and_groups():
    T, D = 6, 4
    rng = np.random.default_rng(0)
    q = rng.normal(size=(T, 4, D))
    k = rng.normal(size=(T, 2, D))
    v = rng.normal(size=(T, 2, D))
    full = plain.attention(q, k, v, 0.5, 0)
    assert np.allclose(full[0, 0], v[0, 0]) and np.allclose(full[0, 3], v[0, 1])     # heads 2, 3 read kv head 1
    win = plain.attention(q, k, v, 0.5, 2)
    s = 0.5 * (k[4:6, 0] @ q[5, 1])
    p = np.exp(s - s.max())
    assert np.allclose(win[5, 1], (p / p.sum()) @ v[4:6, 0])                         # exactly the last two keys
    assert not np.allclose(win[5, 1], full[5, 1])


def test_sampler_cuts_follow_the_reference_order():
    logits = np.log(np.array([0.5, 0.2, 0.2, 0.06, 0.04]))
    w = plain.kept_weights(logits, 1.0, 0, 1.0, 0.0)
    assert np.allclose(w / w.sum(), [0.5, 0.2, 0.2, 0.06, 0.04])
    assert np.count_nonzero(plain.kept_weights(logits, 1.0, 2, 1.0, 0.0)) == 2
    assert np.nonzero(plain.kept_weights(logits, 1.0, 2, 1.0, 0.0))[0].tolist() == [0, 1]   # a tie: the lower id first
    assert np.count_nonzero(plain.kept_weights(logits, 1.0, 0, 0.6, 0.0)) == 2       # stops after reaching 0.6
    assert np.count_nonzero(plain.kept_weights(logits, 1.0, 0, 0.5, 0.0)) == 1       # kept / total >= top_p at the first
    assert np.count_nonzero(plain.kept_weights(logits, 1.0, 3, 0.75, 0.0)) == 2      # total is the top-k's: 0.7 / 0.9 >= 0.75
    assert np.count_nonzero(plain.kept_weights(logits, 1.0, 0, 0.75, 0.0)) == 3      # over the vocabulary: 0.7 < 0.75
    assert np.count_nonzero(plain.kept_weights(logits, 1.0, 0, 1.0, 0.3)) == 3       # weights relative to the largest
    assert plain.sample(logits, 0.0, 0, 1.0, 0.0, 0.99) == 0 and plain.sample(logits, 1.0, 1, 1.0, 0.0, 0.99) == 0
    assert plain.sample(logits, 1.0, 0, 1.0, 0.0, 0.49) == 0 and plain.sample(logits, 1.0, 0, 1.0, 0.0, 0.51) == 1
    assert plain.sample(logits, 1.0, 0, 1.0, 0.0, 0.999) == 4
    counts = np.bincount([plain.sample(logits, 1.0, 0, 1.0, 0.0, plain.uniform(7, i)) for i in range(4000)], minlength=5)
    assert np.abs(counts / 4000 - [0.5, 0.2, 0.2, 0.06, 0.04]).max() < 0.03


def test_penalties():
    l = plain.apply_penalties(np.array([2.0, -2.0, 1.0, 1.0]), [0, 1], [2, 2], 2.0, 0.5, 0.25)
    assert l.tolist() == [1.0, -4.0, 0.5 - 0.5 - 0.5, 1.0]


def test_bf16_rounding_helper():
    x = np.array([1.0, 1.00390625, 1.005859375, 3.14159])
    r = plain.to_bf16(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == 1.0078125 and abs(r[3] - 3.140625) < 1e-9
