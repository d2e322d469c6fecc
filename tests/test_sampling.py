"""Host-side sampler of the GPT-2 example loop (src/models/gpt2.zig:866-977) against a line-by-line restatement of
the reference's loops, on seeded inputs."""
import numpy as np

import zignn_b200
from zignn_b200 import api


def reference_top_k(logits, top_k, temperature, r):
    """The reference's control flow with Python scalars (f32 arithmetic through numpy scalars)."""
    f = np.float32
    n = len(logits)
    k = top_k if 0 < top_k < n else n
    inv = f(1.0) / f(temperature) if (temperature > 0 and temperature != 1.0) else f(1.0)
    if k >= n:
        v = [f(x) * inv if inv != 1.0 else f(x) for x in logits]
        mx = max(v)
        e = [f(np.exp(np.float64(x - mx))) for x in v]
        tot = f(0)
        for x in e:
            tot = f(tot + x)
        c = f(0)
        for i, x in enumerate(e):
            c = f(c + x * (f(1.0) / tot))
            if c >= r:
                return i
        return n - 1
    k = min(k, 256)
    vals, idxs = [], []
    mn, pos = None, 0
    for i in range(n):
        v = f(logits[i]) * inv
        if len(vals) < k:
            vals.append(v)
            idxs.append(i)
            if len(vals) == k:
                pos = min(range(k), key=lambda j: (vals[j], j))
                mn = vals[pos]
        elif v > mn:
            vals[pos], idxs[pos] = v, i
            pos = min(range(k), key=lambda j: (vals[j], j))
            mn = vals[pos]
    mx = max(vals)
    e = [f(np.exp(np.float64(x - mx))) for x in vals]
    tot = f(0)
    for x in e:
        tot = f(tot + x)
    c = f(0)
    for j in range(k):
        c = f(c + e[j] * (f(1.0) / tot))
        if c >= r:
            return idxs[j]
    return idxs[k - 1]


def test_top_k_matches_the_reference_loops():
    rng = np.random.default_rng(7)
    for n, k, temp in ((50, 5, 0.8), (1000, 40, 1.0), (3000, 256, 1.3), (3000, 400, 0.7), (64, 1, 1.0)):
        logits = (rng.standard_normal(n) * 3).astype(np.float32)
        for seed in range(6):
            r = np.float32(np.random.default_rng(seed).random(dtype=np.float32))
            got = api.sample_top_k(logits, k, temp, np.random.default_rng(seed))
            assert got == reference_top_k(logits, k, temp, r), (n, k, temp, seed)


def test_full_softmax_fallback_and_input_left_alone():
    rng = np.random.default_rng(9)
    logits = (rng.standard_normal(300) * 2).astype(np.float32)
    keep = logits.copy()
    for k in (0, 300, 1000):
        for seed in range(4):
            r = np.float32(np.random.default_rng(seed).random(dtype=np.float32))
            got = api.sample_top_k(logits, k, 0.9, np.random.default_rng(seed))
            assert got == reference_top_k(logits, k, 0.9, r)
    assert np.array_equal(logits, keep)


def test_top_1_is_argmax_and_frequencies_follow_the_softmax():
    rng = np.random.default_rng(11)
    logits = rng.standard_normal(500).astype(np.float32)
    assert api.sample_top_k(logits, 1, 1.0, rng) == int(np.argmax(logits))
    small = np.array([2.0, 1.0, 0.0, -1.0], dtype=np.float32)
    draws = np.bincount([api.sample_top_k(small, 3, 1.0, rng) for _ in range(4000)], minlength=4)
    p = np.exp(small[:3]) / np.exp(small[:3]).sum()
    assert draws[3] == 0
    assert np.allclose(draws[:3] / 4000.0, p, atol=0.03)
