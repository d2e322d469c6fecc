"""Generates tests/golden/quant_golden.npz from the CPU oracle.

zig-nn is Zig and cannot be run where this repository is built, so these vectors are outputs of the
oracle (oracle/*.cpp), which is itself pinned by the reference's in-file known-answer tests
(tests/test_oracle_kat.py). They freeze the oracle's behaviour: a later change to the oracle or to a
kernel that alters any of these bytes shows up as a test failure.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
sys.path.insert(0, os.path.join(REPO, "oracle"))
import oracle  # noqa: E402

Q4_0, Q4_1, Q8_0 = 2, 3, 8


def main():
    rng = np.random.default_rng(20240611)
    out = {}
    n, k = 40, 160  # 5 blocks per row: exercises the padded quad of the device layout
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((3, k)).astype(np.float32)
    x[1, :32] = 0.0
    out["w_f32"] = w
    out["x"] = x
    for name, t in (("q4_0", Q4_0), ("q4_1", Q4_1), ("q8_0", Q8_0)):
        raw = oracle.quantize(t, w)
        out[name + "_raw"] = raw
        out[name + "_dequant"] = oracle.dequantize(t, raw, n * k).reshape(n, k)
        out[name + "_y_f32"] = oracle.linear(t, raw, x, n, k, act_mode=0)
        out[name + "_y_q8"] = oracle.linear(t, raw, x, n, k, act_mode=1)
    q, scale, s, _ = oracle.quantize_row_q8(x[0])
    out["x0_q8"], out["x0_q8_scale"], out["x0_q8_sum"] = q, scale, s
    # small ops
    v = rng.standard_normal((2, 96)).astype(np.float32) * 3
    g = (1 + 0.1 * rng.standard_normal(96)).astype(np.float32)
    b = (0.1 * rng.standard_normal(96)).astype(np.float32)
    out["ops_x"], out["ops_g"], out["ops_b"] = v, g, b
    out["rms_norm"] = oracle.rms_norm_rows(v, g, 1e-6)
    out["layer_norm"] = oracle.layer_norm_rows(v, g, b)
    out["gelu"] = oracle.gelu(v)
    out["softmax"] = oracle.softmax_forward(v)
    freqs = oracle.rope_freqs(32, 1000000.0)
    out["rope_freqs"] = freqs
    out["rope_pos37"] = oracle.rope(v[0, :32], 37, freqs)
    # single-query attention, gemma flavour: 2 heads, 1 kv head, head_dim 32, window [3, 19)
    qv = rng.standard_normal(64).astype(np.float32)
    kc = rng.standard_normal((19, 32)).astype(np.float32)
    vc = rng.standard_normal((19, 32)).astype(np.float32)
    out["att_q"], out["att_k"], out["att_v"] = qv, kc, vc
    out["att_out"] = oracle.gqa_cached_attention(qv, kc, vc, 3, 19, 2, 32, 32)
    np.savez_compressed(os.path.join(HERE, "quant_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "quant_golden.npz"), os.path.getsize(os.path.join(HERE, "quant_golden.npz")), "bytes")


if __name__ == "__main__":
    main()
