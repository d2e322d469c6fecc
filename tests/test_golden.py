"""Committed golden vectors (tests/golden/quant_golden.npz, made by tests/golden/make_golden.py).
CPU: the oracle still reproduces them bit for bit. GPU: the kernels match them through the C ABI."""
import os

import numpy as np
import pytest

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_golden.npz"))
TYPES = {"q4_0": 2, "q4_1": 3, "q8_0": 8}
N, K = 40, 160


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("name", list(TYPES))
def test_oracle_reproduces_golden(oracle, name):
    t = TYPES[name]
    raw = oracle.quantize(t, G["w_f32"])
    assert np.array_equal(raw, G[name + "_raw"])
    assert np.array_equal(oracle.dequantize(t, raw, N * K).reshape(N, K), G[name + "_dequant"])
    assert np.array_equal(oracle.linear(t, raw, G["x"], N, K, act_mode=0), G[name + "_y_f32"])
    assert np.array_equal(oracle.linear(t, raw, G["x"], N, K, act_mode=1), G[name + "_y_q8"])


def test_oracle_small_ops_reproduce_golden(oracle):
    v, g, b = G["ops_x"], G["ops_g"], G["ops_b"]
    assert np.array_equal(oracle.rms_norm_rows(v, g, 1e-6), G["rms_norm"])
    assert np.array_equal(oracle.layer_norm_rows(v, g, b), G["layer_norm"])
    assert np.array_equal(oracle.gelu(v), G["gelu"])
    assert np.array_equal(oracle.softmax_forward(v), G["softmax"])
    assert np.array_equal(oracle.rope(v[0, :32], 37, G["rope_freqs"]), G["rope_pos37"])
    q, scale, s, _ = oracle.quantize_row_q8(G["x"][0])
    assert np.array_equal(q, G["x0_q8"]) and np.array_equal(scale, G["x0_q8_scale"]) and np.array_equal(s, G["x0_q8_sum"])
    out = oracle.gqa_cached_attention(G["att_q"], G["att_k"], G["att_v"], 3, 19, 2, 32, 32)
    assert np.array_equal(out, G["att_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(TYPES))
def test_kernels_match_golden(zq, name):
    import torch
    qw = zq.QuantWeight(G[name + "_raw"], TYPES[name], N, K)
    assert np.array_equal(qw.dequantize().cpu().numpy(), G[name + "_dequant"])      # bit-exact
    x = torch.from_numpy(G["x"]).cuda()
    y32 = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32).cpu().numpy()
    assert rel_l2(y32, G[name + "_y_f32"]) <= 2e-6                                    # bar: 1e-3
    yq8 = zq.quant_matmul_no_grad(x, qw, zq.ACT_Q8).cpu().numpy()
    assert np.array_equal(yq8, G[name + "_y_q8"])                                     # bit-exact


@pytest.mark.gpu
def test_small_op_kernels_match_golden(zq):
    import torch
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    v, g, b = G["ops_x"], G["ops_g"], G["ops_b"]
    assert np.array_equal(zq.rms_norm(t(v), t(g), 1e-6).cpu().numpy(), G["rms_norm"])
    assert rel_l2(zq.layer_norm(t(v), t(g), t(b), 1e-5).cpu().numpy(), G["layer_norm"]) <= 2e-6
    assert np.array_equal(zq.gelu(t(v)).cpu().numpy(), G["gelu"])
    assert rel_l2(zq.softmax(t(v)).cpu().numpy(), G["softmax"]) <= 1e-5
    assert np.array_equal(zq.rope(t(v[0, :32].copy()), t(G["rope_freqs"]), 1, 37).cpu().numpy(), G["rope_pos37"])
    out = zq.attention_decode(t(G["att_q"]), t(G["att_k"]), t(G["att_v"]), 2, 1, 32, 3, 19).cpu().numpy()
    assert np.array_equal(out, G["att_out"])
