"""The CPU oracle against the reference's own known-answer tests (zig-nn in-file `test` blocks).
Each test names the Zig test it restates. These pin the oracle at block level."""
import struct

import numpy as np
import pytest

Q4_0, Q4_1, Q8_0, F32, F16 = 2, 3, 8, 0, 1


def f16(v):
    return np.array([v], dtype=np.float16).view(np.uint8)


def q4_0_block(scale, fill, first=None):
    b = np.full(18, fill, dtype=np.uint8)
    b[0:2] = f16(scale)
    if first:
        for i, v in enumerate(first):
            b[2 + i] = v
    return b


def q4_1_block(scale, mn, fill):
    b = np.full(20, fill, dtype=np.uint8)
    b[0:2] = f16(scale)
    b[2:4] = f16(mn)
    return b


def q8_0_block(scale, fill, first=None):
    b = np.full(34, fill & 0xFF, dtype=np.uint8)
    b[0:2] = f16(scale)
    if first:
        for i, v in enumerate(first):
            b[2 + i] = v & 0xFF
    return b


# ---- src/gguf/dequant.zig:426-694 ----

def test_dequantize_f32(oracle):  # "dequantize F32"
    src = np.array([1.0, -2.5, 3.14], dtype=np.float32).view(np.uint8)
    np.testing.assert_allclose(oracle.dequantize(F32, src, 3), [1.0, -2.5, 3.14], atol=1e-6)


def test_dequantize_f16(oracle):  # "dequantize F16"
    src = np.array([1.0, -0.5], dtype=np.float16).view(np.uint8)
    np.testing.assert_allclose(oracle.dequantize(F16, src, 2), [1.0, -0.5], atol=1e-3)


def test_dequantize_q4_0_basic(oracle):  # "dequantize Q4_0 basic"
    out = oracle.dequantize(Q4_0, q4_0_block(1.0, 0x88), 32)
    np.testing.assert_allclose(out, np.zeros(32), atol=1e-6)


def test_dequantize_q4_0_nonzero(oracle):  # "dequantize Q4_0 non-zero"
    out = oracle.dequantize(Q4_0, q4_0_block(2.0, 0x88, [0x0F]), 32)
    assert abs(out[0] - 14.0) < 0.01 and abs(out[16] + 16.0) < 0.01


def test_dequantize_q8_0_basic(oracle):  # "dequantize Q8_0 basic"
    out = oracle.dequantize(Q8_0, q8_0_block(0.5, 0, [4, -3]), 32)
    assert abs(out[0] - 2.0) < 0.01 and abs(out[1] + 1.5) < 0.01 and abs(out[2]) < 1e-6


def test_dot_q4_0_f32_basic(oracle):  # "dotQ4_0_f32 basic"
    assert abs(oracle.dot_f32(Q4_0, q4_0_block(1.0, 0x99), np.ones(32)) - 32.0) < 0.01


def test_dot_q4_0_f32_matches_dequantize(oracle):  # "dotQ4_0_f32 matches dequantize"
    blk = q4_0_block(2.0, 0x88, [0x0F, 0x17])
    expected = np.float32(0)
    for v in oracle.dequantize(Q4_0, blk, 32):
        expected = np.float32(expected + v)
    assert abs(oracle.dot_f32(Q4_0, blk, np.ones(32)) - expected) < 0.01


def test_matmul_q4_0_f32_basic(oracle):  # "matmulQ4_0_f32 basic"
    w = np.concatenate([q4_0_block(1.0, 0x99), q4_0_block(0.5, 0xAA)])
    y = oracle.matmul_f32(Q4_0, w, np.ones(32), 2, 32)
    np.testing.assert_allclose(y, [32.0, 32.0], atol=0.01)


def test_dequantize_q4_1_basic(oracle):  # "dequantize Q4_1 basic"
    out = oracle.dequantize(Q4_1, q4_1_block(1.0, 0.5, 0x00), 32)
    np.testing.assert_allclose(out, np.full(32, 0.5), atol=1e-3)


def test_dot_q4_1_f32_basic(oracle):  # "dotQ4_1_f32 basic"
    assert abs(oracle.dot_f32(Q4_1, q4_1_block(1.0, 0.0, 0x11), np.ones(32)) - 32.0) < 0.1


def test_dot_q4_1_f32_with_min(oracle):  # "dotQ4_1_f32 with min"
    assert abs(oracle.dot_f32(Q4_1, q4_1_block(2.0, 1.0, 0x00), np.ones(32)) - 32.0) < 0.1


def test_dot_q8_0_f32_basic(oracle):  # "dotQ8_0_f32 basic"
    assert abs(oracle.dot_f32(Q8_0, q8_0_block(1.0, 2), np.ones(32)) - 64.0) < 0.01


def test_dot_q8_0_f32_matches_dequantize(oracle):  # "dotQ8_0_f32 matches dequantize"
    blk = q8_0_block(0.5, 0, [4, -3])
    expected = float(np.sum(oracle.dequantize(Q8_0, blk, 32), dtype=np.float32))
    assert abs(oracle.dot_f32(Q8_0, blk, np.ones(32)) - expected) < 0.01


def test_matmul_q8_0_f32_basic(oracle):  # "matmulQ8_0_f32 basic"
    w = np.concatenate([q8_0_block(1.0, 1), q8_0_block(0.5, 2)])
    np.testing.assert_allclose(oracle.matmul_f32(Q8_0, w, np.ones(32), 2, 32), [32.0, 32.0], atol=0.01)


def test_tensor_bytes(oracle):  # "tensorBytes calculation"
    assert oracle.tensor_bytes(F32, 32) == 128
    assert oracle.tensor_bytes(F16, 32) == 64
    assert oracle.tensor_bytes(Q4_0, 32) == 18
    assert oracle.tensor_bytes(Q4_0, 64) == 36
    assert oracle.tensor_bytes(Q4_1, 32) == 20
    assert oracle.tensor_bytes(Q8_0, 32) == 34


def test_unsupported_type(oracle):  # dequantize(): else => error.UnsupportedQuantType
    with pytest.raises(ValueError):
        oracle.dequantize(6, np.zeros(22, np.uint8), 32)


# ---- src/gguf/simd_dot.zig:158-326 ----

def test_quantize_row_q8_basic(oracle):  # "quantizeRowQ8 basic"
    x = np.arange(32, dtype=np.float32) - 16.0
    q, scale, s, _ = oracle.quantize_row_q8(x)
    assert 0 < scale[0] < 0.2
    assert q[0, 16] == 0 and q[0, 0] == -127


def test_quantize_row_q8_zero(oracle):  # "quantizeRowQ8 zero input"
    q, scale, s, _ = oracle.quantize_row_q8(np.zeros(32, np.float32))
    assert (q == 0).all() and s[0] == 0 and scale[0] == 1.0


def test_dot_q4_0_q8_matches_f32(oracle):  # "dotQ4_0_q8 matches dotQ4_0_f32"
    blk = q4_0_block(2.0, 0x99, [0x0F, 0x17])
    x = (np.arange(32, dtype=np.float32) * np.float32(0.1) - np.float32(1.5)).astype(np.float32)
    expected = oracle.dot_f32(Q4_0, blk, x)
    _, _, _, blocks = oracle.quantize_row_q8(x)
    assert abs(oracle.dot_q8(Q4_0, blk, blocks) - expected) <= abs(expected) * 0.05 + 0.5


def test_dot_q4_0_q8_unit(oracle):  # "dotQ4_0_q8 unit values"
    blk = q4_0_block(1.0, 0x99)
    x = np.ones(32, np.float32)
    _, _, _, blocks = oracle.quantize_row_q8(x)
    assert abs(oracle.dot_q8(Q4_0, blk, blocks) - oracle.dot_f32(Q4_0, blk, x)) <= 0.5


def test_dot_q4_1_q8_matches_f32(oracle):  # "dotQ4_1_q8 matches dotQ4_1_f32"
    blk = q4_1_block(2.0, 1.0, 0x33)
    x = (np.arange(32, dtype=np.float32) * np.float32(0.2) - np.float32(3.0)).astype(np.float32)
    expected = oracle.dot_f32(Q4_1, blk, x)
    _, _, _, blocks = oracle.quantize_row_q8(x)
    assert abs(oracle.dot_q8(Q4_1, blk, blocks) - expected) <= abs(expected) * 0.05 + 1.0


def test_dot_q8_0_q8_matches_f32(oracle):  # "dotQ8_0_q8 matches dotQ8_0_f32"
    blk = q8_0_block(0.5, 1, [4, -3, 10])
    x = (np.arange(32, dtype=np.float32) * np.float32(0.3) - np.float32(4.0)).astype(np.float32)
    expected = oracle.dot_f32(Q8_0, blk, x)
    _, _, _, blocks = oracle.quantize_row_q8(x)
    assert abs(oracle.dot_q8(Q8_0, blk, blocks) - expected) <= abs(expected) * 0.05 + 0.5


def test_dot_q8_0_q8_unit(oracle):  # "dotQ8_0_q8 unit values"
    blk = q8_0_block(1.0, 2)
    x = np.ones(32, np.float32)
    _, _, _, blocks = oracle.quantize_row_q8(x)
    assert abs(oracle.dot_q8(Q8_0, blk, blocks) - 64.0) <= 1.0


def test_multi_block_dot_q4_0_q8(oracle):  # "multi-block dotQ4_0_q8"
    w = np.concatenate([q4_0_block(1.0, 0x99), q4_0_block(0.5, 0xAA)])
    x = np.ones(64, np.float32)
    _, _, _, blocks = oracle.quantize_row_q8(x)
    assert abs(oracle.dot_q8(Q4_0, w, blocks) - oracle.dot_f32(Q4_0, w, x)) <= 1.0
    assert abs(oracle.dot_f32(Q4_0, w, x) - 64.0) < 0.01


def test_thread_pool_limit(oracle):  # MAX_Q8_BLOCKS = 256 -> in_dim <= 8192 (thread_pool.zig:21)
    w = oracle.quantize(Q4_0, np.zeros((1, 8224), np.float32))
    with pytest.raises(ValueError):
        oracle.matmul_q8(Q4_0, w, np.zeros(8224, np.float32), 1, 8224)
    oracle.matmul_q8(Q4_0, w, np.zeros(8224, np.float32), 1, 8224, allow_long=True)


# ---- src/models/gpt2.zig:996-1084 ----

def test_layer_norm_basic(oracle):  # "layerNorm basic"
    out = oracle.layer_norm_rows(np.array([[1, 2, 3, 4]], np.float32), np.ones(4), np.zeros(4))[0]
    assert abs(out.sum()) < 1e-5 and out[0] < 0 and out[3] > 0


def test_gelu_basic(oracle):  # "gelu basic" and gemma3 "geluInPlace basic"
    x = oracle.gelu(np.array([0, 1, -1, 2, -2], np.float32))
    assert abs(x[0]) < 1e-5 and abs(x[1] - 0.8412) < 0.01 and abs(x[2] + 0.1588) < 0.01
    assert x[3] > 0 and abs(x[4]) < 0.1


def test_softmax_basic(oracle):  # "softmax basic"
    for fn in (oracle.softmax_gpt2, oracle.softmax_gemma):
        x = fn(np.array([1, 2, 3], np.float32))
        assert abs(x.sum() - 1.0) < 1e-5 and x[0] < x[1] < x[2]


def test_linear_forward_basic(oracle):  # "linearForward basic": f32 weight [3,2], bias
    w = np.array([1, 0, 0, 1, 0, 0], np.float32)
    y = oracle.matmul_f32(F32, w.view(np.uint8), np.array([1, 2], np.float32), 3, 2)
    np.testing.assert_allclose(y + np.array([10, 20, 30], np.float32), [11, 22, 30], atol=1e-5)


def test_causal_self_attention_single_head(oracle):  # "causalSelfAttention single head"
    qkv = np.array([1, 0, 1, 0, 1, 2, 0, 1, 0, 1, 3, 4], np.float32)
    out = oracle.causal_self_attention(qkv, 2, 1, 2)
    np.testing.assert_allclose(out[0], [1.0, 2.0], atol=1e-4)
    # pos 1 is a convex combination of v0 and v1
    assert 1.0 < out[1, 0] < 3.0 and 2.0 < out[1, 1] < 4.0


def test_argmax(oracle):  # "argmax"
    assert oracle.argmax(np.array([-1, 3, 2, 5, 0], np.float32)) == 3
    assert oracle.argmax(np.array([1, 7, 7, 7], np.float32)) == 1  # first maximum wins


# ---- src/models/gemma3.zig:1210-1252 ----

def test_rms_norm_basic(oracle):  # "rmsNorm basic"
    x = np.array([[1, 2, 3, 4]], np.float32)
    out = oracle.rms_norm_rows(x, np.ones(4), 1e-6)[0]
    np.testing.assert_allclose(out, x[0] / np.sqrt(7.5 + 1e-6), atol=1e-4)


def test_rope_pos0_identity(oracle):  # "applyRoPE basic"
    freqs = oracle.rope_freqs(4, 10000.0)
    out = oracle.rope(np.array([1, 2, 3, 4], np.float32), 0, freqs)
    np.testing.assert_allclose(out, [1, 2, 3, 4], atol=1e-5)


def test_is_global_layer(oracle):  # "isGlobalLayer": layers 5, 11, 17, 23 of 26
    glob = [l for l in range(26) if l % 6 == 5]
    assert glob == [5, 11, 17, 23]


# ---- src/runtime_kernels.zig:325-399 and src/diff/mps_runtime_test.zig:694-752 ----

def test_runtime_softmax_rows(oracle):
    x = np.array([[1, 2, 3], [0, 0, 0]], np.float32)
    out = oracle.softmax_forward(x)
    np.testing.assert_allclose(out.sum(axis=1), [1, 1], atol=1e-6)
    np.testing.assert_allclose(out[1], [1 / 3] * 3, atol=1e-6)


def test_quant_matmul_q8_0_forward(oracle):  # "quantMatmulNoGrad Q8_0 forward": M=2, IN=32, OUT=4
    M, IN, OUT = 2, 32, 4
    i = np.arange(OUT * IN, dtype=np.float32)
    w = (np.float32(0.01) * ((i - np.float32(50.0)) * (i + np.float32(3.0))) * np.float32(0.001)).astype(np.float32)
    raw = oracle.quantize(Q8_0, w)
    wd = oracle.dequantize(Q8_0, raw, OUT * IN).reshape(OUT, IN)
    x = (np.float32(0.05) * (np.arange(M * IN, dtype=np.float32) - np.float32(15.0))).reshape(M, IN)
    y = oracle.linear(Q8_0, raw, x, OUT, IN, act_mode=0)
    np.testing.assert_allclose(y, x @ wd.T, atol=1e-3)


@pytest.mark.parametrize("qtype", [2, 3, 8])
def test_transposed_product_is_the_decoded_matrix_times_the_gradient(oracle, qtype):
    """nn_training_kernels.metal:1149-1242 decodes W[j][k] and sums grad_out[m][j] * W[j][k] over j; with
    one weight row the sum has one term, and with many rows it stays within f32 rounding of the f64 product."""
    rng = np.random.default_rng(qtype)
    w = (rng.standard_normal((40, 64)) * 0.05).astype(np.float32)
    raw = oracle.quantize(qtype, w.reshape(-1))
    dec = oracle.dequantize(qtype, raw, w.size).reshape(40, 64)
    g = rng.standard_normal((3, 40)).astype(np.float32)
    got = oracle.matmul_transposed(qtype, raw, g, 40, 64)
    ref = g.astype(np.float64) @ dec.astype(np.float64)
    assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()
    row_bytes = raw.size // 40
    one = oracle.matmul_transposed(qtype, raw[:row_bytes], g[:, :1], 1, 64)
    assert np.array_equal(one, g[:, :1] * dec[:1])  # a single f32 product per element, added to zero
    acc = oracle.matmul_transposed(qtype, raw, g, 40, 64, grad_x=np.full((3, 64), 2.0, np.float32))
    assert np.array_equal(acc, np.float32(2.0) + got)
    with pytest.raises(ValueError):
        oracle.matmul_transposed(0, raw, g, 40, 64)
