"""The small f32 ops between the linears against the CPU oracle (tolerances: these are f32
reductions evaluated in a different order, so a few ulp)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-6


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


RNG = np.random.default_rng(11)


@pytest.mark.parametrize("rows,dim", [(1, 1152), (5, 768), (3, 33), (2, 4)])
def test_rms_norm(zq, oracle, rows, dim):
    x = RNG.standard_normal((rows, dim)).astype(np.float32)
    w = (1 + 0.1 * RNG.standard_normal(dim)).astype(np.float32)
    assert np.array_equal(zq.rms_norm(t(x), t(w), 1e-6).cpu().numpy(), oracle.rms_norm_rows(x, w, 1e-6))
    res = RNG.standard_normal((rows, dim)).astype(np.float32)
    got = zq.rms_norm_residual(t(x), t(w), t(res), 1e-6).cpu().numpy()
    assert np.array_equal(got, res + oracle.rms_norm_rows(x, w, 1e-6))


def test_rms_norm_known_answer(zq):  # src/models/gemma3.zig:1210-1223
    x = np.array([[1, 2, 3, 4]], np.float32)
    out = zq.rms_norm(t(x), t(np.ones(4)), 1e-6).cpu().numpy()[0]
    np.testing.assert_allclose(out, x[0] / np.sqrt(7.5 + 1e-6), atol=1e-4)


def test_rms_norm_in_place_per_head(zq, oracle):
    x = RNG.standard_normal((4, 256)).astype(np.float32)
    w = (1 + 0.1 * RNG.standard_normal(256)).astype(np.float32)
    got = zq.rms_norm_in_place(t(x), t(w), 256, 1e-6).cpu().numpy()
    want = np.stack([oracle.rms_norm_in_place(x[h], w, 1e-6) for h in range(4)])
    assert np.array_equal(got, want)


@pytest.mark.parametrize("pos", [0, 1, 17, 2047])
def test_rope(zq, oracle, pos):
    freqs = zq.rope_freqs(256, 1000000.0)
    assert np.array_equal(freqs, oracle.rope_freqs(256, 1000000.0))
    x = RNG.standard_normal((4, 256)).astype(np.float32)
    got = zq.rope(t(x), t(freqs), 4, pos).cpu().numpy()
    want = np.stack([oracle.rope(x[h], pos, freqs) for h in range(4)])
    if pos == 0:  # src/models/gemma3.zig:1225-1233
        assert np.array_equal(got, x)
    assert np.array_equal(got, want)


def test_gelu_and_gelu_mul(zq, oracle):
    x = (3 * RNG.standard_normal(6912)).astype(np.float32)
    up = RNG.standard_normal(6912).astype(np.float32)
    assert np.array_equal(zq.gelu(t(x)).cpu().numpy(), oracle.gelu(x))
    assert np.array_equal(zq.gelu_mul(t(x), t(up)).cpu().numpy(), oracle.gelu(x) * up)
    k = zq.gelu(t(np.array([0, 1, -1, 2, -2]))).cpu().numpy()  # src/models/gpt2.zig:1015-1028
    assert abs(k[0]) < 1e-6 and abs(k[1] - 0.8412) < 0.01 and abs(k[2] + 0.1588) < 0.01 and k[3] > 0 and abs(k[4]) < 0.1


@pytest.mark.parametrize("rows,cols", [(1, 3), (7, 1000), (2, 2048), (3, 1)])
def test_softmax(zq, oracle, rows, cols):
    x = (4 * RNG.standard_normal((rows, cols))).astype(np.float32)
    want = oracle.softmax_forward(x)  # sums its exponentials one by one; 2048 terms drift a few ulp
    assert rel_l2(zq.softmax(t(x)).cpu().numpy(), want) <= 1e-5
    assert rel_l2(zq.softmax_(t(x)).cpu().numpy(), want) <= 1e-5
    np.testing.assert_allclose(zq.softmax(t(x)).sum(dim=-1).cpu().numpy(), np.ones(rows), atol=1e-5)


@pytest.mark.parametrize("rows,cols", [(1, 768), (4, 100), (2, 4)])
def test_layer_norm(zq, oracle, rows, cols):
    x = (2 + 3 * RNG.standard_normal((rows, cols))).astype(np.float32)
    g = (1 + 0.1 * RNG.standard_normal(cols)).astype(np.float32)
    b = (0.1 * RNG.standard_normal(cols)).astype(np.float32)
    got = zq.layer_norm(t(x), t(g), t(b), 1e-5).cpu().numpy()
    assert rel_l2(got, oracle.layer_norm_rows(x, g, b)) <= TOL          # gpt2.zig two-pass form
    assert rel_l2(got, oracle.layer_norm_forward(x, g, b, 1e-5)) <= 1e-5  # runtime_kernels one-pass form


def test_layer_norm_known_answer(zq):  # src/models/gpt2.zig:996-1013
    out = zq.layer_norm(t(np.array([[1, 2, 3, 4]])), t(np.ones(4)), t(np.zeros(4)), 1e-5).cpu().numpy()[0]
    assert abs(out.sum()) < 1e-5 and out[0] < 0 < out[3]


def test_broadcast_gather_scale(zq):
    a = RNG.standard_normal((5, 64)).astype(np.float32)
    b = RNG.standard_normal(64).astype(np.float32)
    assert np.array_equal(zq.add_broadcast(t(a), t(b)).cpu().numpy(), a + b)
    assert np.array_equal(zq.mul_broadcast(t(a), t(b)).cpu().numpy(), a * b)
    table = RNG.standard_normal((100, 48)).astype(np.float32)
    idx = torch.tensor([3, 99, 0, 3])
    assert np.array_equal(zq.gather(t(table), idx).cpu().numpy(), table[[3, 99, 0, 3]])
    assert np.array_equal(zq.scale(t(a), 0.5).cpu().numpy(), a * np.float32(0.5))


@pytest.mark.parametrize("n_head,n_kv,hd,kv_start,kv_end", [
    (12, 12, 64, 0, 1), (12, 12, 64, 0, 160), (4, 1, 256, 0, 37), (4, 1, 256, 100, 612), (4, 1, 256, 0, 2048),
    (2, 1, 32, 3, 11), (3, 1, 40, 0, 21)])
def test_attention_decode(zq, oracle, n_head, n_kv, hd, kv_start, kv_end):
    kv_dim = n_kv * hd
    ctx = kv_end
    q = RNG.standard_normal(n_head * hd).astype(np.float32)
    kc = RNG.standard_normal((ctx, kv_dim)).astype(np.float32)
    vc = RNG.standard_normal((ctx, kv_dim)).astype(np.float32)
    if n_kv == n_head:
        assert kv_start == 0
        got = zq.attention_decode(t(q), t(kc), t(vc), n_head, n_kv, hd, kv_start, kv_end,
                                  flags=zq.ATTN_GPT2_SOFTMAX).cpu().numpy()
        want = oracle.cached_attention(q, kc, vc, kv_end, n_head, hd)
    else:
        got = zq.attention_decode(t(q), t(kc), t(vc), n_head, n_kv, hd, kv_start, kv_end).cpu().numpy()
        want = oracle.gqa_cached_attention(q, kc, vc, kv_start, kv_end, n_head, hd, kv_dim)
    assert np.array_equal(got, want), rel_l2(got, want)


def test_attention_single_position_returns_v(zq):  # src/models/gpt2.zig:1059-1079
    q = np.array([1, 0], np.float32)
    out = zq.attention_decode(t(q), t(np.array([[1, 0]])), t(np.array([[1, 2]])), 1, 1, 2, 0, 1).cpu().numpy()
    np.testing.assert_allclose(out, [1, 2], atol=1e-6)


def test_write_kv_cache(zq):
    kc, vc = torch.zeros(8, 256, device="cuda"), torch.zeros(8, 256, device="cuda")
    k, v = t(RNG.standard_normal(256)), t(RNG.standard_normal(256))
    zq.write_kv_cache(k, v, kc, vc, 5)
    assert torch.equal(kc[5], k) and torch.equal(vc[5], v) and kc[4].abs().sum() == 0


def test_dequant_rows_scaled(zq, oracle):
    """Embedding lookup: dequant_row then * sqrt(EMBED) (src/models/gemma3.zig:800-803)."""
    from zignn_b200 import ggml
    n, k = 500, 1152
    w = (RNG.standard_normal((n, k)) * 0.02).astype(np.float32)
    for qtype in (ggml.Q8_0, ggml.Q4_0, ggml.Q4_1):
        raw = oracle.quantize(qtype, w)
        qw = zq.QuantWeight(raw, qtype, n, k)
        ids = torch.tensor([499, 0, 17])
        s = np.sqrt(np.float32(k))
        got = qw.dequant_rows_scaled(ids, s).cpu().numpy()
        full = oracle.dequantize(qtype, raw, n * k).reshape(n, k)
        want = full[[499, 0, 17]] * np.float32(s)
        assert np.array_equal(got, want)
