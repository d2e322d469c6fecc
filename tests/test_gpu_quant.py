"""Parity of the CUDA quantised linears with the CPU oracle, through the C ABI.

Bars: dequantised weights bit-exact; Q8-activation outputs bit-exact; f32-activation outputs
rel-L2 <= 1e-3 (the stated bar) — and <= 2e-6 as an implementation guard, since both sides
compute in f32."""
import numpy as np
import pytest
import torch

from zignn_b200 import ggml

pytestmark = pytest.mark.gpu

TYPES = [ggml.Q4_0, ggml.Q4_1, ggml.Q8_0]
REL_L2_BAR = 1e-3
REL_L2_GUARD = 2e-6


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def make_weight(oracle, qtype, n, k, seed=42, std=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * std).astype(np.float32)
    return oracle.quantize(qtype, w)


def make_x(m, k, seed=43):
    return np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("n,k", [(64, 256), (33, 96), (1, 32), (5, 1152)])
def test_dequant_bit_exact_and_raw_round_trip(zq, oracle, qtype, n, k):
    raw = make_weight(oracle, qtype, n, k)
    qw = zq.QuantWeight(raw, qtype, n, k)
    got = qw.dequantize().cpu().numpy().reshape(-1)
    want = oracle.dequantize(qtype, raw, n * k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(qw.raw_bytes().cpu().numpy(), raw)


@pytest.mark.parametrize("qtype", TYPES)
def test_weight_from_device_bytes(zq, oracle, qtype):
    raw = make_weight(oracle, qtype, 48, 128)
    qw = zq.QuantWeight(torch.from_numpy(raw).cuda(), qtype, 48, 128)
    want = oracle.dequantize(qtype, raw, 48 * 128)
    assert np.array_equal(qw.dequantize().cpu().numpy().reshape(-1), want)


def test_reference_known_answers_through_the_gpu(zq):
    """The block-level known answers of src/gguf/dequant.zig:449-685 run on the device."""
    def f16b(v):
        return np.array([v], np.float16).view(np.uint8)
    ones = torch.ones(1, 32, device="cuda")
    # q4_0: scale 1, nibbles 9 -> 32.0 ; scale 0.5, nibbles 10 -> 32.0
    w = np.concatenate([f16b(1.0), np.full(16, 0x99, np.uint8), f16b(0.5), np.full(16, 0xAA, np.uint8)])
    qw = zq.QuantWeight(w, ggml.Q4_0, 2, 32)
    np.testing.assert_allclose(zq.quant_matmul_no_grad(ones, qw).cpu().numpy()[0], [32.0, 32.0], atol=0.01)
    # q4_0 decode: scale 2, byte0 = 0x0F -> elem0 = 14, elem16 = -16
    w = np.concatenate([f16b(2.0), np.array([0x0F], np.uint8), np.full(15, 0x88, np.uint8)])
    d = zq.QuantWeight(w, ggml.Q4_0, 1, 32).dequantize().cpu().numpy()[0]
    assert d[0] == 14.0 and d[16] == -16.0 and d[1] == 0.0
    # q4_1: scale 2, min 1, nibbles 0 -> every value 1.0, dot with ones = 32
    w = np.concatenate([f16b(2.0), f16b(1.0), np.zeros(16, np.uint8)])
    qw = zq.QuantWeight(w, ggml.Q4_1, 1, 32)
    assert np.all(qw.dequantize().cpu().numpy() == 1.0)
    assert abs(zq.quant_matmul_no_grad(ones, qw).item() - 32.0) < 0.1
    # q8_0: scale 0.5, q = {4, -3, 0...} -> {2.0, -1.5, 0}; q = 2 everywhere, scale 1 -> 64
    w = np.concatenate([f16b(0.5), np.array([4, 0xFD], np.uint8), np.zeros(30, np.uint8)])
    d = zq.QuantWeight(w, ggml.Q8_0, 1, 32).dequantize().cpu().numpy()[0]
    assert d[0] == 2.0 and d[1] == -1.5 and d[2] == 0.0
    w = np.concatenate([f16b(1.0), np.full(32, 2, np.uint8)])
    assert abs(zq.quant_matmul_no_grad(ones, zq.QuantWeight(w, ggml.Q8_0, 1, 32)).item() - 64.0) < 0.01


SHAPES = [(2304, 768), (768, 3072), (6912, 1152), (1152, 6912), (100, 32), (7, 64), (1, 32), (257, 1152),
          (130, 2048), (96, 160)]


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("n,k", SHAPES)
def test_gemv_f32_activations(zq, oracle, qtype, n, k):
    raw = make_weight(oracle, qtype, n, k)
    qw = zq.QuantWeight(raw, qtype, n, k)
    x = make_x(1, k)
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_F32).cpu().numpy()
    want = oracle.linear(qtype, raw, x, n, k, act_mode=0, n_threads=4)
    err = rel_l2(got, want)
    assert err <= REL_L2_BAR
    assert err <= REL_L2_GUARD, err


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("m", [2, 4, 16])
def test_matmul_small_batches_f32(zq, oracle, qtype, m):
    n, k = 520, 768
    raw = make_weight(oracle, qtype, n, k)
    qw = zq.QuantWeight(raw, qtype, n, k)
    x = make_x(m, k)
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_F32).cpu().numpy()
    want = oracle.linear(qtype, raw, x, n, k, act_mode=0, n_threads=4)
    assert got.shape == (m, n)
    assert rel_l2(got, want) <= REL_L2_GUARD


REL_L2_GEMM_GUARD = 6e-4  # fp16 operands (weights and activations each rounded once, <= 2^-12 relative)


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("m,n,k", [(64, 520, 768), (128, 256, 1152), (200, 1000, 96), (513, 136, 2048),
                                   (1030, 6420, 96)])
def test_matmul_many_rows_tensor_core_gemm(zq, oracle, qtype, m, n, k):
    """More than 48 activation rows take the GEMM: ragged M and N tiles, K that is not a multiple of
    the 128-wide stage, and the full epilogue. The last shape has enough tiles for the form with two
    128-row weight tiles per CTA (ragged in both directions: the last pair holds 20 rows)."""
    raw = make_weight(oracle, qtype, n, k)
    qw = zq.QuantWeight(raw, qtype, n, k)
    x = make_x(m, k)
    x[1] *= 1000.0    # rows of very different magnitude: the per-row scale must cope
    x[2] *= 1e-4
    x[3] = 0.0
    rng = np.random.default_rng(9)
    bias = rng.standard_normal(n).astype(np.float32) * 0.1
    res = rng.standard_normal((m, n)).astype(np.float32) * 0.1
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_F32).cpu().numpy()
    want = oracle.linear(qtype, raw, x, n, k, act_mode=0, n_threads=8)
    assert got.shape == (m, n)
    for r in (0, 1, 2, m - 1):
        assert rel_l2(got[r], want[r]) <= REL_L2_BAR
        assert rel_l2(got[r], want[r]) <= REL_L2_GEMM_GUARD, (r, rel_l2(got[r], want[r]))
    assert np.all(got[3] == 0.0)
    assert rel_l2(got, want) <= REL_L2_GEMM_GUARD
    got2 = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_F32, bias=torch.from_numpy(bias).cuda(),
                                   residual=torch.from_numpy(res).cuda()).cpu().numpy()
    assert rel_l2(got2, want + bias + res) <= REL_L2_GEMM_GUARD


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("m", [1, 5, 33])
def test_f16_activation_mode_any_row_count(zq, oracle, qtype, m):
    """ZQ_ACT_F16 sends any number of rows through the tensor-core GEMM (fp16 operands)."""
    n, k = 300, 1152
    raw = make_weight(oracle, qtype, n, k)
    qw = zq.QuantWeight(raw, qtype, n, k)
    x = make_x(m, k)
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_F16).cpu().numpy()
    want = oracle.linear(qtype, raw, x, n, k, act_mode=0, n_threads=4)
    assert got.shape == (m, n)
    assert rel_l2(got, want) <= REL_L2_GEMM_GUARD


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("n,k", SHAPES)
def test_gemv_q8_activations_bit_exact(zq, oracle, qtype, n, k):
    raw = make_weight(oracle, qtype, n, k)
    qw = zq.QuantWeight(raw, qtype, n, k)
    x = make_x(1, k)
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_Q8).cpu().numpy()
    want = oracle.linear(qtype, raw, x, n, k, act_mode=1, n_threads=4)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), rel_l2(got, want)


@pytest.mark.parametrize("m", [3, 16])
def test_matmul_small_batches_q8_bit_exact(zq, oracle, m):
    n, k = 300, 1152
    raw = make_weight(oracle, ggml.Q4_1, n, k)
    qw = zq.QuantWeight(raw, ggml.Q4_1, n, k)
    x = make_x(m, k)
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_Q8).cpu().numpy()
    want = oracle.linear(ggml.Q4_1, raw, x, n, k, act_mode=1, n_threads=4)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("m,n,k", [(17, 300, 1152), (64, 520, 768), (100, 129, 96), (200, 1000, 6912)])
def test_matmul_many_rows_q8_bit_exact(zq, oracle, qtype, m, n, k):
    """More than 16 Q8-quantised activation rows take the exact int8 tensor-core GEMM; every output must
    equal the CPU path bit for bit (ragged M / N tiles, K not a multiple of 128, full epilogue)."""
    raw = make_weight(oracle, qtype, n, k)
    qw = zq.QuantWeight(raw, qtype, n, k)
    x = make_x(m, k)
    x[1] *= 100.0
    x[2, :64] = 0.0
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_Q8).cpu().numpy()
    want = oracle.linear(qtype, raw, x, n, k, act_mode=1, n_threads=8)
    assert got.shape == (m, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), rel_l2(got, want)
    rng = np.random.default_rng(3)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((m, n)).astype(np.float32)
    got2 = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_Q8, bias=torch.from_numpy(bias).cuda(),
                                   residual=torch.from_numpy(res).cuda()).cpu().numpy()
    assert np.array_equal(got2, res + (want + bias))


def test_quantize_rows_q8_bit_exact(zq, oracle):
    x = make_x(3, 1152)
    x[0, :32] = 0.0                                  # all-zero block: scale 1, q 0
    x[1, 32:64] = np.arange(32, dtype=np.float32) - 16.0  # the reference's ramp
    x[2, 5] = 1e-30
    q, scale, s = zq.quantize_rows_q8(torch.from_numpy(x).cuda())
    for m in range(3):
        oq, oscale, osum, _ = oracle.quantize_row_q8(x[m])
        assert np.array_equal(q[m].cpu().numpy().reshape(-1, 32), oq)
        assert np.array_equal(scale[m].cpu().numpy().view(np.uint32), oscale.view(np.uint32))
        assert np.array_equal(s[m].cpu().numpy(), osum)
    assert scale[0, 0].item() == 1.0 and q[1, 32].item() == -127 and q[1, 48].item() == 0


@pytest.mark.parametrize("act", [0, 1])
def test_epilogue_bias_gelu_mul_residual(zq, oracle, act):
    n, k = 384, 256
    raw = make_weight(oracle, ggml.Q4_0, n, k, std=0.1)
    qw = zq.QuantWeight(raw, ggml.Q4_0, n, k)
    x = make_x(1, k)
    rng = np.random.default_rng(5)
    bias, mul, res = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    base = oracle.linear(ggml.Q4_0, raw, x, n, k, act_mode=act, n_threads=2)[0]
    want = oracle.gelu(base + bias) * mul + res
    t = lambda a: torch.from_numpy(a).cuda()
    got = zq.quant_matmul_no_grad(t(x), qw, act, bias=t(bias), gelu=True, mul=t(mul[None]), residual=t(res[None]))
    assert rel_l2(got.cpu().numpy()[0], want) <= 1e-5
    if act == 1:  # exact dots + exactly ordered epilogue
        assert np.array_equal(got.cpu().numpy()[0], want)
    # residual may alias the output (x += W h, src/models/gpt2.zig:495-496)
    y = t(res[None].copy())
    zq.quant_matmul_no_grad(t(x), qw, act, bias=t(bias), residual=y, out=y)
    assert rel_l2(y.cpu().numpy()[0], base + bias + res) <= 1e-6


@pytest.mark.parametrize("qtype", TYPES)
def test_vocab_head_full_size(zq, oracle, qtype):
    """1152 -> 262144, the largest GEMV of the path (Gemma-3 logits, gemma3.zig:830-846)."""
    n, k = 262144, 1152
    g = torch.Generator(device="cuda").manual_seed(42)
    w = torch.randn(n, k, generator=g, device="cuda") * 0.02
    raw_d = ggml.quantize(qtype, w)
    del w
    qw = zq.QuantWeight(raw_d, qtype, n, k)
    raw = raw_d.cpu().numpy()
    x = make_x(1, k)
    xd = torch.from_numpy(x).cuda()
    got32 = zq.quant_matmul_no_grad(xd, qw, zq.ACT_F32).cpu().numpy()
    gotq8 = zq.quant_matmul_no_grad(xd, qw, zq.ACT_Q8).cpu().numpy()
    want32 = oracle.linear(qtype, raw, x, n, k, act_mode=0, n_threads=8)
    wantq8 = oracle.linear(qtype, raw, x, n, k, act_mode=1, n_threads=8)
    assert rel_l2(got32, want32) <= REL_L2_GUARD
    assert np.array_equal(gotq8, wantq8)
    assert int(zq.argmax(torch.from_numpy(got32[0]).cuda()).item()) == oracle.argmax(want32[0])


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("k", [1152, 2048])
def test_single_row_kernel_ragged_tail(zq, oracle, qtype, k):
    """Enough row tiles for the one-activation-row kernel (whole rows per warp), with a row count that
    is not a multiple of 16 and a bias + residual epilogue."""
    n = 148 * 2 * 8 * 16 + 77
    raw = make_weight(oracle, qtype, n, k)
    qw = zq.QuantWeight(raw, qtype, n, k)
    x = make_x(1, k)
    rng = np.random.default_rng(5)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((1, n)).astype(np.float32)
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_F32, bias=torch.from_numpy(bias).cuda(),
                                  residual=torch.from_numpy(res).cuda()).cpu().numpy()
    want = oracle.linear(qtype, raw, x, n, k, act_mode=0, n_threads=8) + bias + res
    assert rel_l2(got, want) <= REL_L2_GUARD


def test_large_k_f32(zq, oracle):
    """14336 -> 4096 (sharded-GEMM shape); K beyond the reference thread pool's 8192 limit, so only
    the f32-activation path has a CPU counterpart."""
    n, k = 512, 14336
    raw = make_weight(oracle, ggml.Q4_0, n, k)
    qw = zq.QuantWeight(raw, ggml.Q4_0, n, k)
    x = make_x(1, k)
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_F32).cpu().numpy()
    want = oracle.linear(ggml.Q4_0, raw, x, n, k, act_mode=0, n_threads=4)
    assert rel_l2(got, want) <= REL_L2_GUARD


def test_linearity_property(zq, oracle):
    """W(a x1 + x2) == a W x1 + W x2 to f32 accuracy — a size-independent check of the f32 path."""
    n, k = 4096, 4096
    raw = make_weight(oracle, ggml.Q8_0, n, k)
    qw = zq.QuantWeight(raw, ggml.Q8_0, n, k)
    x1, x2 = torch.from_numpy(make_x(1, k, 1)).cuda(), torch.from_numpy(make_x(1, k, 2)).cuda()
    lhs = zq.quant_matmul_no_grad(2.0 * x1 + x2, qw)
    rhs = 2.0 * zq.quant_matmul_no_grad(x1, qw) + zq.quant_matmul_no_grad(x2, qw)
    assert rel_l2(lhs.cpu().numpy(), rhs.cpu().numpy()) <= 1e-5


def test_error_statuses(zq):
    from zignn_b200 import _lib
    with pytest.raises(_lib.ZqError) as e:
        zq.QuantWeight(np.zeros(22, np.uint8), 6, 1, 32)  # q5_0
    assert e.value.status == 2
    with pytest.raises(_lib.ZqError) as e:
        zq.QuantWeight(np.zeros(18, np.uint8), ggml.Q4_0, 1, 48)  # in_dim % 32 != 0
    assert e.value.status == 1
    qw = zq.QuantWeight(np.zeros(18, np.uint8), ggml.Q4_0, 1, 32)
    with pytest.raises(ValueError):
        zq.quant_matmul_no_grad(torch.zeros(1, 64, device="cuda"), qw)
    # zero rows is a no-op
    assert zq.quant_matmul_no_grad(torch.zeros(0, 32, device="cuda"), qw).shape == (0, 1)


def test_matvec_f32_and_argmax(zq, oracle):
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((5003, 768)) * 0.02).astype(np.float32)
    x = rng.standard_normal(768).astype(np.float32)
    got = zq.matvec_f32(torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()).cpu().numpy()
    want = oracle.matmul_f32(0, w.view(np.uint8), x, 5003, 768, 4)
    assert rel_l2(got, want) <= REL_L2_GUARD
    assert int(zq.argmax(torch.from_numpy(want).cuda()).item()) == oracle.argmax(want)
    ties = np.array([1, 7, 7, 7, -2], np.float32)
    assert int(zq.argmax(torch.from_numpy(ties).cuda()).item()) == 1
    big = np.zeros(300000, np.float32)
    big[[250000, 123456]] = 3.0
    assert int(zq.argmax(torch.from_numpy(big).cuda()).item()) == 123456


# ---- transposed product (backward with respect to the activations) ----------------------------------

REL_L2_TRANS = 6e-4  # fp16 copies of weights and gradients, f32 accumulation: about 3e-4


@pytest.mark.parametrize("qtype", [ggml.Q4_0, ggml.Q4_1, ggml.Q8_0])
@pytest.mark.parametrize("shape", [(256, 128, 130), (72, 96, 5), (1152, 6912, 64), (6912, 1152, 300)])
def test_matmul_transposed_against_oracle(zq, oracle, qtype, shape):
    """grad_x = grad_out . W for ragged row counts, weight-row counts that are not a multiple of the 128-row
    stage, in_dim below one 128-column tile, and shapes whose weight rows are split over several CTAs."""
    out_dim, in_dim, m = shape
    g = torch.Generator().manual_seed(out_dim + m)
    w = torch.randn(out_dim, in_dim, generator=g) * 0.02
    raw = ggml.quantize(qtype, w).numpy()
    go = torch.randn(m, out_dim, generator=g) * 1e-3  # gradient-sized values: the row scale matters
    go[0] = 0.0
    qw = zq.QuantWeight(raw, qtype, out_dim, in_dim)
    got = zq.quant_matmul_transposed(go.cuda(), qw).cpu().numpy()
    want = oracle.matmul_transposed(qtype, raw, go.numpy(), out_dim, in_dim, n_threads=8)
    assert rel_l2(got, want) <= REL_L2_TRANS, rel_l2(got, want)
    assert np.all(got[0] == 0.0)


def test_matmul_transposed_accumulates_like_the_reference_kernels(zq, oracle):
    out_dim, in_dim, m = 4096, 256, 40  # 32 stages: split over CTAs, partial sums meet by atomic adds
    g = torch.Generator().manual_seed(3)
    raw = ggml.quantize(ggml.Q4_0, torch.randn(out_dim, in_dim, generator=g) * 0.02).numpy()
    go = torch.randn(m, out_dim, generator=g)
    base = torch.randn(m, in_dim, generator=g)
    qw = zq.QuantWeight(raw, ggml.Q4_0, out_dim, in_dim)
    gx = base.clone().cuda()
    out = zq.quant_matmul_transposed(go.cuda(), qw, grad_x=gx, accumulate=True)
    assert out.data_ptr() == gx.data_ptr()
    want = oracle.matmul_transposed(ggml.Q4_0, raw, go.numpy(), out_dim, in_dim, grad_x=base.numpy(), n_threads=8)
    assert rel_l2(gx.cpu().numpy(), want) <= REL_L2_TRANS
    # overwrite mode ignores what grad_x held
    gx2 = torch.full((m, in_dim), 7.0, device="cuda")
    zq.quant_matmul_transposed(go.cuda(), qw, grad_x=gx2)
    want2 = oracle.matmul_transposed(ggml.Q4_0, raw, go.numpy(), out_dim, in_dim, n_threads=8)
    assert rel_l2(gx2.cpu().numpy(), want2) <= REL_L2_TRANS


def test_quant_matmul_backward_to_activations(zq, oracle):
    """quant_matmul_no_grad on an input that requires grad carries the backward to x (the weight stays
    frozen): d/dx sum(y * c) = c . W."""
    out_dim, in_dim = 384, 160
    g = torch.Generator().manual_seed(11)
    raw = ggml.quantize(ggml.Q8_0, torch.randn(out_dim, in_dim, generator=g) * 0.05).numpy()
    qw = zq.QuantWeight(raw, ggml.Q8_0, out_dim, in_dim)
    x = torch.randn(3, 7, in_dim, generator=g).cuda().requires_grad_(True)
    c = torch.randn(3, 7, out_dim, generator=g).cuda()
    y = zq.quant_matmul_no_grad(x, qw)
    assert y.requires_grad and y.shape == (3, 7, out_dim)
    (y * c).sum().backward()
    want = oracle.matmul_transposed(ggml.Q8_0, raw, c.cpu().numpy().reshape(-1, out_dim), out_dim, in_dim)
    assert rel_l2(x.grad.cpu().numpy().reshape(-1, in_dim), want) <= REL_L2_TRANS
    with torch.no_grad():
        assert not zq.quant_matmul_no_grad(x, qw).requires_grad


def test_matmul_transposed_rejects_bad_arguments(zq):
    raw = ggml.quantize(ggml.Q4_0, torch.zeros(12, 32)).numpy()  # 12 weight rows: not a multiple of 8
    qw = zq.QuantWeight(raw, ggml.Q4_0, 12, 32)
    with pytest.raises(RuntimeError, match="UNSUPPORTED"):
        zq.quant_matmul_transposed(torch.zeros(2, 12, device="cuda"), qw)
    with pytest.raises(ValueError):
        zq.quant_matmul_transposed(torch.zeros(2, 16, device="cuda"), qw)


@pytest.mark.parametrize("qtype,mode", [(ggml.Q4_0, 0), (ggml.Q8_0, 1)])
def test_host_buffer_call_writes_the_same_bits_into_pinned_memory(zq, qtype, mode):
    """HostLinear: x from a pinned host buffer, y written by the kernel directly into pinned host memory
    (first call plain, later calls replayed), and the pageable route — all equal to the device-buffer call."""
    out_dim, in_dim = 40000, 1152  # enough row tiles for the whole-rows kernels
    g = torch.Generator().manual_seed(9)
    raw = ggml.quantize(qtype, torch.randn(out_dim, in_dim, generator=g) * 0.02).numpy()
    qw = zq.QuantWeight(raw, qtype, out_dim, in_dim)
    lin = zq.HostLinear(qw, 1, mode)
    hx, hy = torch.empty(1, in_dim).pin_memory(), torch.empty(1, out_dim).pin_memory()
    for seed in (1, 2, 3):
        hx.copy_(torch.randn(1, in_dim, generator=g))
        hy.fill_(float("nan"))
        lin(hx, hy)
        want = zq.quant_matmul_no_grad(hx.cuda(), qw, mode).cpu()
        assert torch.equal(hy, want)
    pageable = torch.empty(1, out_dim)
    lin(hx.clone(), pageable)
    assert torch.equal(pageable, want)
    with pytest.raises(ValueError):
        lin(hx, torch.empty(1, out_dim + 1).pin_memory())


# ---- the many-row products at the shapes of the sweep and of the sharded configuration ------------------


def _sampled_rows(n, count=64, seed=17):
    """Weight rows to compare: both ends, a row on each side of every 128-row tile boundary near the ends,
    and a seeded sample of the middle."""
    rng = np.random.default_rng(seed)
    fixed = [0, 1, 127, 128, 129, 255, 256, n - 257, n - 129, n - 128, n - 2, n - 1]
    rest = rng.choice(n, size=count - len(fixed), replace=False)
    return np.unique(np.clip(np.concatenate([fixed, rest]), 0, n - 1))


@pytest.mark.parametrize("k,n,m", [(4096, 14336, 64), (4096, 14336, 2048), (14336, 4096, 64), (14336, 4096, 2048),
                                   (1152, 6912, 512), (6912, 1152, 512), (1152, 262144, 128)])
def test_tensor_core_gemm_at_full_shapes_sampled_rows(zq, oracle, k, n, m):
    """The tcgen05 GEMM at the real shapes (Q4_0; up to 224 K-stages, the paired-tile form, the 262144-row
    vocabulary head). The CPU side computes a sample of the weight rows: a subset of the raw row bytes is a
    smaller weight whose outputs are exactly those columns of the full product."""
    g = torch.Generator(device="cuda").manual_seed(1000 + k + m)
    raw_d = ggml.quantize(ggml.Q4_0, torch.randn(n, k, generator=g, device="cuda") * 0.02)
    qw = zq.QuantWeight(raw_d, ggml.Q4_0, n, k)
    x = torch.randn(m, k, generator=g, device="cuda")
    got = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32)
    rows = _sampled_rows(n)
    row_bytes = k // 32 * 18
    sub = raw_d.view(n, row_bytes)[torch.from_numpy(rows).cuda()].cpu().numpy().reshape(-1)
    want = oracle.linear(ggml.Q4_0, sub, x.cpu().numpy(), len(rows), k, act_mode=0, n_threads=16)
    got_s = got[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    err = rel_l2(got_s, want)
    assert err <= REL_L2_BAR
    assert err <= REL_L2_GEMM_GUARD, err
    worst = max(rel_l2(got_s[r], want[r]) for r in range(0, m, max(1, m // 16)))
    assert worst <= REL_L2_BAR, worst
    # A size-independent check that touches every output: the sum of an output row equals x . (column sums of
    # W). Independent rounding errors of 3e-4 per output add up to about 3e-4 of the row's 2-norm; a wrong
    # 128-column tile would move the sum by about ten times the bound.
    colsum_w = qw.dequantize().sum(dim=0, dtype=torch.float64)
    want_sum = x.double() @ colsum_w
    got_sum = got.sum(dim=1, dtype=torch.float64)
    bound = 2e-3 * got.double().norm(dim=1)
    assert bool(((got_sum - want_sum).abs() <= bound).all()), float(((got_sum - want_sum).abs() / bound).max())


@pytest.mark.parametrize("m", [64, 512])
def test_exact_int8_gemm_at_vocab_head_sampled_rows(zq, oracle, m):
    """The exact int8 GEMM on the 1152 -> 262144 head in Q4_1 (the batched engine's logits): sampled weight
    rows, every activation row, bit-identical to the CPU path."""
    n, k = 262144, 1152
    g = torch.Generator(device="cuda").manual_seed(77 + m)
    raw_d = ggml.quantize(ggml.Q4_1, torch.randn(n, k, generator=g, device="cuda") * 0.02)
    qw = zq.QuantWeight(raw_d, ggml.Q4_1, n, k)
    x = torch.randn(m, k, generator=g, device="cuda")
    got = zq.quant_matmul_no_grad(x, qw, zq.ACT_Q8)
    rows = _sampled_rows(n)
    sub = raw_d.view(n, k // 32 * 20)[torch.from_numpy(rows).cuda()].cpu().numpy().reshape(-1)
    want = oracle.linear(ggml.Q4_1, sub, x.cpu().numpy(), len(rows), k, act_mode=1, n_threads=16)
    assert np.array_equal(got[:, torch.from_numpy(rows).cuda()].cpu().numpy(), want)


@pytest.mark.parametrize("out_dim,in_dim,m", [(14336, 4096, 2048), (4096, 14336, 64)])
def test_matmul_transposed_at_full_shapes_sampled_columns(zq, oracle, out_dim, in_dim, m):
    """grad_x = grad_out . W at the sharded-GEMM shapes; the CPU side computes a sample of the rows of
    grad_out (each output row depends on its own grad_out row only)."""
    g = torch.Generator(device="cuda").manual_seed(out_dim + m)
    raw_d = ggml.quantize(ggml.Q4_0, torch.randn(out_dim, in_dim, generator=g, device="cuda") * 0.02)
    qw = zq.QuantWeight(raw_d, ggml.Q4_0, out_dim, in_dim)
    go = torch.randn(m, out_dim, generator=g, device="cuda") * 1e-3
    got = zq.quant_matmul_transposed(go, qw)
    rows = np.unique(np.concatenate([[0, 1, m - 1], np.random.default_rng(3).choice(m, size=5, replace=False)]))
    want = oracle.matmul_transposed(ggml.Q4_0, raw_d.cpu().numpy(), go[torch.from_numpy(rows).cuda()].cpu().numpy(),
                                    out_dim, in_dim, n_threads=16)
    err = rel_l2(got[torch.from_numpy(rows).cuda()].cpu().numpy(), want)
    assert err <= REL_L2_TRANS, err


@pytest.mark.parametrize("qt", [ggml.Q4_0, ggml.Q4_1, ggml.Q8_0])
def test_matmul_transposed_many_rows_on_pairs_of_ctas(zq, oracle, qt):
    """Many rows on a matrix of 1024 weight rows and more: W^T is laid out as fp16 operand tiles and the product runs
    on the tcgen05 kernel of the forward GEMM (13 ragged tiles of output columns x 5 ragged tiles of rows = 65 tiles
    for the 74 pairs of CTAs). Sampled rows against the CPU statement; accumulation adds to grad_x exactly; with
    cluster launches switched off the earlier kernel gives the same within the tolerance."""
    from zignn_b200 import _lib
    out_dim, in_dim, m = 1024, 3104, 2100
    g = torch.Generator(device="cuda").manual_seed(int(qt) + 5)
    raw_d = ggml.quantize(qt, torch.randn(out_dim, in_dim, generator=g, device="cuda") * 0.02)
    qw = zq.QuantWeight(raw_d, qt, out_dim, in_dim)
    go = torch.randn(m, out_dim, generator=g, device="cuda") * 1e-3
    go[3] = 0.0
    got = zq.quant_matmul_transposed(go, qw)
    rows = np.unique(np.concatenate([[0, 1, 3, 255, 256, 511, 512, m - 1], np.random.default_rng(4).choice(m, size=24, replace=False)]))
    sel = torch.from_numpy(rows).cuda()
    want = oracle.matmul_transposed(qt, raw_d.cpu().numpy(), go[sel].cpu().numpy(), out_dim, in_dim, n_threads=16)
    err = rel_l2(got[sel].cpu().numpy(), want)
    assert err <= REL_L2_TRANS, err
    assert bool((got[3] == 0).all())
    full = go @ qw.dequantize()
    assert torch.allclose(got, full, rtol=0, atol=4e-3 * float(full.abs().max()))
    base = torch.randn(m, in_dim, generator=g, device="cuda") * 1e-3
    acc = zq.quant_matmul_transposed(go, qw, grad_x=base.clone(), accumulate=True)
    assert torch.equal(acc, base + got)
    lib = _lib.load()
    lib.zq_set_cluster_launch(0)
    try:
        earlier = zq.quant_matmul_transposed(go, qw)
    finally:
        lib.zq_set_cluster_launch(1)
    assert rel_l2(earlier.cpu().numpy(), got.cpu().numpy()) <= 1e-5  # the same fp16 operands, another order of the sums
    assert _lib.device_error() == 0


# ---- the weight-streaming tensor-core form (17-128 activation rows, matrices of 12 288 rows and more) ----


STREAM_TYPES = [(ggml.Q4_0, 18), (ggml.Q4_1, 20), (ggml.Q8_0, 34)]


@pytest.mark.parametrize("qt,block_bytes", STREAM_TYPES)
@pytest.mark.parametrize("k,n", [(1152, 37888 + 24), (1024, 12416), (4096, 14336)])
@pytest.mark.parametrize("m", [17, 32, 33, 64, 100, 128])
def test_streaming_gemm_sampled_rows(zq, oracle, qt, block_bytes, k, n, m):
    """Few activation rows against many weight rows: f32-activation calls of 17-128 rows that bring the workspace
    zq_matmul_workspace_bytes asks for run the persistent weight-streaming kernel (weights as the N operand of
    tcgen05.mma, packed quants by tensor copies). Covers both tile heights (256 rows from 37 888 weight rows on,
    128 below), a last tile that is cut off (n not a multiple of the tile), a K whose last chunk is short (1152 =
    9 quads), up to 32 rows spread over the lane quarters and more in natural order. Sampled weight rows against
    the CPU path (dequant.zig:170-309), every output against the dequantised product."""
    g = torch.Generator(device="cuda").manual_seed(31 * m + k + int(qt))
    raw_d = ggml.quantize(qt, torch.randn(n, k, generator=g, device="cuda") * 0.02)
    qw = zq.QuantWeight(raw_d, qt, n, k)
    x = torch.randn(m, k, generator=g, device="cuda")
    from zignn_b200 import _lib
    assert _lib.load().zq_matmul_workspace_bytes(qw.handle, m, zq.ACT_F32) > 0  # the streaming form is on offer
    got = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32)
    assert bool(torch.isfinite(got).all())
    rows = _sampled_rows(n)
    sub = raw_d.view(n, k // 32 * block_bytes)[torch.from_numpy(rows).cuda()].cpu().numpy().reshape(-1)
    want = oracle.linear(qt, sub, x.cpu().numpy(), len(rows), k, act_mode=0, n_threads=16)
    got_s = got[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    err = rel_l2(got_s, want)
    assert err <= REL_L2_BAR
    assert err <= REL_L2_GEMM_GUARD, err
    worst = max(rel_l2(got_s[r], want[r]) for r in range(m))
    assert worst <= REL_L2_BAR, worst
    full = x @ qw.dequantize().t()
    assert float((got - full).norm() / full.norm()) <= REL_L2_GEMM_GUARD
    # no output is left unwritten or written twice with different values: element-wise closeness everywhere
    assert bool(((got - full).abs() <= 4e-3 * full.abs().max()).all())
    assert _lib.device_error() == 0


def test_streaming_gemm_epilogue_and_row_counts(zq):
    """bias, GELU, multiplier and residual in the streaming form's epilogue, for row counts on both sides of the
    interleaved / natural placement (32 | 33) and a count that leaves lane quarters empty (65)."""
    k, n = 1152, 12800
    g = torch.Generator(device="cuda").manual_seed(5)
    raw_d = ggml.quantize(ggml.Q4_0, torch.randn(n, k, generator=g, device="cuda") * 0.02)
    qw = zq.QuantWeight(raw_d, ggml.Q4_0, n, k)
    wd = qw.dequantize()
    for m in (17, 31, 32, 33, 65, 128):
        x = torch.randn(m, k, generator=g, device="cuda")
        bias = torch.randn(n, generator=g, device="cuda")
        mul = torch.randn(m, n, generator=g, device="cuda")
        res = torch.randn(m, n, generator=g, device="cuda")
        base = x @ wd.t()
        got = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32, bias=bias)
        assert torch.allclose(got, base + bias, rtol=0, atol=4e-3 * float(base.abs().max()))
        got = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32, bias=bias, gelu=True, mul=mul, residual=res)
        want = res + torch.nn.functional.gelu(base + bias, approximate="tanh") * mul
        assert torch.allclose(got, want, rtol=0, atol=6e-3 * float(want.abs().max()))
    # a call without workspace keeps the exact small-batch kernel (passes of 16 rows)
    x = torch.randn(20, k, generator=g, device="cuda")
    from zignn_b200 import _lib
    from zignn_b200 import structs as S
    import ctypes as C
    y = torch.empty(20, n, device="cuda")
    ep = S.Epilogue(None, 0, None, None)
    rc = _lib.load().zq_matmul(qw.handle, x.data_ptr(), y.data_ptr(), 20, zq.ACT_F32, C.byref(ep), None, 0,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert rel_l2(y.cpu().numpy(), (x.double() @ wd.double().t()).float().cpu().numpy()) <= REL_L2_GUARD


@pytest.mark.parametrize("qt,block_bytes", STREAM_TYPES)
@pytest.mark.parametrize("k,n,m", [(256, 2600, 2300), (1024, 2600, 2300), (1024, 3880, 2148)])
def test_streaming_gemm_wide_many_activation_tiles_and_epilogue(zq, qt, block_bytes, k, n, m):
    """More than 128 activation rows on a small matrix, ragged weight and activation tiles, every ring wrapping
    several times within a tile, and the whole epilogue (bias, GELU, multiplier, residual).
    K = 256: one CTA per tile of 256 x 256 (99 tiles). K = 1024: a pair of CTAs per tile of 256 weight rows x 512
    activation rows (tcgen05 with cta_group::2): 55 tiles, less than a round of the 74 pairs; 80 tiles, whose last
    six are walked as twelve half tiles of one activation tile."""
    g = torch.Generator(device="cuda").manual_seed(77 + int(qt))
    raw_d = ggml.quantize(qt, torch.randn(n, k, generator=g, device="cuda") * 0.05)
    qw = zq.QuantWeight(raw_d, qt, n, k)
    x = torch.randn(m, k, generator=g, device="cuda")
    bias = torch.randn(n, generator=g, device="cuda")
    mul = torch.randn(m, n, generator=g, device="cuda")
    res = torch.randn(m, n, generator=g, device="cuda")
    base = x @ qw.dequantize().t()
    got = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32)
    assert torch.allclose(got, base, rtol=0, atol=4e-3 * float(base.abs().max()))
    assert rel_l2(got.cpu().numpy(), base.cpu().numpy()) <= REL_L2_GEMM_GUARD
    got = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32, bias=bias, gelu=True, mul=mul, residual=res)
    want = res + torch.nn.functional.gelu(base + bias, approximate="tanh") * mul
    assert torch.allclose(got, want, rtol=0, atol=6e-3 * float(want.abs().max()))
    from zignn_b200 import _lib
    assert _lib.device_error() == 0


def test_many_row_gemm_without_cluster_launches(zq):
    """zq_set_cluster_launch(0): a shape that runs on pairs of CTAs takes the single-CTA form instead, on the activation
    image as it is laid out for the pairs; the same result within the path's tolerance, and the pairs are back
    afterwards."""
    from zignn_b200 import _lib
    lib = _lib.load()
    k, n, m = 1024, 3880, 2148
    g = torch.Generator(device="cuda").manual_seed(91)
    raw_d = ggml.quantize(ggml.Q4_0, torch.randn(n, k, generator=g, device="cuda") * 0.05)
    qw = zq.QuantWeight(raw_d, ggml.Q4_0, n, k)
    x = torch.randn(m, k, generator=g, device="cuda")
    base = x @ qw.dequantize().t()
    pairs = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32)
    assert lib.zq_set_cluster_launch(0) == 0
    try:
        single = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32)
    finally:
        lib.zq_set_cluster_launch(1)
    for got in (pairs, single):
        assert torch.allclose(got, base, rtol=0, atol=4e-3 * float(base.abs().max()))
    # both forms multiply the same fp16 operands and add in the same K order
    assert rel_l2(single.cpu().numpy(), pairs.cpu().numpy()) <= 1e-6
    assert _lib.device_error() == 0


@pytest.mark.parametrize("qt,block_bytes", STREAM_TYPES)
@pytest.mark.parametrize("m", [129, 256, 300, 520])
def test_streaming_gemm_wide_sampled_rows(zq, oracle, qt, block_bytes, m):
    """More than 128 activation rows on a matrix with a 256-row weight tile for every SM: the streaming kernel with
    two activation tiles per CTA tile (both accumulators of tensor memory in one tile), activation rows tiled in
    256s with a ragged last tile."""
    k, n = 1152, 148 * 256 + 40
    g = torch.Generator(device="cuda").manual_seed(m + int(qt))
    raw_d = ggml.quantize(qt, torch.randn(n, k, generator=g, device="cuda") * 0.02)
    qw = zq.QuantWeight(raw_d, qt, n, k)
    x = torch.randn(m, k, generator=g, device="cuda")
    bias = torch.randn(n, generator=g, device="cuda")
    got = zq.quant_matmul_no_grad(x, qw, zq.ACT_F32, bias=bias)
    rows = _sampled_rows(n)
    sub = raw_d.view(n, k // 32 * block_bytes)[torch.from_numpy(rows).cuda()].cpu().numpy().reshape(-1)
    want = oracle.linear(qt, sub, x.cpu().numpy(), len(rows), k, act_mode=0, n_threads=16) + bias.cpu().numpy()[rows]
    got_s = got[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    assert rel_l2(got_s, want) <= REL_L2_GEMM_GUARD
    full = x @ qw.dequantize().t() + bias
    assert bool(((got - full).abs() <= 4e-3 * full.abs().max()).all())
    from zignn_b200 import _lib
    assert _lib.device_error() == 0
