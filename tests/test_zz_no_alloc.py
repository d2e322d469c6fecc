"""The entry point that brings its own scratch (zq_matmul_q8_static) against the ordinary one.

Some hosts cannot allocate device memory when they call the matmul (all of it already belongs to their
own pool, or an allocation's hidden synchronisation / possible failure is not acceptable in their
decode loop), so the library carries a fixed scratch array for them. This file is named to be collected
last: if it fails under `-x`, every other test has already run. It must pass alone in a fresh process
and after the other tests."""
import numpy as np
import pytest
import torch

from zignn_b200 import ggml

pytestmark = pytest.mark.gpu


def _weight(zq, oracle, qtype, n, k, seed):
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
    return zq.QuantWeight(oracle.quantize(qtype, w), qtype, n, k)


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(zq, oracle):
    from zignn_b200 import _lib
    rng = np.random.default_rng(5)
    # two different shapes and types back to back: the second call reuses the array the first one left
    cases = [(ggml.Q4_0, 600, 1152, 3), (ggml.Q8_0, 300, 6912, 16), (ggml.Q4_1, 96, 160, 1)]
    for qtype, n, k, m in cases:
        qw = _weight(zq, oracle, qtype, n, k, seed=n)
        for call in range(2):
            x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
            want = zq.quant_matmul_no_grad(x, qw, zq.ACT_Q8)
            got = zq.quant_matmul_q8_static(x, qw)
            assert torch.equal(got, want), (qtype, call)  # same kernels, same bits: tolerance 0
    # epilogue goes through as well
    qw = _weight(zq, oracle, ggml.Q4_0, 256, 256, seed=1)
    x = torch.from_numpy(rng.standard_normal((2, 256)).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(256).astype(np.float32)).cuda()
    res = torch.from_numpy(rng.standard_normal((2, 256)).astype(np.float32)).cuda()
    want = zq.quant_matmul_no_grad(x, qw, zq.ACT_Q8, bias=bias, gelu=True, residual=res)
    got = zq.quant_matmul_q8_static(x, qw, bias=bias, gelu=True, residual=res)
    assert torch.equal(got, want)
    # sizes beyond the built-in scratch are refused with the limit status, not truncated
    with pytest.raises(_lib.ZqError) as e:
        zq.quant_matmul_q8_static(torch.zeros(17, 256, device="cuda"), qw)
    assert e.value.status == 5
    big = zq.QuantWeight(np.zeros(ggml.tensor_bytes(ggml.Q4_0, 16416), np.uint8), ggml.Q4_0, 1, 16416)
    with pytest.raises(_lib.ZqError) as e:
        zq.quant_matmul_q8_static(torch.zeros(1, 16416, device="cuda"), big)
    assert e.value.status == 5
