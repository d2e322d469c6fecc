"""The sm_100a module image of the f32 forward kernels, loaded the way zig-nn's CUDA backend loads its
kernels: cuModuleLoadData on the image bytes, cuModuleGetFunction by NAME, cuLaunchKernel with exactly the
grid / block / shared-memory sizes that src/cuda_ops.zig computes (grid_for, next_pow2, block * 4 bytes).
Results are compared with the CPU statements of the same ops (runtime_kernels.zig:40-81, 148-213, 262-268,
restated in the oracle) and with numpy for the index-shuffling kernels."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BLOCK_SIZE = 256  # cuda_ops.zig:11


def grid_for(n):  # cuda_ops.zig:13-15
    return (n + BLOCK_SIZE - 1) // BLOCK_SIZE


def next_pow2(v):  # cuda_ops.zig:17-27
    if v == 0:
        return 1
    x = v - 1
    for s in (1, 2, 4, 8, 16):
        x |= x >> s
    return x + 1


class Module:
    """CudaContext.load_module / get_function / launch_kernel (src/backend/cuda_context.zig:200-240)."""

    def __init__(self, image_path):
        torch.zeros(1, device="cuda")  # a current context, as CudaContext.init provides one
        self.cu = C.CDLL("libcuda.so.1")
        self.image = open(image_path, "rb").read()
        self.mod = C.c_void_p()
        rc = self.cu.cuModuleLoadData(C.byref(self.mod), self.image)
        assert rc == 0, "cuModuleLoadData failed: %d" % rc
        self.funcs = {}

    def get_function(self, name):
        if name not in self.funcs:
            f = C.c_void_p()
            rc = self.cu.cuModuleGetFunction(C.byref(f), self.mod, name.encode())
            assert rc == 0, "cuModuleGetFunction(%s) failed: %d" % (name, rc)
            self.funcs[name] = f
        return self.funcs[name]

    def launch(self, name, grid, block, shared, *params):
        """params: torch tensors (device pointers), ints (c_int) or floats (c_float), in kernel order."""
        vals = []
        for p in params:
            if isinstance(p, torch.Tensor):
                vals.append(C.c_uint64(p.data_ptr()))
            elif isinstance(p, float):
                vals.append(C.c_float(p))
            else:
                vals.append(C.c_int(int(p)))
        arr = (C.c_void_p * len(vals))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = self.cu.cuLaunchKernel(self.get_function(name), grid, 1, 1, block, 1, 1, shared, stream, arr, None)
        assert rc == 0, "cuLaunchKernel(%s) failed: %d" % (name, rc)
        torch.cuda.synchronize()

    def close(self):
        if self.mod:
            self.cu.cuModuleUnload(self.mod)
            self.mod = None


@pytest.fixture(scope="module", params=["cuda_kernels.fatbin", "cuda_kernels.cubin"])
def module(request):
    path = os.path.join(REPO, "zig-nn_b200", request.param)
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    assert os.path.exists(path), "module image missing: run zig-nn_b200/build.py"
    m = Module(path)
    yield m
    m.close()


NAMES = ["add_broadcast", "mul_broadcast", "gelu_kernel", "scale_kernel", "softmax_kernel", "softmax_out_kernel",
         "layernorm_kernel", "layernorm_fwd_kernel", "reduction_sum_rows_kernel", "reduction_sum_cols_kernel",
         "reduction_sum_1d_kernel", "transpose_2d_kernel", "modulate_adaln_kernel", "gather_kernel"]


def test_every_kernel_name_resolves(module):
    for name in NAMES:
        module.get_function(name)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (7, 64), (4, 257), (2, 1024), (3, 2500)])
def test_softmax_in_place_and_out_of_place(module, oracle, rows, cols):
    x = np.random.default_rng(rows * 131 + cols).standard_normal((rows, cols)).astype(np.float32) * 3
    want = oracle.softmax_forward(x)
    block = next_pow2(min(cols, 1024))
    d = dev(x)
    module.launch("softmax_kernel", rows, block, block * 4, d, rows, cols)  # dispatch_softmax, cuda_ops.zig:88-111
    np.testing.assert_allclose(d.cpu().numpy(), want, rtol=2e-6, atol=1e-7)
    src, out = dev(x), torch.zeros(rows, cols, device="cuda")
    module.launch("softmax_out_kernel", rows, block, block * 4, out, src, rows, cols)  # dispatch_softmax_out, :518-543
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=2e-6, atol=1e-7)
    assert torch.equal(src.cpu(), torch.from_numpy(x))  # x untouched
    np.testing.assert_allclose(out.sum(dim=1).cpu().numpy(), 1.0, rtol=1e-5)


@pytest.mark.parametrize("rows,cols", [(1, 2), (5, 48), (3, 768), (2, 1152), (2, 3000)])
def test_layer_norm_both_forms(module, oracle, rows, cols):
    rng = np.random.default_rng(cols)
    x = (rng.standard_normal((rows, cols)) * 2 + 0.5).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(cols)).astype(np.float32)
    eps = 1e-5
    want = oracle.layer_norm_forward(x, gamma, beta, eps)
    block = next_pow2(min(cols, 1024))
    dx, dg, db = dev(x), dev(gamma), dev(beta)
    out = torch.zeros(rows, cols, device="cuda")
    module.launch("layernorm_kernel", rows, block, block * 4, out, dx, dg, db, rows, cols, eps)  # :113-146
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=2e-5, atol=2e-5)
    out2, xn, inv = torch.zeros(rows, cols, device="cuda"), torch.zeros(rows, cols, device="cuda"), torch.zeros(rows, device="cuda")
    module.launch("layernorm_fwd_kernel", rows, block, block * 4, out2, xn, inv, dx, dg, db, rows, cols, eps)  # :545-575
    np.testing.assert_allclose(out2.cpu().numpy(), want, rtol=2e-5, atol=2e-5)
    mean = x.astype(np.float64).mean(axis=1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=1, keepdims=True)
    np.testing.assert_allclose(inv.cpu().numpy(), (1.0 / np.sqrt(var + eps)).reshape(-1), rtol=1e-5)
    np.testing.assert_allclose(xn.cpu().numpy(), (x - mean) / np.sqrt(var + eps), rtol=1e-4, atol=1e-5)


def test_elementwise_and_broadcast(module, oracle):
    rng = np.random.default_rng(3)
    n, nb = 6912 * 3 + 5, 1152 * 3  # a_total need not be a multiple of the block; b divides the index by modulo
    a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(nb).astype(np.float32)
    da, db_, out = dev(a), dev(b), torch.zeros(n, device="cuda")
    idx = np.arange(n) % nb
    module.launch("add_broadcast", grid_for(n), BLOCK_SIZE, 0, out, da, db_, n, nb)  # dispatch_broadcast_binop, :36-63
    assert np.array_equal(out.cpu().numpy(), a + b[idx])
    module.launch("mul_broadcast", grid_for(n), BLOCK_SIZE, 0, out, da, db_, n, nb)
    assert np.array_equal(out.cpu().numpy(), a * b[idx])
    module.launch("scale_kernel", grid_for(n), BLOCK_SIZE, 0, out, da, 0.125, n)  # dispatch_scale, :236-260
    assert np.array_equal(out.cpu().numpy(), a * np.float32(0.125))
    module.launch("gelu_kernel", grid_for(n), BLOCK_SIZE, 0, out, da, n)  # dispatch_elementwise, :65-86
    np.testing.assert_allclose(out.cpu().numpy(), oracle.gelu(a), rtol=5e-6, atol=5e-7)
    one = torch.tensor([1.0, -1.0], device="cuda")
    g = torch.zeros(2, device="cuda")
    module.launch("gelu_kernel", grid_for(2), BLOCK_SIZE, 0, g, one, 2)
    assert abs(g[0].item() - 0.8412) < 0.01 and abs(g[1].item() + 0.1588) < 0.01  # runtime_kernels.zig:325-335


def test_gather_transpose_adaln(module):
    rng = np.random.default_rng(4)
    table = rng.standard_normal((50, 24)).astype(np.float32)
    idx = rng.integers(0, 50, size=17).astype(np.int32)
    out = torch.zeros(17, 24, device="cuda")
    module.launch("gather_kernel", grid_for(17 * 24), BLOCK_SIZE, 0, out, dev(table), dev(idx), 17, 24)  # :207-234
    assert np.array_equal(out.cpu().numpy(), table[idx])
    x = rng.standard_normal((13, 37)).astype(np.float32)
    t = torch.zeros(37, 13, device="cuda")
    module.launch("transpose_2d_kernel", grid_for(13 * 37), BLOCK_SIZE, 0, t, dev(x), 13, 37)  # :147-170
    assert np.array_equal(t.cpu().numpy(), x.T)
    B, S, D = 3, 5, 16
    norm = rng.standard_normal((B, S, D)).astype(np.float32)
    scale, beta = rng.standard_normal((B, D)).astype(np.float32), rng.standard_normal((B, D)).astype(np.float32)
    o = torch.zeros(B, S, D, device="cuda")
    module.launch("modulate_adaln_kernel", grid_for(B * S * D), BLOCK_SIZE, 0, o, dev(norm), dev(scale), dev(beta), B, S, D)
    np.testing.assert_allclose(o.cpu().numpy(), norm * scale[:, None, :] + beta[:, None, :], rtol=1e-6, atol=1e-6)


def test_reductions(module):
    rng = np.random.default_rng(6)
    for rows, cols in ((1, 1), (4, 33), (5, 1500)):
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        block = next_pow2(min(cols, 1024))
        out = torch.zeros(rows, device="cuda")
        module.launch("reduction_sum_rows_kernel", rows, block, block * 4, out, dev(x), rows, cols)  # :996-1021
        np.testing.assert_allclose(out.cpu().numpy(), x.astype(np.float64).sum(axis=1), rtol=1e-5, atol=1e-4)
        oc = torch.zeros(cols, device="cuda")
        module.launch("reduction_sum_cols_kernel", grid_for(cols), BLOCK_SIZE, 0, oc, dev(x), rows, cols)  # :1023-1047
        np.testing.assert_allclose(oc.cpu().numpy(), x.astype(np.float64).sum(axis=0), rtol=1e-5, atol=1e-4)
    for n in (1, 7, 300, 1024, 5000):  # one block of next_pow2(min(n, 1024)) threads, :1049-1069; adds into out[0]
        x = rng.standard_normal(n).astype(np.float32)
        block = next_pow2(min(n, 1024))
        out = torch.full((1,), 2.0, device="cuda")
        module.launch("reduction_sum_1d_kernel", 1, block, block * 4, out, dev(x), n)
        np.testing.assert_allclose(out.item(), 2.0 + x.astype(np.float64).sum(), rtol=1e-5, atol=1e-4)
