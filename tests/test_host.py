"""Host-side logic that needs no GPU: block geometry, encoders, struct layouts, and that the
C-ABI library loads and exports every symbol include/zq.h declares."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

import zignn_b200
from zignn_b200 import ggml, hostmodel, structs

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tensor_bytes_matches_reference_table():
    # src/gguf/dequant.zig:687-694
    assert ggml.tensor_bytes(ggml.F32, 32) == 128
    assert ggml.tensor_bytes(ggml.F16, 32) == 64
    assert ggml.tensor_bytes(ggml.Q4_0, 32) == 18
    assert ggml.tensor_bytes(ggml.Q4_0, 64) == 36
    assert ggml.tensor_bytes(ggml.Q4_1, 32) == 20
    assert ggml.tensor_bytes(ggml.Q8_0, 32) == 34
    assert ggml.tensor_bytes(99, 32) == 0


@pytest.mark.parametrize("qtype", [ggml.Q4_0, ggml.Q4_1, ggml.Q8_0])
def test_encoders_match_oracle(oracle, qtype):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(32 * 500) * 0.02).astype(np.float32)
    x[:32] = 0.0          # all-zero block
    x[32:64] = 0.125      # constant block
    x[64:96] *= 1e4       # large values
    a = oracle.quantize(qtype, x)
    b = ggml.quantize(qtype, torch.from_numpy(x)).numpy()
    assert np.array_equal(a, b)


def test_unsupported_encoder_type():
    with pytest.raises(ValueError):
        ggml.quantize(ggml.F16, torch.zeros(32))


def test_header_symbols_exported_and_bound():
    from zignn_b200 import _lib
    hdr = open(os.path.join(REPO, "include", "zq.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(zq_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) > 40
    lib = _lib.load()
    for name in sorted(declared):
        assert hasattr(lib, name), "libzq.so does not export %s" % name
        assert name in _lib.SIGNATURES, "no ctypes signature for %s" % name
    assert set(_lib.SIGNATURES) == declared


def test_no_compute_entry_points_without_args():
    from zignn_b200 import _lib
    lib = _lib.load()
    assert lib.zq_abi_version() == 1
    assert lib.zq_status_string(0) == b"ok"
    assert lib.zq_tensor_bytes(2, 64) == 36
    assert lib.zq_block_size(8) == 32 and lib.zq_bytes_per_block(3) == 20
    # argument validation happens before any CUDA call
    h = C.c_void_p()
    assert lib.zq_weight_upload(None, 2, 4, 32, None, C.byref(h)) == 1          # null host pointer
    buf = (C.c_uint8 * 64)()
    assert lib.zq_weight_upload(buf, 6, 1, 32, None, C.byref(h)) == 2           # q5_0: unsupported
    assert lib.zq_weight_upload(buf, 2, 1, 48, None, C.byref(h)) == 1           # in_dim % 32 != 0
    assert lib.zq_matmul(None, None, None, 1, 0, None, None, 0, None) == 1


def test_rope_freqs_host_matches_oracle(oracle):
    from zignn_b200 import _lib
    f = np.empty(128, np.float32)
    assert _lib.load().zq_rope_freqs_host(256, 1000000.0, f.ctypes.data_as(C.c_void_p)) == 0
    assert np.array_equal(f, oracle.rope_freqs(256, 1000000.0))


def test_struct_sizes_match_c_layout():
    assert C.sizeof(structs.TensorRef) == 24
    assert C.sizeof(structs.Epilogue) == 32
    assert C.sizeof(structs.Gpt2Config) == 24
    assert C.sizeof(structs.Gemma3Config) == 48
    assert C.sizeof(structs.Gpt2Block) == 8 * 8 + 4 * 24
    assert C.sizeof(structs.Gemma3Block) == 6 * 8 + 7 * 24


def test_synthetic_models_are_seeded():
    cfg = dict(vocab=64, embed=32, head=2, layer=1, ctx=8, ffn=64)
    a = hostmodel.Gpt2Host.synthetic(cfg, seed=42)
    b = hostmodel.Gpt2Host.synthetic(cfg, seed=42)
    c = hostmodel.Gpt2Host.synthetic(cfg, seed=43)
    assert np.array_equal(a.wte, b.wte) and not np.array_equal(a.wte, c.wte)
    assert np.array_equal(a.blocks[0]["mlp_fc_weight"].raw, b.blocks[0]["mlp_fc_weight"].raw)
    assert a.blocks[0]["attn_qkv_weight"].raw.size == ggml.tensor_bytes(ggml.Q4_0, 96 * 32)
