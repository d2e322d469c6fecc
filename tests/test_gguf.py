"""GGUF container: the reader against zig-nn's own parser test and error rules, the writer through
round trips of the synthetic models (no GPU)."""
import struct

import numpy as np
import pytest

import zignn_b200  # noqa: F401
from zignn_b200 import ggml, gguf, hostmodel

TINY_GPT2 = dict(vocab=97, embed=64, head=2, layer=2, ctx=16, ffn=128)
TINY_GEMMA = dict(vocab=160, embed=64, head=2, head_kv=1, head_dim=32, layer=3, ctx=24, ffn=96,
                  rope_base=1000000.0, sliding_window=8, rms_eps=1e-6, global_every=3)


def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _minimal(version=3, magic=gguf.GGUF_MAGIC, n_dims=1, value_type=gguf.T_UINT32):
    """The hand-made file of zig-nn's parser test (src/gguf/gguf.zig:580-620): one uint32 metadata pair
    test.key = 42, one f32 tensor "w" of 4 elements at offset 0, data padded to 32 bytes."""
    b = struct.pack("<IIQQ", magic, version, 1, 1)
    b += _s("test.key") + struct.pack("<II", value_type, 42)
    b += _s("w") + struct.pack("<I", n_dims) + struct.pack("<Q", 4) * n_dims + struct.pack("<IQ", 0, 0)
    b += b"\0" * ((len(b) + 31) // 32 * 32 - len(b))
    return b + np.array([1.0, 2.0, 3.0, 4.0], dtype="<f4").tobytes()


def test_parse_minimal_file_like_the_reference_test():
    # expectations of src/gguf/gguf.zig:627-648
    f = gguf.parse_from_buffer(_minimal(), "test.gguf")
    assert f.version == 3
    assert len(f.metadata) == 1 and len(f.tensors) == 1
    assert f.get_metadata_u32("test.key") == 42
    assert f.get_metadata_u64("test.key") is None and f.get_metadata_string("test.key") is None
    t = f.get_tensor_info("w")
    assert t.n_dims == 1 and t.dimensions[0] == 4 and t.type_ == ggml.F32
    assert f.alignment == 32 and f.data_offset % 32 == 0
    data = f.load_tensor_f32("w")
    assert data.dtype == np.float32 and data.tolist() == [1.0, 2.0, 3.0, 4.0]
    r = f.get_tensor_raw_bytes("w")
    assert (r.out_dim, r.in_dim, r.n_elem) == (4, 1, 4)  # 1-D: out_dim = dims[0], in_dim = 1


def test_reader_errors():
    with pytest.raises(gguf.InvalidMagic):
        gguf.parse_from_buffer(_minimal(magic=0x46554746))
    for v in (1, 4):  # only versions 2 and 3 (gguf.zig:339)
        with pytest.raises(gguf.UnsupportedVersion):
            gguf.parse_from_buffer(_minimal(version=v))
    assert gguf.parse_from_buffer(_minimal(version=2)).version == 2
    with pytest.raises(gguf.TooManyDimensions):
        gguf.parse_from_buffer(_minimal(n_dims=5))
    with pytest.raises(gguf.UnsupportedValueType):
        gguf.parse_from_buffer(_minimal(value_type=13))
    good = _minimal()
    for cut in (3, 10, 30, 50, 70):  # inside the header, the key, the value, the tensor info
        with pytest.raises(gguf.UnexpectedEof):
            gguf.parse_from_buffer(good[:cut])
    f = gguf.parse_from_buffer(good[:-4])  # tensor data cut short: found when the tensor is asked for
    with pytest.raises(gguf.UnexpectedEof):
        f.get_tensor_raw_bytes("w")
    with pytest.raises(gguf.TensorNotFound):
        f.get_tensor_raw_bytes("nope")


def test_metadata_value_types_and_alignment(tmp_path):
    meta = [("a.u8", gguf.T_UINT8, 200), ("a.i8", gguf.T_INT8, -5), ("a.u16", gguf.T_UINT16, 60000),
            ("a.i16", gguf.T_INT16, -30000), ("a.i32", gguf.T_INT32, -7), ("a.f32", gguf.T_FLOAT32, 0.5),
            ("a.bool", gguf.T_BOOL, True), ("a.str", gguf.T_STRING, "héllo"), ("a.u64", gguf.T_UINT64, 1 << 40),
            ("a.i64", gguf.T_INT64, -(1 << 40)), ("a.f64", gguf.T_FLOAT64, 0.25),
            ("a.strs", gguf.T_ARRAY, (gguf.T_STRING, ["x", "", "tok en"])),
            ("a.ints", gguf.T_ARRAY, (gguf.T_INT32, [1, -2, 3])),
            ("general.alignment", gguf.T_UINT32, 64)]
    w = np.arange(8, dtype=np.float32)
    h = np.arange(6, dtype=np.float16)
    path = str(tmp_path / "m.gguf")
    gguf.write(path, meta, [("w", (8,), ggml.F32, w), ("h", (3, 2), ggml.F16, h)], alignment=64)
    f = gguf.parse(path)
    assert f.alignment == 64 and f.data_offset % 64 == 0
    for key, _, v in meta[:11]:
        assert f.get_metadata(key) == v
    assert f.get_array_strings("a.strs") == ["x", "", "tok en"]
    assert f.get_metadata("a.ints").values() == [1, -2, 3]
    assert f.get_array_strings("a.ints") is None
    assert [t.offset % 64 for t in f.tensors] == [0, 0]
    assert np.array_equal(f.load_tensor_f32("w"), w)
    assert np.array_equal(f.load_tensor_f32("h"), h.astype(np.float32))
    # stored (cols = 3, rows = 2) -> row-major (rows, cols) (gguf.zig:196-221)
    assert np.array_equal(f.load_tensor_f32_transposed("h"), h.astype(np.float32).reshape(3, 2).T.reshape(-1))
    r = f.get_tensor_raw_bytes("h")
    assert (r.out_dim, r.in_dim) == (2, 3)  # 2-D: out_dim = dims[1], in_dim = dims[0]


def test_writer_rejects_wrong_sizes(tmp_path):
    with pytest.raises(gguf.GGUFError):
        gguf.write(str(tmp_path / "x.gguf"), [], [("w", (64,), ggml.Q4_0, np.zeros(35, np.uint8))])
    with pytest.raises(gguf.GGUFError):
        gguf.write(str(tmp_path / "y.gguf"), [], [("w", (64,), 99, np.zeros(36, np.uint8))])


def _same(a, b):
    if isinstance(a, hostmodel.QuantTensor):
        return (isinstance(b, hostmodel.QuantTensor) and (a.qtype, a.out_dim, a.in_dim) == (b.qtype, b.out_dim, b.in_dim)
                and np.array_equal(a.raw, b.raw))
    return a.dtype == b.dtype and np.array_equal(np.asarray(a).reshape(-1), np.asarray(b).reshape(-1))


def test_gpt2_round_trip_uses_the_reference_tensor_names(tmp_path):
    m = hostmodel.Gpt2Host.synthetic(cfg=TINY_GPT2, qtype=ggml.Q4_0, seed=5).randomize_small_params()
    path = str(tmp_path / "gpt2.gguf")
    m.to_gguf(path)
    f = gguf.parse(path)
    # the names gpt2.zig:77-82,134-181 loads, dims innermost-first
    for name in ("token_embd.weight", "position_embd.weight", "output_norm.weight", "output_norm.bias",
                 "blk.0.attn_norm.weight", "blk.0.attn_norm.bias", "blk.1.attn_qkv.weight", "blk.1.attn_qkv.bias",
                 "blk.0.attn_output.weight", "blk.0.attn_output.bias", "blk.0.ffn_norm.weight",
                 "blk.0.ffn_norm.bias", "blk.0.ffn_up.weight", "blk.0.ffn_up.bias", "blk.1.ffn_down.weight",
                 "blk.1.ffn_down.bias"):
        assert f.get_tensor_info(name) is not None, name
    assert f.get_tensor_info("token_embd.weight").dimensions == (64, 97)
    q = f.get_tensor_raw_bytes("blk.0.attn_qkv.weight")
    assert (q.type_, q.out_dim, q.in_dim) == (ggml.Q4_0, 192, 64)
    assert all(t.offset % 32 == 0 for t in f.tensors)
    assert f.get_metadata_string("general.architecture") == "gpt2"
    back = hostmodel.Gpt2Host.from_gguf(path)
    assert back.cfg == m.cfg
    for name in ("wte", "wpe", "ln_f_weight", "ln_f_bias"):
        assert _same(getattr(m, name), getattr(back, name)), name
    for a, b in zip(m.blocks, back.blocks):
        assert a.keys() == b.keys()
        for k in a:
            assert _same(a[k], b[k]), k
    back.weights_struct()  # the C structs can be built from the mapped file


@pytest.mark.parametrize("qtype,down,embd", [(ggml.Q8_0, None, None), (ggml.Q4_0, ggml.Q4_1, ggml.Q8_0)])
def test_gemma3_round_trip_uses_the_reference_tensor_names(tmp_path, qtype, down, embd):
    m = hostmodel.Gemma3Host.synthetic(cfg=TINY_GEMMA, qtype=qtype, seed=6, down_qtype=down,
                                       embd_qtype=embd).randomize_small_params()
    path = str(tmp_path / "gemma.gguf")
    m.to_gguf(path)
    f = gguf.parse(path)
    for suffix in ("attn_norm", "post_attention_norm", "attn_q", "attn_k", "attn_v", "attn_output", "attn_q_norm",
                   "attn_k_norm", "ffn_norm", "post_ffw_norm", "ffn_gate", "ffn_up", "ffn_down"):
        assert f.get_tensor_info("blk.2.%s.weight" % suffix) is not None, suffix  # gemma3.zig:174-226
    e = f.get_tensor_raw_bytes("token_embd.weight")
    assert (e.type_, e.out_dim, e.in_dim) == (embd or qtype, 160, 64)
    d = f.get_tensor_raw_bytes("blk.0.ffn_down.weight")
    assert (d.type_, d.out_dim, d.in_dim) == (down or qtype, 64, 96)
    back = hostmodel.Gemma3Host.from_gguf(path)
    assert back.cfg == pytest.approx(m.cfg)
    assert _same(m.token_embd, back.token_embd) and _same(m.output_norm_weight, back.output_norm_weight)
    for a, b in zip(m.blocks, back.blocks):
        for k in a:
            assert _same(a[k], b[k]), k
    back.weights_struct()
