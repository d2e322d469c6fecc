"""ctypes binding of the CPU oracle (libzq_oracle.so).

Test infrastructure: imported only by tests/, by __graft_entry__.smoke() and by the CPU
baseline / reference legs of bench.py. The shipped package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_here = os.path.dirname(os.path.abspath(__file__))
_repo = os.path.dirname(_here)

import sys

if _repo not in sys.path:
    sys.path.insert(0, _repo)
from zignn_b200 import structs as S  # noqa: E402  (struct layouts shared with include/zq.h)

F32 = 0
F16 = 1
Q4_0 = 2
Q4_1 = 3
Q8_0 = 8


class Q8Block(C.Structure):
    _fields_ = [("q", C.c_int8 * 32), ("scale", C.c_float), ("sum", C.c_int32)]


def build(arch="x86-64-v3", out=None):
    """Compile the oracle with make; returns the path of the shared library."""
    out = out or os.path.join(_here, "libzq_oracle.so")
    subprocess.run(
        ["make", "-s", "-C", _here, f"ARCH={arch}", f"OUT={out}"], check=True, capture_output=True
    )
    return out


def _load(path=None):
    path = path or os.path.join(_here, "libzq_oracle.so")
    if not os.path.exists(path):
        build(out=path)
    lib = C.CDLL(path)
    vp, sz, i, u32, f = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_float
    sig = {
        "zqo_block_size": (sz, [i]),
        "zqo_bytes_per_block": (sz, [i]),
        "zqo_tensor_bytes": (sz, [i, sz]),
        "zqo_f16_to_f32": (f, [C.c_uint16]),
        "zqo_f32_to_f16": (C.c_uint16, [f]),
        "zqo_quantize": (i, [i, vp, vp, sz]),
        "zqo_dequantize": (i, [i, vp, vp, sz]),
        "zqo_dot_f32": (f, [i, vp, vp, sz]),
        "zqo_matmul_f32": (i, [i, vp, vp, vp, sz, sz, i]),
        "zqo_quantize_row_q8": (None, [vp, vp, sz]),
        "zqo_dot_q8": (f, [i, vp, vp, sz]),
        "zqo_matmul_q8": (i, [i, vp, vp, vp, sz, sz, i, i]),
        "zqo_linear": (i, [i, vp, vp, vp, sz, sz, sz, i, i]),
        "zqo_matmul_transposed": (i, [i, vp, vp, vp, sz, sz, sz, i, i]),
        "zqo_layer_norm_rows": (None, [vp, vp, vp, vp, sz, sz]),
        "zqo_layer_norm_forward": (None, [vp, vp, vp, vp, sz, sz, f]),
        "zqo_rms_norm_rows": (None, [vp, vp, vp, sz, sz, f]),
        "zqo_rms_norm_in_place": (None, [vp, vp, sz, f]),
        "zqo_gelu_in_place": (None, [vp, sz]),
        "zqo_softmax_gpt2": (None, [vp, sz]),
        "zqo_softmax_gemma": (None, [vp, sz]),
        "zqo_softmax_forward": (None, [vp, sz, sz]),
        "zqo_rope_freqs": (None, [sz, f, vp]),
        "zqo_rope": (None, [vp, sz, vp, sz]),
        "zqo_argmax": (u32, [vp, sz]),
        "zqo_cached_attention": (None, [vp, vp, vp, vp, vp, sz, sz, sz, sz]),
        "zqo_causal_self_attention": (None, [vp, vp, vp, sz, sz, sz, sz]),
        "zqo_gqa_cached_attention": (None, [vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, sz]),
        "zqo_gqa_causal_attention_prefill": (None, [vp, vp, vp, vp, sz, sz, sz, sz, sz, sz]),
        "zqo_gpt2_create": (vp, [vp, vp, i]),
        "zqo_gpt2_free": (None, [vp]),
        "zqo_gpt2_prefill": (i, [vp, vp, sz, vp]),
        "zqo_gpt2_decode_next": (i, [vp, u32, vp]),
        "zqo_gemma3_create": (vp, [vp, vp, i]),
        "zqo_gemma3_free": (None, [vp]),
        "zqo_gemma3_prefill": (i, [vp, vp, sz, vp]),
        "zqo_gemma3_decode_next": (i, [vp, u32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_lib = None
_lib_path = None


def lib(path=None):
    global _lib, _lib_path
    if _lib is None or (path is not None and path != _lib_path):
        _lib = _load(path)
        _lib_path = path
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def tensor_bytes(t, n):
    return lib().zqo_tensor_bytes(t, n)


def quantize(t, x):
    """x: float32 array with last dim % 32 == 0 -> uint8 array of GGUF bytes (flat)."""
    x = _f32(x)
    out = np.empty(tensor_bytes(t, x.size), dtype=np.uint8)
    rc = lib().zqo_quantize(t, _p(x), _p(out), x.size)
    if rc:
        raise ValueError("unsupported quant type %d" % t)
    return out


def dequantize(t, raw, n):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    rc = lib().zqo_dequantize(t, _p(raw), _p(out), n)
    if rc:
        raise ValueError("UnsupportedQuantType")
    return out


def dot_f32(t, row, x):
    row = np.ascontiguousarray(row, dtype=np.uint8)
    x = _f32(x)
    return float(lib().zqo_dot_f32(t, _p(row), _p(x), x.size))


def matmul_f32(t, w, x, out_dim, in_dim, n_threads=1):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = _f32(x)
    y = np.empty(out_dim, dtype=np.float32)
    rc = lib().zqo_matmul_f32(t, _p(w), _p(x), _p(y), out_dim, in_dim, n_threads)
    if rc:
        raise ValueError("unsupported type")
    return y


def quantize_row_q8(x):
    x = _f32(x)
    nb = x.size // 32
    blocks = (Q8Block * nb)()
    lib().zqo_quantize_row_q8(_p(x), C.cast(blocks, C.c_void_p), x.size)
    q = np.array([list(b.q) for b in blocks], dtype=np.int8).reshape(nb, 32)
    scale = np.array([b.scale for b in blocks], dtype=np.float32)
    s = np.array([b.sum for b in blocks], dtype=np.int32)
    return q, scale, s, blocks


def dot_q8(t, row, blocks):
    row = np.ascontiguousarray(row, dtype=np.uint8)
    return float(lib().zqo_dot_q8(t, _p(row), C.cast(blocks, C.c_void_p), len(blocks)))


def matmul_q8(t, w, x, out_dim, in_dim, n_threads=1, allow_long=False):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = _f32(x)
    y = np.empty(out_dim, dtype=np.float32)
    rc = lib().zqo_matmul_q8(t, _p(w), _p(x), _p(y), out_dim, in_dim, n_threads, int(allow_long))
    if rc == 2:
        raise ValueError("in_dim exceeds the reference thread pool's 8192-element buffer")
    if rc:
        raise ValueError("unsupported type")
    return y


def linear(t, w, x, out_dim, in_dim, act_mode=0, n_threads=1):
    """x [m, in_dim] -> y [m, out_dim]; act_mode 0 = f32 activations, 1 = Q8 activations."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = _f32(x).reshape(-1, in_dim)
    y = np.empty((x.shape[0], out_dim), dtype=np.float32)
    rc = lib().zqo_linear(t, _p(w), _p(x), _p(y), x.shape[0], out_dim, in_dim, act_mode, n_threads)
    if rc:
        raise ValueError("zqo_linear failed: %d" % rc)
    return y


def matmul_transposed(t, w, grad_out, out_dim, in_dim, grad_x=None, n_threads=1):
    """grad_x [m, in_dim] (+)= grad_out [m, out_dim] . W; grad_x given = accumulate into a copy of it."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    g = _f32(grad_out).reshape(-1, out_dim)
    acc = grad_x is not None
    o = _f32(grad_x).reshape(-1, in_dim).copy() if acc else np.empty((g.shape[0], in_dim), dtype=np.float32)
    rc = lib().zqo_matmul_transposed(t, _p(w), _p(g), _p(o), g.shape[0], out_dim, in_dim, int(acc), n_threads)
    if rc:
        raise ValueError("UnsupportedQuantType")
    return o


def layer_norm_rows(x, w, b):
    x = _f32(x)
    rows, dim = x.reshape(-1, x.shape[-1]).shape
    out = np.empty_like(x)
    lib().zqo_layer_norm_rows(_p(x), _p(_f32(w)), _p(_f32(b)), _p(out), rows, dim)
    return out


def layer_norm_forward(x, gamma, beta, eps):
    x = _f32(x)
    rows, dim = x.reshape(-1, x.shape[-1]).shape
    out = np.empty_like(x)
    lib().zqo_layer_norm_forward(_p(x), _p(out), _p(_f32(gamma)), _p(_f32(beta)), rows, dim, eps)
    return out


def rms_norm_rows(x, w, eps):
    x = _f32(x)
    rows, dim = x.reshape(-1, x.shape[-1]).shape
    out = np.empty_like(x)
    lib().zqo_rms_norm_rows(_p(x), _p(_f32(w)), _p(out), rows, dim, eps)
    return out


def rms_norm_in_place(x, w, eps):
    x = _f32(x).copy()
    lib().zqo_rms_norm_in_place(_p(x), _p(_f32(w)), x.size, eps)
    return x


def gelu(x):
    x = _f32(x).copy()
    lib().zqo_gelu_in_place(_p(x), x.size)
    return x


def softmax_gpt2(x):
    x = _f32(x).copy()
    lib().zqo_softmax_gpt2(_p(x), x.size)
    return x


def softmax_gemma(x):
    x = _f32(x).copy()
    lib().zqo_softmax_gemma(_p(x), x.size)
    return x


def softmax_forward(x):
    x = _f32(x).copy()
    rows, cols = x.reshape(-1, x.shape[-1]).shape
    lib().zqo_softmax_forward(_p(x), rows, cols)
    return x


def rope_freqs(head_dim, base):
    f = np.empty(head_dim // 2, dtype=np.float32)
    lib().zqo_rope_freqs(head_dim, base, _p(f))
    return f


def rope(x, pos, freqs):
    x = _f32(x).copy()
    freqs = _f32(freqs)
    lib().zqo_rope(_p(x), pos, _p(freqs), freqs.size)
    return x


def argmax(logits):
    logits = _f32(logits)
    return int(lib().zqo_argmax(_p(logits), logits.size))


def cached_attention(q, k_cache, v_cache, kv_len, n_head, head_dim):
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    embed = n_head * head_dim
    out = np.empty(embed, dtype=np.float32)
    scores = np.empty(kv_len, dtype=np.float32)
    lib().zqo_cached_attention(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(scores), kv_len, n_head, head_dim, embed
    )
    return out


def causal_self_attention(qkv, seq_len, n_head, head_dim):
    qkv = _f32(qkv)
    embed = n_head * head_dim
    out = np.empty((seq_len, embed), dtype=np.float32)
    scores = np.empty(seq_len * seq_len, dtype=np.float32)
    lib().zqo_causal_self_attention(_p(qkv), _p(out), _p(scores), seq_len, n_head, head_dim, embed)
    return out


def gqa_cached_attention(q, k_cache, v_cache, kv_start, kv_end, n_head, head_dim, kv_dim):
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    q_dim = n_head * head_dim
    out = np.empty(q_dim, dtype=np.float32)
    scores = np.empty(max(1, kv_end - kv_start), dtype=np.float32)
    lib().zqo_gqa_cached_attention(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(scores), kv_start, kv_end, n_head, head_dim,
        q_dim, kv_dim,
    )
    return out


def gqa_causal_attention_prefill(q, k_cache, v_cache, seq_len, n_head, head_dim, kv_dim, window):
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    q_dim = n_head * head_dim
    out = np.empty((seq_len, q_dim), dtype=np.float32)
    lib().zqo_gqa_causal_attention_prefill(
        _p(q), _p(k_cache), _p(v_cache), _p(out), seq_len, n_head, head_dim, q_dim, kv_dim, window
    )
    return out


class _Model:
    """Common driver of the two oracle models. `weights` is a zignn_b200 host-model object that
    keeps the numpy arrays alive and exposes .config_struct() / .weights_struct()."""

    _create = _free = _prefill = _decode = None

    def __init__(self, host_model, n_threads=1):
        self._host = host_model
        self._cfg = host_model.config_struct()
        self._w = host_model.weights_struct()
        L = lib()
        self._h = getattr(L, self._create)(C.byref(self._cfg), C.byref(self._w), n_threads)
        self.vocab = self._cfg.vocab

    def _logits(self, ptr):
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(self.vocab,)).copy()

    def prefill(self, tokens):
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        ptr = C.c_void_p()
        rc = getattr(lib(), self._prefill)(self._h, _p(toks), toks.size, C.byref(ptr))
        if rc:
            raise RuntimeError("oracle prefill failed: status %d" % rc)
        return self._logits(ptr)

    def decode_next(self, token):
        ptr = C.c_void_p()
        rc = getattr(lib(), self._decode)(self._h, int(token), C.byref(ptr))
        if rc:
            raise RuntimeError("oracle decode_next failed: status %d" % rc)
        return self._logits(ptr)

    def greedy(self, prompt, n_steps):
        """prefill + n_steps greedy tokens; returns (tokens, list of logits per step)."""
        logits = self.prefill(prompt)
        toks, all_logits = [], []
        for _ in range(n_steps):
            t = argmax(logits)
            toks.append(t)
            all_logits.append(logits)
            logits = self.decode_next(t)
        return toks, all_logits

    def close(self):
        if self._h:
            getattr(lib(), self._free)(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Gpt2(_Model):
    _create, _free = "zqo_gpt2_create", "zqo_gpt2_free"
    _prefill, _decode = "zqo_gpt2_prefill", "zqo_gpt2_decode_next"


class Gemma3(_Model):
    _create, _free = "zqo_gemma3_create", "zqo_gemma3_free"
    _prefill, _decode = "zqo_gemma3_prefill", "zqo_gemma3_decode_next"
