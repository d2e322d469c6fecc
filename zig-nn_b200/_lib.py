"""Loads libzq.so and declares the C ABI of include/zq.h for ctypes.

There is no fallback: if the shared library is missing or fails to load, importing this
module raises, and every operation of the package is unavailable.
"""
import ctypes as C
import os

from . import structs as S

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libzq.so")

STATUS_NAMES = {
    0: "ZQ_OK", 1: "ZQ_ERR_BAD_ARG", 2: "ZQ_ERR_UNSUPPORTED", 3: "ZQ_ERR_CUDA", 4: "ZQ_ERR_NO_MEM",
    5: "ZQ_ERR_LIMIT", 6: "ZQ_ERR_SEQUENCE", 7: "ZQ_ERR_TIMEOUT", 8: "ZQ_ERR_PEER",
}

vp, sz, i, u32, f = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_float
P = C.POINTER

# name -> (restype, argtypes); one entry per function declared in include/zq.h
SIGNATURES = {
    "zq_status_string": (C.c_char_p, [i]),
    "zq_last_cuda_error": (i, []),
    "zq_abi_version": (i, []),
    "zq_device_error": (i, [P(u32), i]),
    "zq_device_check": (i, [i]),
    "zq_set_wait_limit": (i, [u32]),
    "zq_block_size": (sz, [i]),
    "zq_bytes_per_block": (sz, [i]),
    "zq_tensor_bytes": (sz, [i, sz]),
    "zq_weight_upload": (i, [vp, i, u32, u32, vp, P(vp)]),
    "zq_weight_from_device": (i, [vp, i, u32, u32, vp, P(vp)]),
    "zq_weight_free": (i, [vp]),
    "zq_weight_info": (i, [vp, P(i), P(u32), P(u32)]),
    "zq_weight_device_bytes": (sz, [vp]),
    "zq_weight_download_raw": (i, [vp, vp, vp]),
    "zq_dequantize": (i, [vp, vp, vp]),
    "zq_dequant_rows_scaled": (i, [vp, vp, u32, f, vp, vp]),
    "zq_matmul_workspace_bytes": (sz, [vp, u32, i]),
    "zq_matmul": (i, [vp, vp, vp, u32, i, P(S.Epilogue), vp, sz, vp]),
    "zq_matmul_q8_static": (i, [vp, vp, vp, u32, P(S.Epilogue), vp]),
    "zq_matmul_transposed_workspace_bytes": (sz, [vp, u32]),
    "zq_matmul_transposed": (i, [vp, vp, vp, u32, i, vp, sz, vp]),
    "zq_quantize_rows_q8": (i, [vp, u32, u32, vp, vp, vp, vp]),
    "zq_matvec_f32": (i, [vp, vp, vp, u32, u32, vp]),
    "zq_argmax": (i, [vp, u32, vp, vp]),
    "zq_peer_gather": (i, [vp, vp, u32, u32, C.c_size_t, C.c_size_t, u32, vp]),
    "zq_peer_gather_step": (i, [vp, vp, vp, u32, u32, C.c_size_t, C.c_size_t, vp, vp]),
    "zq_peer_gather_cols_step": (i, [vp, vp, vp, u32, u32, vp, u32, C.c_size_t, C.c_size_t, u32, vp, vp]),
    "zq_matmul_gather": (i, [vp, vp, vp, vp, vp, vp, u32, u32, u32, vp, vp]),
    "zq_matmul_gather_tagged": (i, [vp, vp, vp, vp, vp, vp, vp, u32, u32, vp, vp]),
    "zq_set_cluster_launch": (i, [C.c_int]),
    "zq_matmul_argmax": (i, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, vp, vp]),
    "zq_rms_norm": (i, [vp, vp, vp, u32, u32, f, vp]),
    "zq_rms_norm_residual": (i, [vp, vp, vp, u32, u32, f, vp]),
    "zq_rms_norm_in_place": (i, [vp, vp, u32, u32, f, vp]),
    "zq_rope": (i, [vp, vp, u32, u32, f, vp]),
    "zq_rope_freqs_host": (i, [u32, f, vp]),
    "zq_gelu_mul": (i, [vp, vp, sz, vp]),
    "zq_write_kv_cache": (i, [vp, vp, vp, vp, u32, u32, vp]),
    "zq_attention_decode": (i, [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, i, vp]),
    "zq_softmax": (i, [vp, u32, u32, vp]),
    "zq_softmax_out": (i, [vp, vp, u32, u32, vp]),
    "zq_layer_norm": (i, [vp, vp, vp, vp, u32, u32, f, vp]),
    "zq_gelu": (i, [vp, vp, sz, vp]),
    "zq_add_broadcast": (i, [vp, vp, vp, sz, sz, vp]),
    "zq_mul_broadcast": (i, [vp, vp, vp, sz, sz, vp]),
    "zq_gather": (i, [vp, vp, vp, u32, u32, vp]),
    "zq_scale": (i, [vp, vp, f, sz, vp]),
    "zq_copy_f32": (i, [vp, vp, sz, vp]),
    "zq_gpt2_create": (i, [P(S.Gpt2Config), P(S.Gpt2Weights), vp, P(vp)]),
    "zq_gpt2_free": (i, [vp]),
    "zq_gpt2_reset_cache": (i, [vp]),
    "zq_gpt2_seq_len": (i, [vp, P(u32)]),
    "zq_gpt2_prefill": (i, [vp, vp, u32, vp, P(vp)]),
    "zq_gpt2_decode_next": (i, [vp, u32, vp, P(vp)]),
    "zq_gpt2_decode_greedy": (i, [vp, u32, u32, vp, vp]),
    "zq_gemma3_create": (i, [P(S.Gemma3Config), P(S.Gemma3Weights), vp, P(vp)]),
    "zq_gemma3_free": (i, [vp]),
    "zq_gemma3_reset_cache": (i, [vp]),
    "zq_gemma3_seq_len": (i, [vp, P(u32)]),
    "zq_gemma3_prefill": (i, [vp, vp, u32, vp, P(vp)]),
    "zq_gemma3_decode_next": (i, [vp, u32, vp, P(vp)]),
    "zq_gemma3_decode_greedy": (i, [vp, u32, u32, vp, vp]),
    "zq_gemma3_create_batch": (i, [P(S.Gemma3Config), P(S.Gemma3Weights), u32, vp, P(vp)]),
    "zq_gemma3_prefill_seq": (i, [vp, u32, vp, u32, vp, P(vp)]),
    "zq_gemma3_decode_next_batch": (i, [vp, vp, vp, P(vp)]),
    "zq_gemma3_seq_len_of": (i, [vp, u32, P(u32)]),
    "zq_gemma3_set_decode_mode": (i, [vp, i]),
    "zq_gpt2_set_decode_mode": (i, [vp, i]),
    "zq_gpt2_decode_mode": (i, [vp, P(i)]),
    "zq_gemma3_decode_mode": (i, [vp, P(i)]),
    "zq_gemma3_profile_step": (i, [vp, u32, vp, vp, u32, P(u32)]),
}


class ZqError(RuntimeError):
    def __init__(self, status, where=""):
        self.status = status
        name = STATUS_NAMES.get(status, "status %d" % status)
        extra = ""
        if status == 3 and _lib is not None:
            extra = " (cudaError %d)" % _lib.zq_last_cuda_error()
        super().__init__("%s failed: %s%s" % (where or "libzq call", name, extra))


_lib = None


def load():
    """Return the loaded library; raises if libzq.so is not there."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libzq.so not found at %s — build it with `python zig-nn_b200/build.py`. "
            "There is no CPU fallback." % LIB_PATH
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the library is stale
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status, where=""):
    if status != 0:
        raise ZqError(status, where)


def device_error(clear=True):
    """The code a kernel's bounded device-side wait left behind when it ran out (0 = none): the four
    characters of a tag such as 'GATH' (peer gather), 'GBAR' (grid barrier of the persistent decode
    kernel) packed into an integer. clear=True resets the word."""
    v = C.c_uint()
    check(load().zq_device_error(C.byref(v), int(bool(clear))), "zq_device_error")
    return v.value
