"""ctypes mirrors of the structs in include/zq.h."""
import ctypes as C


class Epilogue(C.Structure):
    _fields_ = [
        ("d_bias", C.c_void_p),
        ("gelu", C.c_int),
        ("d_mul", C.c_void_p),
        ("d_residual", C.c_void_p),
    ]


class TensorRef(C.Structure):
    _fields_ = [
        ("data", C.c_void_p),
        ("type", C.c_int32),
        ("out_dim", C.c_uint32),
        ("in_dim", C.c_uint32),
    ]


class Gpt2Config(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("vocab", "embed", "head", "layer", "ctx", "ffn")]


class Gpt2Block(C.Structure):
    _fields_ = [
        ("ln1_weight", C.c_void_p),
        ("ln1_bias", C.c_void_p),
        ("attn_qkv_weight", TensorRef),
        ("attn_qkv_bias", C.c_void_p),
        ("attn_proj_weight", TensorRef),
        ("attn_proj_bias", C.c_void_p),
        ("ln2_weight", C.c_void_p),
        ("ln2_bias", C.c_void_p),
        ("mlp_fc_weight", TensorRef),
        ("mlp_fc_bias", C.c_void_p),
        ("mlp_proj_weight", TensorRef),
        ("mlp_proj_bias", C.c_void_p),
    ]


class Gpt2Weights(C.Structure):
    _fields_ = [
        ("wte", C.c_void_p),
        ("wpe", C.c_void_p),
        ("ln_f_weight", C.c_void_p),
        ("ln_f_bias", C.c_void_p),
        ("blocks", C.POINTER(Gpt2Block)),
    ]


class Gemma3Config(C.Structure):
    _fields_ = [
        ("vocab", C.c_uint32),
        ("embed", C.c_uint32),
        ("head", C.c_uint32),
        ("head_kv", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("layer", C.c_uint32),
        ("ctx", C.c_uint32),
        ("ffn", C.c_uint32),
        ("rope_base", C.c_float),
        ("sliding_window", C.c_uint32),
        ("rms_eps", C.c_float),
        ("global_every", C.c_uint32),
    ]


class Gemma3Block(C.Structure):
    _fields_ = [
        ("attn_norm_weight", C.c_void_p),
        ("post_attention_norm_weight", C.c_void_p),
        ("attn_q_weight", TensorRef),
        ("attn_k_weight", TensorRef),
        ("attn_v_weight", TensorRef),
        ("attn_output_weight", TensorRef),
        ("attn_q_norm_weight", C.c_void_p),
        ("attn_k_norm_weight", C.c_void_p),
        ("ffn_norm_weight", C.c_void_p),
        ("post_ffw_norm_weight", C.c_void_p),
        ("ffn_gate_weight", TensorRef),
        ("ffn_up_weight", TensorRef),
        ("ffn_down_weight", TensorRef),
    ]


class Gemma3Weights(C.Structure):
    _fields_ = [
        ("token_embd", TensorRef),
        ("output_norm_weight", C.c_void_p),
        ("blocks", C.POINTER(Gemma3Block)),
    ]
