"""Host-side model containers: the tensors a GGUF loader hands over, seeded synthetic generators
for GPT-2 and Gemma-3 shaped models, and their GGUF form (`to_gguf` / `from_gguf`) under the tensor
names zig-nn's loaders use (src/models/gpt2.zig:70-181, src/models/gemma3.zig:129-226).

A container keeps every numpy array alive and builds the C structs of include/zq.h
(zq_gpt2_weights / zq_gemma3_weights) that point into them.
"""
import ctypes as C

import numpy as np
import torch

from . import ggml
from . import gguf
from . import structs as S

GPT2_SMALL = dict(vocab=50257, embed=768, head=12, layer=12, ctx=1024, ffn=3072)
GEMMA3_1B = dict(vocab=262144, embed=1152, head=4, head_kv=1, head_dim=256, layer=26, ctx=2048, ffn=6912,
                 rope_base=1000000.0, sliding_window=512, rms_eps=1e-6, global_every=6)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class QuantTensor:
    """Raw GGUF bytes of one [out_dim, in_dim] tensor (host, numpy uint8)."""

    def __init__(self, raw, qtype, out_dim, in_dim):
        self.raw = np.ascontiguousarray(raw, dtype=np.uint8)
        self.qtype, self.out_dim, self.in_dim = qtype, out_dim, in_dim
        assert self.raw.size == ggml.tensor_bytes(qtype, out_dim * in_dim)

    def ref(self):
        return S.TensorRef(_p(self.raw), self.qtype, self.out_dim, self.in_dim)


class _Gen:
    """Seeded N(0, std) generator; 2-D weights are quantised, the rest stay f32."""

    def __init__(self, seed, std, device):
        self.g = torch.Generator(device=device)
        self.g.manual_seed(seed)
        self.std, self.device = std, device

    def normal(self, *shape):
        return torch.randn(*shape, generator=self.g, device=self.device, dtype=torch.float32) * self.std

    def quant(self, qtype, out_dim, in_dim):
        w = self.normal(out_dim, in_dim)
        raw = ggml.quantize(qtype, w)
        return QuantTensor(raw.cpu().numpy(), qtype, out_dim, in_dim)

    def f32(self, *shape):
        return np.ascontiguousarray(self.normal(*shape).cpu().numpy())


class Gpt2Host:
    def __init__(self, cfg):
        self.cfg = dict(cfg)
        self.wte = self.wpe = self.ln_f_weight = self.ln_f_bias = None
        self.blocks = []

    @classmethod
    def synthetic(cls, cfg=GPT2_SMALL, qtype=ggml.Q4_0, seed=42, std=0.02, device="cpu"):
        """Random-init model: 2-D linear weights ~ N(0, std) quantised to `qtype`; embeddings f32
        N(0, std); LayerNorm gamma = 1, beta = 0, biases = 0."""
        m = cls(cfg)
        c = m.cfg
        g = _Gen(seed, std, device)
        E, F = c["embed"], c["ffn"]
        m.wte = g.f32(c["vocab"], E)
        m.wpe = g.f32(c["ctx"], E)
        m.ln_f_weight = np.ones(E, np.float32)
        m.ln_f_bias = np.zeros(E, np.float32)
        for _ in range(c["layer"]):
            m.blocks.append(dict(
                ln1_weight=np.ones(E, np.float32), ln1_bias=np.zeros(E, np.float32),
                attn_qkv_weight=g.quant(qtype, 3 * E, E), attn_qkv_bias=np.zeros(3 * E, np.float32),
                attn_proj_weight=g.quant(qtype, E, E), attn_proj_bias=np.zeros(E, np.float32),
                ln2_weight=np.ones(E, np.float32), ln2_bias=np.zeros(E, np.float32),
                mlp_fc_weight=g.quant(qtype, F, E), mlp_fc_bias=np.zeros(F, np.float32),
                mlp_proj_weight=g.quant(qtype, E, F), mlp_proj_bias=np.zeros(E, np.float32),
            ))
        return m

    def randomize_small_params(self, seed=7, std=0.1):
        """Give norms and biases non-trivial values (tests)."""
        rng = np.random.default_rng(seed)
        def r(a, base):
            return (base + std * rng.standard_normal(a.shape)).astype(np.float32)
        self.ln_f_weight, self.ln_f_bias = r(self.ln_f_weight, 1), r(self.ln_f_bias, 0)
        for b in self.blocks:
            for k in list(b):
                if isinstance(b[k], np.ndarray):
                    b[k] = r(b[k], 1.0 if k.endswith("weight") else 0.0)
        return self

    def config_struct(self):
        c = self.cfg
        return S.Gpt2Config(c["vocab"], c["embed"], c["head"], c["layer"], c["ctx"], c["ffn"])

    def weights_struct(self):
        arr = (S.Gpt2Block * len(self.blocks))()
        for i, b in enumerate(self.blocks):
            for name, _ in S.Gpt2Block._fields_:
                v = b[name]
                setattr(arr[i], name, v.ref() if isinstance(v, QuantTensor) else _p(v))
        self._blocks_arr = arr
        return S.Gpt2Weights(_p(self.wte), _p(self.wpe), _p(self.ln_f_weight), _p(self.ln_f_bias), arr)

    def quant_bytes(self):
        return sum(v.raw.size for b in self.blocks for v in b.values() if isinstance(v, QuantTensor))

    # field of a block -> tensor name suffix (gpt2.zig:134-181)
    _BLOCK_NAMES = dict(
        ln1_weight="attn_norm.weight", ln1_bias="attn_norm.bias",
        attn_qkv_weight="attn_qkv.weight", attn_qkv_bias="attn_qkv.bias",
        attn_proj_weight="attn_output.weight", attn_proj_bias="attn_output.bias",
        ln2_weight="ffn_norm.weight", ln2_bias="ffn_norm.bias",
        mlp_fc_weight="ffn_up.weight", mlp_fc_bias="ffn_up.bias",
        mlp_proj_weight="ffn_down.weight", mlp_proj_bias="ffn_down.bias")

    def to_gguf(self, path):
        """GGUF v3 file that zig-nn's gpt2_weights.load_from_gguf reads (gpt2.zig:70-90)."""
        c = self.cfg
        meta = [("general.architecture", gguf.T_STRING, "gpt2"),
                ("general.name", gguf.T_STRING, "synthetic gpt2"),
                ("gpt2.context_length", gguf.T_UINT32, c["ctx"]),
                ("gpt2.embedding_length", gguf.T_UINT32, c["embed"]),
                ("gpt2.block_count", gguf.T_UINT32, c["layer"]),
                ("gpt2.feed_forward_length", gguf.T_UINT32, c["ffn"]),
                ("gpt2.attention.head_count", gguf.T_UINT32, c["head"]),
                ("gpt2.attention.layer_norm_epsilon", gguf.T_FLOAT32, 1e-5)]
        tensors = [_f32_tensor("token_embd.weight", self.wte), _f32_tensor("position_embd.weight", self.wpe),
                   _f32_tensor("output_norm.weight", self.ln_f_weight),
                   _f32_tensor("output_norm.bias", self.ln_f_bias)]
        for i, b in enumerate(self.blocks):
            for field, suffix in self._BLOCK_NAMES.items():
                tensors.append(_any_tensor("blk.%d.%s" % (i, suffix), b[field]))
        gguf.write(path, meta, tensors)

    @classmethod
    def from_gguf(cls, path_or_file):
        """Model geometry from the tensor shapes (zig-nn fixes it at compile time), head count from metadata."""
        f = path_or_file if isinstance(path_or_file, gguf.GGUFFile) else gguf.parse(path_or_file)
        wte, wpe = f.get_tensor_raw_bytes("token_embd.weight"), f.get_tensor_raw_bytes("position_embd.weight")
        layer = 0
        while f.get_tensor_info("blk.%d.attn_qkv.weight" % layer) is not None:
            layer += 1
        embed = wte.in_dim
        head = f.get_metadata_u32("gpt2.attention.head_count") or max(1, embed // 64)
        ffn = f.get_tensor_raw_bytes("blk.0.ffn_up.weight").out_dim
        m = cls(dict(vocab=wte.out_dim, embed=embed, head=head, layer=layer, ctx=wpe.out_dim, ffn=ffn))
        m._gguf = f  # quantised tensors are views into the mapped file
        m.wte = f.load_tensor_f32("token_embd.weight")
        m.wpe = f.load_tensor_f32("position_embd.weight")
        m.ln_f_weight = f.load_tensor_f32("output_norm.weight")
        m.ln_f_bias = f.load_tensor_f32("output_norm.bias")
        for i in range(layer):
            m.blocks.append({field: _load_field(f, "blk.%d.%s" % (i, suffix), quant=field.endswith("_weight")
                                                and not field.startswith("ln"))
                             for field, suffix in cls._BLOCK_NAMES.items()})
        return m


def _f32_tensor(name, a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return (name, tuple(reversed(a.shape)), ggml.F32, a)


def _any_tensor(name, v):
    if isinstance(v, QuantTensor):
        return (name, (v.in_dim, v.out_dim), v.qtype, v.raw)  # GGUF order: innermost dimension first
    return _f32_tensor(name, v)


def _load_field(f, name, quant):
    if not quant:
        return f.load_tensor_f32(name)
    r = f.get_tensor_raw_bytes(name)
    return QuantTensor(r.data, r.type_, r.out_dim, r.in_dim)


class Gemma3Host:
    def __init__(self, cfg):
        self.cfg = dict(cfg)
        self.token_embd = None
        self.output_norm_weight = None
        self.blocks = []

    @classmethod
    def synthetic(cls, cfg=GEMMA3_1B, qtype=ggml.Q8_0, seed=42, std=0.02, device="cpu", embd_qtype=None,
                  down_qtype=None):
        """Random-init model: every 2-D weight ~ N(0, std) quantised to `qtype` (token_embd and
        ffn_down may use their own types, as the real model does: src/models/gemma3.zig:103-120);
        RMSNorm weights = 1."""
        m = cls(cfg)
        c = m.cfg
        g = _Gen(seed, std, device)
        E, F, D = c["embed"], c["ffn"], c["head_dim"]
        QD, KD = c["head"] * D, c["head_kv"] * D
        m.token_embd = g.quant(embd_qtype or qtype, c["vocab"], E)
        m.output_norm_weight = np.ones(E, np.float32)
        for _ in range(c["layer"]):
            m.blocks.append(dict(
                attn_norm_weight=np.ones(E, np.float32), post_attention_norm_weight=np.ones(E, np.float32),
                attn_q_weight=g.quant(qtype, QD, E), attn_k_weight=g.quant(qtype, KD, E),
                attn_v_weight=g.quant(qtype, KD, E), attn_output_weight=g.quant(qtype, E, QD),
                attn_q_norm_weight=np.ones(D, np.float32), attn_k_norm_weight=np.ones(D, np.float32),
                ffn_norm_weight=np.ones(E, np.float32), post_ffw_norm_weight=np.ones(E, np.float32),
                ffn_gate_weight=g.quant(qtype, F, E), ffn_up_weight=g.quant(qtype, F, E),
                ffn_down_weight=g.quant(down_qtype or qtype, E, F),
            ))
        return m

    def randomize_small_params(self, seed=7, std=0.1):
        rng = np.random.default_rng(seed)
        def r(a):
            return (1.0 + std * rng.standard_normal(a.shape)).astype(np.float32)
        self.output_norm_weight = r(self.output_norm_weight)
        for b in self.blocks:
            for k in list(b):
                if isinstance(b[k], np.ndarray):
                    b[k] = r(b[k])
        return self

    def config_struct(self):
        c = self.cfg
        return S.Gemma3Config(c["vocab"], c["embed"], c["head"], c["head_kv"], c["head_dim"], c["layer"],
                              c["ctx"], c["ffn"], c["rope_base"], c["sliding_window"], c["rms_eps"],
                              c["global_every"])

    def weights_struct(self):
        arr = (S.Gemma3Block * len(self.blocks))()
        for i, b in enumerate(self.blocks):
            for name, _ in S.Gemma3Block._fields_:
                v = b[name]
                setattr(arr[i], name, v.ref() if isinstance(v, QuantTensor) else _p(v))
        self._blocks_arr = arr
        return S.Gemma3Weights(self.token_embd.ref(), _p(self.output_norm_weight), arr)

    def quant_bytes(self):
        n = self.token_embd.raw.size
        return n + sum(v.raw.size for b in self.blocks for v in b.values() if isinstance(v, QuantTensor))

    # field of a block -> tensor name suffix (gemma3.zig:174-226)
    _BLOCK_NAMES = dict(
        attn_norm_weight="attn_norm.weight", post_attention_norm_weight="post_attention_norm.weight",
        attn_q_weight="attn_q.weight", attn_k_weight="attn_k.weight", attn_v_weight="attn_v.weight",
        attn_output_weight="attn_output.weight", attn_q_norm_weight="attn_q_norm.weight",
        attn_k_norm_weight="attn_k_norm.weight", ffn_norm_weight="ffn_norm.weight",
        post_ffw_norm_weight="post_ffw_norm.weight", ffn_gate_weight="ffn_gate.weight",
        ffn_up_weight="ffn_up.weight", ffn_down_weight="ffn_down.weight")
    _QUANT_FIELDS = ("attn_q_weight", "attn_k_weight", "attn_v_weight", "attn_output_weight", "ffn_gate_weight",
                     "ffn_up_weight", "ffn_down_weight")

    def to_gguf(self, path):
        """GGUF v3 file that zig-nn's gemma3_weights.load_from_gguf reads (gemma3.zig:129-143)."""
        c = self.cfg
        meta = [("general.architecture", gguf.T_STRING, "gemma3"),
                ("general.name", gguf.T_STRING, "synthetic gemma3"),
                ("gemma3.context_length", gguf.T_UINT32, c["ctx"]),
                ("gemma3.embedding_length", gguf.T_UINT32, c["embed"]),
                ("gemma3.block_count", gguf.T_UINT32, c["layer"]),
                ("gemma3.feed_forward_length", gguf.T_UINT32, c["ffn"]),
                ("gemma3.attention.head_count", gguf.T_UINT32, c["head"]),
                ("gemma3.attention.head_count_kv", gguf.T_UINT32, c["head_kv"]),
                ("gemma3.attention.key_length", gguf.T_UINT32, c["head_dim"]),
                ("gemma3.attention.value_length", gguf.T_UINT32, c["head_dim"]),
                ("gemma3.attention.layer_norm_rms_epsilon", gguf.T_FLOAT32, c["rms_eps"]),
                ("gemma3.attention.sliding_window", gguf.T_UINT32, c["sliding_window"]),
                ("gemma3.attention.sliding_window_pattern", gguf.T_UINT32, c["global_every"]),
                ("gemma3.rope.freq_base", gguf.T_FLOAT32, c["rope_base"])]
        tensors = [_any_tensor("token_embd.weight", self.token_embd),
                   _f32_tensor("output_norm.weight", self.output_norm_weight)]
        for i, b in enumerate(self.blocks):
            for field, suffix in self._BLOCK_NAMES.items():
                tensors.append(_any_tensor("blk.%d.%s" % (i, suffix), b[field]))
        gguf.write(path, meta, tensors)

    @classmethod
    def from_gguf(cls, path_or_file, ctx=None):
        """Geometry from tensor shapes and metadata; what a file does not say falls back to the constants
        zig-nn compiles in (gemma3.zig:15-29)."""
        f = path_or_file if isinstance(path_or_file, gguf.GGUFFile) else gguf.parse(path_or_file)
        embd = f.get_tensor_raw_bytes("token_embd.weight")
        layer = 0
        while f.get_tensor_info("blk.%d.attn_q.weight" % layer) is not None:
            layer += 1
        u32, f32 = f.get_metadata_u32, f.get_metadata_f32
        head_dim = f.get_tensor_raw_bytes("blk.0.attn_q_norm.weight").n_elem
        q, k = f.get_tensor_raw_bytes("blk.0.attn_q.weight"), f.get_tensor_raw_bytes("blk.0.attn_k.weight")
        cfg = dict(GEMMA3_1B)
        cfg.update(vocab=embd.out_dim, embed=embd.in_dim, head=q.out_dim // head_dim, head_kv=k.out_dim // head_dim,
                   head_dim=head_dim, layer=layer, ffn=f.get_tensor_raw_bytes("blk.0.ffn_gate.weight").out_dim)
        cfg["ctx"] = ctx or u32("gemma3.context_length") or cfg["ctx"]
        cfg["rope_base"] = f32("gemma3.rope.freq_base") or cfg["rope_base"]
        cfg["sliding_window"] = u32("gemma3.attention.sliding_window") or cfg["sliding_window"]
        cfg["rms_eps"] = f32("gemma3.attention.layer_norm_rms_epsilon") or cfg["rms_eps"]
        cfg["global_every"] = u32("gemma3.attention.sliding_window_pattern") or cfg["global_every"]
        m = cls(cfg)
        m._gguf = f  # quantised tensors are views into the mapped file
        m.token_embd = _load_field(f, "token_embd.weight", quant=True)
        m.output_norm_weight = f.load_tensor_f32("output_norm.weight")
        for i in range(layer):
            m.blocks.append({field: _load_field(f, "blk.%d.%s" % (i, suffix), quant=field in cls._QUANT_FIELDS)
                             for field, suffix in cls._BLOCK_NAMES.items()})
        return m
