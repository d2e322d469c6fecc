"""Host-side model containers: the tensors a GGUF loader would hand over, plus seeded
synthetic generators for GPT-2 and Gemma-3 shaped models.

A container keeps every numpy array alive and builds the C structs of include/zq.h
(zq_gpt2_weights / zq_gemma3_weights) that point into them.
"""
import ctypes as C

import numpy as np
import torch

from . import ggml
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
