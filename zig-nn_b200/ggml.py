"""GGML block geometry and weight encoders (host-side, torch tensors on any device).

Geometry mirrors src/gguf/dequant.zig:9-61 of zig-nn. zig-nn has no Q4_0 / Q4_1 / Q8_0
weight quantiser in library code; the encoders here produce the synthetic models and
benchmark weights:
  q4_0: d = signed-absmax / -8, q = clamp(round(x/d) + 8, 0, 15)
  q4_1: m = min, d = (max - min) / 15, q = clamp(round((x - m)/d), 0, 15)
  q8_0: scale = absmax / 127, q = clamp(round(x/scale), -128, 127)
        (the test encoder at src/diff/mps_runtime_test.zig:649-674)
with f16 d / m / scale and round-half-away-from-zero.
"""
import torch

F32, F16, Q4_0, Q4_1, Q8_0 = 0, 1, 2, 3, 8
BLOCK_SIZE = 32
_BPB = {F32: 4, F16: 2, Q4_0: 18, Q4_1: 20, Q8_0: 34}
_BS = {F32: 1, F16: 1, Q4_0: 32, Q4_1: 32, Q8_0: 32}
TYPE_NAMES = {F32: "f32", F16: "f16", Q4_0: "q4_0", Q4_1: "q4_1", Q8_0: "q8_0"}
TYPE_IDS = {v: k for k, v in TYPE_NAMES.items()}


def block_size(t):
    return _BS.get(t, 0)


def bytes_per_block(t):
    return _BPB.get(t, 0)


def tensor_bytes(t, num_elements):
    bs = block_size(t)
    if bs == 0:
        return 0
    return (num_elements // bs) * bytes_per_block(t)


def _round_half_away(v):
    t = torch.trunc(v)
    frac = v - t  # exact
    return t + torch.where(frac.abs() >= 0.5, torch.sign(v), torch.zeros_like(v))


def _f16_bytes(v):
    return v.to(torch.float16).view(torch.uint8).reshape(-1, 2)


def _pack_nibbles(q):
    return (q[:, :16] | (q[:, 16:] << 4)).to(torch.uint8)


def quantize_q4_0(x):
    xb = x.reshape(-1, 32).to(torch.float32)
    idx = xb.abs().argmax(dim=1, keepdim=True)
    smax = xb.gather(1, idx)
    d = smax / -8.0
    nz = d != 0
    safe = torch.where(nz, d, torch.ones_like(d))
    r = torch.where(nz, _round_half_away(xb / safe) + 8.0, torch.full_like(xb, 8.0))
    q = r.clamp(0, 15).to(torch.uint8)
    return torch.cat([_f16_bytes(d), _pack_nibbles(q)], dim=1).reshape(-1)


def quantize_q4_1(x):
    xb = x.reshape(-1, 32).to(torch.float32)
    mn = xb.min(dim=1, keepdim=True).values
    mx = xb.max(dim=1, keepdim=True).values
    d = (mx - mn) / 15.0
    nz = d != 0
    safe = torch.where(nz, d, torch.ones_like(d))
    r = torch.where(nz, _round_half_away((xb - mn) / safe), torch.zeros_like(xb))
    q = r.clamp(0, 15).to(torch.uint8)
    return torch.cat([_f16_bytes(d), _f16_bytes(mn), _pack_nibbles(q)], dim=1).reshape(-1)


def quantize_q8_0(x):
    xb = x.reshape(-1, 32).to(torch.float32)
    amax = xb.abs().max(dim=1, keepdim=True).values
    scale = amax / 127.0
    nz = scale != 0
    inv = torch.where(nz, 1.0 / torch.where(nz, scale, torch.ones_like(scale)), torch.zeros_like(scale))
    q = _round_half_away(xb * inv).clamp(-128, 127).to(torch.int8).view(torch.uint8)
    return torch.cat([_f16_bytes(scale), q], dim=1).reshape(-1)


def quantize(t, x):
    """x: float tensor whose element count is a multiple of 32 -> flat uint8 GGUF bytes."""
    if t == Q4_0:
        return quantize_q4_0(x)
    if t == Q4_1:
        return quantize_q4_1(x)
    if t == Q8_0:
        return quantize_q8_0(x)
    raise ValueError("UnsupportedQuantType: %r" % (t,))
