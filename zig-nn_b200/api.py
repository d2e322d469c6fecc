"""Host-side mirror of zig-nn's quantised-inference interface on top of libzq's C ABI.

Names follow the reference: QuantWeight / quant_matmul_no_grad (src/diff/mps_runtime.zig:1164-1205),
MetalContext.dispatch_* (src/backend/metal.zig:729-1096), cuda_ops.zig dispatchers, and the
gpt2(C) / gemma3(C) engines (src/models). torch is used for device memory and streams only.
"""
import ctypes as C

import numpy as np
import torch

from . import _lib, ggml
from . import structs as S

ACT_F32, ACT_Q8, ACT_F16 = 0, 1, 2
DECODE_AUTO, DECODE_LAUNCH_SEQUENCE, DECODE_PERSISTENT = 0, 1, 2


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _dev_f32(t):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise ValueError("expected a contiguous float32 CUDA tensor")
    return t


class QuantWeight:
    """A GGUF-quantised weight [out_dim, in_dim] resident on the device."""

    def __init__(self, raw, quant_type, out_dim, in_dim):
        """raw: the GGUF tensor bytes — uint8 numpy array / CPU tensor (host) or CUDA uint8 tensor."""
        lib = _lib.load()
        self.quant_type, self.out_dim, self.in_dim = int(quant_type), int(out_dim), int(in_dim)
        nbytes = ggml.tensor_bytes(self.quant_type, self.out_dim * self.in_dim)
        h = C.c_void_p()
        if isinstance(raw, torch.Tensor) and raw.is_cuda:
            raw = raw.contiguous().view(torch.uint8).reshape(-1)
            if raw.numel() != nbytes and nbytes:
                raise ValueError("raw byte count %d != %d" % (raw.numel(), nbytes))
            rc = lib.zq_weight_from_device(_ptr(raw), self.quant_type, self.out_dim, self.in_dim,
                                           _stream(), C.byref(h))
            torch.cuda.current_stream().synchronize()  # raw may be freed by the caller afterwards
        else:
            if isinstance(raw, torch.Tensor):
                raw = raw.numpy()
            raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
            if raw.size != nbytes and nbytes:
                raise ValueError("raw byte count %d != %d" % (raw.size, nbytes))
            rc = lib.zq_weight_upload(raw.ctypes.data_as(C.c_void_p), self.quant_type, self.out_dim,
                                      self.in_dim, _stream(), C.byref(h))
        _lib.check(rc, "zq_weight_upload")
        self._h = h

    @property
    def handle(self):
        return self._h

    def device_bytes(self):
        return _lib.load().zq_weight_device_bytes(self._h)

    def raw_bytes(self):
        """The original GGUF bytes, rebuilt on the device (uint8 CUDA tensor)."""
        n = ggml.tensor_bytes(self.quant_type, self.out_dim * self.in_dim)
        out = torch.empty(n, dtype=torch.uint8, device="cuda")
        _lib.check(_lib.load().zq_weight_download_raw(self._h, _ptr(out), _stream()), "zq_weight_download_raw")
        return out

    def dequantize(self):
        out = torch.empty(self.out_dim, self.in_dim, dtype=torch.float32, device="cuda")
        _lib.check(_lib.load().zq_dequantize(self._h, _ptr(out), _stream()), "zq_dequantize")
        return out

    def dequant_rows_scaled(self, token_ids, scale):
        ids = token_ids.to(device="cuda", dtype=torch.int32).contiguous()
        out = torch.empty(ids.numel(), self.in_dim, dtype=torch.float32, device="cuda")
        _lib.check(_lib.load().zq_dequant_rows_scaled(self._h, _ptr(ids), ids.numel(), float(scale),
                                                      _ptr(out), _stream()), "zq_dequant_rows_scaled")
        return out

    def close(self):
        if getattr(self, "_h", None):
            _lib.load().zq_weight_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _quant_matmul(x, qw, act_mode, bias, gelu, mul, residual, out, workspace):
    lib = _lib.load()
    x = _dev_f32(x)
    if x.shape[-1] != qw.in_dim:
        raise ValueError("last dim %d != in_dim %d" % (x.shape[-1], qw.in_dim))
    m = x.numel() // qw.in_dim
    y = out if out is not None else torch.empty(*x.shape[:-1], qw.out_dim, dtype=torch.float32, device=x.device)
    ep = S.Epilogue(_ptr(bias), int(bool(gelu)), _ptr(mul), _ptr(residual))
    need = lib.zq_matmul_workspace_bytes(qw.handle, m, act_mode)
    ws = workspace
    if need and (ws is None or ws.numel() < need):
        ws = torch.empty(need, dtype=torch.uint8, device=x.device)
    rc = lib.zq_matmul(qw.handle, _ptr(x), _ptr(y), m, act_mode, C.byref(ep), _ptr(ws) if need else None,
                       need, _stream())
    _lib.check(rc, "zq_matmul")
    return y


class _QuantMatmulFn(torch.autograd.Function):
    """The node quant_matmul_no_grad builds when x requires grad: backward_quant_matmul
    (src/diff/mps_runtime.zig:1212-1230) is the transposed product."""

    @staticmethod
    def forward(ctx, x, qw, act_mode):
        ctx.qw = qw
        return _quant_matmul(x.detach(), qw, act_mode, None, False, None, None, None, None)

    @staticmethod
    def backward(ctx, grad_out):
        return quant_matmul_transposed(grad_out.contiguous(), ctx.qw), None, None


def quant_matmul_no_grad(x, qw, act_mode=ACT_F32, bias=None, gelu=False, mul=None, residual=None,
                         out=None, workspace=None):
    """x [..., in_dim] f32 CUDA -> [..., out_dim]; quantised weight times activations
    (DiffMpsRuntime.quant_matmul_no_grad, src/diff/mps_runtime.zig:1171-1205). "no_grad" refers to the
    frozen weight: when x requires grad the result carries the backward to x, as in the reference."""
    if torch.is_grad_enabled() and isinstance(x, torch.Tensor) and x.requires_grad:
        if bias is not None or gelu or mul is not None or residual is not None or out is not None:
            raise ValueError("the differentiable form takes no epilogue and no out=")
        return _QuantMatmulFn.apply(x, qw, act_mode)
    return _quant_matmul(x, qw, act_mode, bias, gelu, mul, residual, out, workspace)


def quant_matmul_transposed(grad_out, qw, grad_x=None, accumulate=False, workspace=None):
    """grad_x [..., in_dim] (+)= grad_out [..., out_dim] . W — dispatch_quant_trans_batched of the
    reference's Metal runtime (src/diff/mps_runtime.zig:1217-1227). accumulate=True adds into grad_x."""
    lib = _lib.load()
    g = _dev_f32(grad_out)
    if g.shape[-1] != qw.out_dim:
        raise ValueError("last dim %d != out_dim %d" % (g.shape[-1], qw.out_dim))
    m = g.numel() // qw.out_dim
    if grad_x is None:
        if accumulate:
            raise ValueError("accumulate=True needs grad_x")
        grad_x = torch.empty(*g.shape[:-1], qw.in_dim, dtype=torch.float32, device=g.device)
    elif grad_x.numel() != m * qw.in_dim or grad_x.dtype != torch.float32 or not grad_x.is_contiguous():
        raise ValueError("grad_x must be a contiguous f32 tensor of %d x %d" % (m, qw.in_dim))
    need = lib.zq_matmul_transposed_workspace_bytes(qw.handle, m)
    ws = workspace
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=g.device)
    rc = lib.zq_matmul_transposed(qw.handle, _ptr(g), _ptr(grad_x), m, int(bool(accumulate)), _ptr(ws), need,
                                  _stream())
    _lib.check(rc, "zq_matmul_transposed")
    return grad_x


class HostLinear:
    """y = x . W^T with HOST buffers, the call shape of zig-nn's CPU path (matmul_q4_0_f32(weight, input,
    output, ...) on slices in host memory, src/gguf/dequant.zig:170-182; ThreadPool.matmul,
    src/gguf/thread_pool.zig:96-160).

    x and y are page-locked host tensors. x is copied into a device buffer; y is not copied at all: page-locked
    memory is addressable from the device, the kernels only ever write y, so the GEMV stores its rows straight
    into the caller's buffer over PCIe while the weights are still streaming. The copy and the launch are
    recorded once per (x, y) buffer pair and replayed afterwards. Pageable buffers take the plain route
    (device result, then a copy)."""

    def __init__(self, qw, m_rows=1, act_mode=ACT_F32, use_graph=True):
        self.qw, self.m, self.act_mode, self.use_graph = qw, int(m_rows), act_mode, use_graph
        self._x = torch.empty(self.m, qw.in_dim, dtype=torch.float32, device="cuda")
        need = _lib.load().zq_matmul_workspace_bytes(qw.handle, self.m, act_mode)
        self._ws = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
        self._need = need
        self._graphs = {}

    def _launch(self, hx, y_ptr):
        if hx.is_pinned():  # a kernel copy: the matmul behind it starts on its weights meanwhile
            _lib.check(_lib.load().zq_copy_f32(_ptr(self._x), C.c_void_p(hx.data_ptr()), hx.numel(), _stream()),
                       "zq_copy_f32")
        else:
            self._x.copy_(hx.reshape(self.m, self.qw.in_dim), non_blocking=True)
        ep = S.Epilogue(None, 0, None, None)
        rc = _lib.load().zq_matmul(self.qw.handle, _ptr(self._x), y_ptr, self.m, self.act_mode, C.byref(ep),
                                   _ptr(self._ws) if self._need else None, self._need, _stream())
        _lib.check(rc, "zq_matmul")

    def __call__(self, hx, hy):
        """hx: [m_rows, in_dim] f32 host; hy: [m_rows, out_dim] f32 host, overwritten. Returns hy; the result is
        complete when the call returns."""
        for t, n in ((hx, self.m * self.qw.in_dim), (hy, self.m * self.qw.out_dim)):
            if t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n:
                raise ValueError("expected contiguous float32 host tensors of %d x in_dim / out_dim" % self.m)
        if not (hx.is_pinned() and hy.is_pinned()):
            y = torch.empty(self.m, self.qw.out_dim, dtype=torch.float32, device="cuda")
            self._launch(hx, C.c_void_p(y.data_ptr()))
            hy.copy_(y.reshape(hy.shape))  # synchronises
            return hy
        key = (hx.data_ptr(), hy.data_ptr())
        g = self._graphs.get(key)
        if g is None and self.use_graph:
            self._launch(hx, C.c_void_p(hy.data_ptr()))  # plain first call: one-time set-up stays out of the capture
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch(hx, C.c_void_p(hy.data_ptr()))
            if len(self._graphs) >= 8:
                self._graphs.clear()
            self._graphs[key] = (g, hx, hy)  # keeps the buffers alive as long as the recording
            g = self._graphs[key]
        if g is not None:
            g[0].replay()
        else:
            self._launch(hx, C.c_void_p(hy.data_ptr()))
        torch.cuda.current_stream().synchronize()
        return hy


def quant_matmul_q8_static(x, qw, bias=None, gelu=False, mul=None, residual=None, out=None):
    """quant_matmul_no_grad(..., ACT_Q8) through the entry point that allocates nothing: its scratch
    is a fixed array inside libzq (at most 16 rows, in_dim <= 16384; one call at a time per device)."""
    lib = _lib.load()
    x = _dev_f32(x)
    if x.shape[-1] != qw.in_dim:
        raise ValueError("last dim %d != in_dim %d" % (x.shape[-1], qw.in_dim))
    m = x.numel() // qw.in_dim
    y = out if out is not None else torch.empty(*x.shape[:-1], qw.out_dim, dtype=torch.float32, device=x.device)
    ep = S.Epilogue(_ptr(bias), int(bool(gelu)), _ptr(mul), _ptr(residual))
    _lib.check(lib.zq_matmul_q8_static(qw.handle, _ptr(x), _ptr(y), m, C.byref(ep), _stream()),
               "zq_matmul_q8_static")
    return y


def quantize_rows_q8(x):
    x = _dev_f32(x)
    k = x.shape[-1]
    m = x.numel() // k
    q = torch.empty(m, k, dtype=torch.int8, device=x.device)
    scale = torch.empty(m, k // 32, dtype=torch.float32, device=x.device)
    s = torch.empty(m, k // 32, dtype=torch.int32, device=x.device)
    _lib.check(_lib.load().zq_quantize_rows_q8(_ptr(x), m, k, _ptr(q), _ptr(scale), _ptr(s), _stream()),
               "zq_quantize_rows_q8")
    return q, scale, s


def matvec_f32(w, x):
    w, x = _dev_f32(w), _dev_f32(x)
    y = torch.empty(w.shape[0], dtype=torch.float32, device=w.device)
    _lib.check(_lib.load().zq_matvec_f32(_ptr(w), _ptr(x), _ptr(y), w.shape[0], w.shape[1], _stream()),
               "zq_matvec_f32")
    return y


def argmax(logits):
    logits = _dev_f32(logits)
    out = torch.empty(1, dtype=torch.int32, device=logits.device)
    _lib.check(_lib.load().zq_argmax(_ptr(logits), logits.numel(), _ptr(out), _stream()), "zq_argmax")
    return out


SAMPLE_MAX_K = 256  # gpt2.zig:865


def _exp_f32(x):
    """exp of f32 values, evaluated in double and rounded once (the convention of every exponential on this path)."""
    return np.exp(np.asarray(x, dtype=np.float64)).astype(np.float32)


def sample_top_k(logits, top_k, temperature, rng):
    """Temperature + top-k sampling on the host, the way gpt2.sample_top_k does it (src/models/gpt2.zig:866-977).

    `logits`: 1-D f32 (torch tensor on any device or numpy array; a copy is taken, the caller's row is left alone).
    `rng`: a numpy.random.Generator; one f32 uniform is drawn per call, as the reference draws `rng.float(f32)`.
    top_k == 0 or top_k >= n samples from the softmax of all logits (sample_full_softmax). Otherwise the (at most
    256) largest scaled logits are kept in the reference's min-buffer ORDER — the first k in index order, every
    later larger value overwriting the slot of the current minimum — because the cumulative distribution is walked
    in that order, and the token returned for a given uniform depends on it."""
    if isinstance(logits, torch.Tensor):
        logits = logits.detach().float().cpu().numpy()
    v = np.array(logits, dtype=np.float32).reshape(-1)
    n = v.size
    k = top_k if 0 < top_k < n else n
    inv_temp = np.float32(1.0) / np.float32(temperature) if (temperature > 0 and temperature != 1.0) else np.float32(1.0)
    if k >= n:
        if inv_temp != 1.0:
            v = v * inv_temp
        e = _exp_f32(v - v.max())
        probs = e * (np.float32(1.0) / np.cumsum(e, dtype=np.float32)[-1])
        r = np.float32(rng.random(dtype=np.float32))
        hit = np.nonzero(np.cumsum(probs, dtype=np.float32) >= r)[0]
        return int(hit[0]) if hit.size else n - 1
    k = min(k, SAMPLE_MAX_K)
    v = v * inv_temp
    vals = v[:k].copy()
    idxs = np.arange(k, dtype=np.int64)
    pos = int(np.argmin(vals))  # first minimum, as the reference's strict `<` scan finds it
    mn = vals[pos]
    BLOCK = 4096
    for b0 in range(k, n, BLOCK):
        blk = v[b0:b0 + BLOCK]
        for j in np.nonzero(blk > mn)[0]:  # the minimum only rises: a value that fails now fails later too
            x = blk[j]
            if x > mn:
                vals[pos] = x
                idxs[pos] = b0 + j
                pos = int(np.argmin(vals))
                mn = vals[pos]
    e = _exp_f32(vals - vals.max())
    total = np.float32(0.0)
    for x in e:
        total = np.float32(total + x)
    probs = e * (np.float32(1.0) / total)
    r = np.float32(rng.random(dtype=np.float32))
    c = np.float32(0.0)
    for j in range(k):
        c = np.float32(c + probs[j])
        if c >= r:
            return int(idxs[j])
    return int(idxs[k - 1])


def rms_norm(x, w, eps):
    x = _dev_f32(x)
    out = torch.empty_like(x)
    dim = x.shape[-1]
    _lib.check(_lib.load().zq_rms_norm(_ptr(x), _ptr(_dev_f32(w)), _ptr(out), dim, x.numel() // dim, eps,
                                       _stream()), "zq_rms_norm")
    return out


def rms_norm_residual(x, w, residual, eps):
    x, residual = _dev_f32(x), _dev_f32(residual)
    dim = x.shape[-1]
    _lib.check(_lib.load().zq_rms_norm_residual(_ptr(x), _ptr(_dev_f32(w)), _ptr(residual), dim,
                                                x.numel() // dim, eps, _stream()), "zq_rms_norm_residual")
    return residual


def rms_norm_in_place(x, w, dim, eps):
    x = _dev_f32(x)
    _lib.check(_lib.load().zq_rms_norm_in_place(_ptr(x), _ptr(_dev_f32(w)), dim, x.numel() // dim, eps,
                                                _stream()), "zq_rms_norm_in_place")
    return x


def rope_freqs(head_dim, base):
    f = np.empty(head_dim // 2, dtype=np.float32)
    _lib.check(_lib.load().zq_rope_freqs_host(head_dim, base, f.ctypes.data_as(C.c_void_p)), "zq_rope_freqs_host")
    return f


def rope(x, freqs, n_heads, pos):
    x, freqs = _dev_f32(x), _dev_f32(freqs)
    _lib.check(_lib.load().zq_rope(_ptr(x), _ptr(freqs), freqs.numel(), n_heads, float(pos), _stream()), "zq_rope")
    return x


def gelu_mul(gate, up):
    gate, up = _dev_f32(gate), _dev_f32(up)
    _lib.check(_lib.load().zq_gelu_mul(_ptr(gate), _ptr(up), gate.numel(), _stream()), "zq_gelu_mul")
    return gate


def write_kv_cache(k, v, k_cache, v_cache, pos):
    _lib.check(_lib.load().zq_write_kv_cache(_ptr(_dev_f32(k)), _ptr(_dev_f32(v)), _ptr(_dev_f32(k_cache)),
                                             _ptr(_dev_f32(v_cache)), pos, k.numel(), _stream()),
               "zq_write_kv_cache")


ATTN_GPT2_SOFTMAX = 1


def attention_decode(q, k_cache, v_cache, n_head, n_kv_head, head_dim, kv_start, kv_end, flags=0, scores=None):
    q = _dev_f32(q)
    out = torch.empty(n_head * head_dim, dtype=torch.float32, device=q.device)
    if scores is None:
        scores = torch.empty(n_head * max(1, kv_end - kv_start), dtype=torch.float32, device=q.device)
    _lib.check(_lib.load().zq_attention_decode(_ptr(q), _ptr(_dev_f32(k_cache)), _ptr(_dev_f32(v_cache)),
                                               _ptr(out), _ptr(scores), n_head, n_kv_head, head_dim, kv_start,
                                               kv_end, flags, _stream()), "zq_attention_decode")
    return out


def softmax(x):
    x = _dev_f32(x)
    out = torch.empty_like(x)
    cols = x.shape[-1]
    _lib.check(_lib.load().zq_softmax_out(_ptr(out), _ptr(x), x.numel() // cols, cols, _stream()), "zq_softmax_out")
    return out


def softmax_(x):
    x = _dev_f32(x)
    cols = x.shape[-1]
    _lib.check(_lib.load().zq_softmax(_ptr(x), x.numel() // cols, cols, _stream()), "zq_softmax")
    return x


def layer_norm(x, gamma, beta, eps):
    x = _dev_f32(x)
    out = torch.empty_like(x)
    cols = x.shape[-1]
    _lib.check(_lib.load().zq_layer_norm(_ptr(out), _ptr(x), _ptr(_dev_f32(gamma)), _ptr(_dev_f32(beta)),
                                         x.numel() // cols, cols, eps, _stream()), "zq_layer_norm")
    return out


def gelu(x):
    x = _dev_f32(x)
    out = torch.empty_like(x)
    _lib.check(_lib.load().zq_gelu(_ptr(out), _ptr(x), x.numel(), _stream()), "zq_gelu")
    return out


def add_broadcast(a, b):
    a, b = _dev_f32(a), _dev_f32(b)
    out = torch.empty_like(a)
    _lib.check(_lib.load().zq_add_broadcast(_ptr(out), _ptr(a), _ptr(b), a.numel(), b.numel(), _stream()),
               "zq_add_broadcast")
    return out


def mul_broadcast(a, b):
    a, b = _dev_f32(a), _dev_f32(b)
    out = torch.empty_like(a)
    _lib.check(_lib.load().zq_mul_broadcast(_ptr(out), _ptr(a), _ptr(b), a.numel(), b.numel(), _stream()),
               "zq_mul_broadcast")
    return out


def gather(table, idx):
    table = _dev_f32(table)
    idx = idx.to(device=table.device, dtype=torch.int32).contiguous()
    out = torch.empty(idx.numel(), table.shape[1], dtype=torch.float32, device=table.device)
    _lib.check(_lib.load().zq_gather(_ptr(out), _ptr(table), _ptr(idx), idx.numel(), table.shape[1], _stream()),
               "zq_gather")
    return out


def scale(x, s):
    x = _dev_f32(x)
    out = torch.empty_like(x)
    _lib.check(_lib.load().zq_scale(_ptr(out), _ptr(x), float(s), x.numel(), _stream()), "zq_scale")
    return out


class _DevicePtrView:
    """Exposes borrowed device memory (n f32 values) through __cuda_array_interface__."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {
            "shape": (n,), "typestr": "<f4", "data": (int(ptr), False), "version": 2, "strides": None,
        }


class _Engine:
    _prefix = None

    def __init__(self, host_model):
        lib = _lib.load()
        self._cfg = host_model.config_struct()
        self._w = host_model.weights_struct()
        self.vocab = self._cfg.vocab
        h = C.c_void_p()
        rc = getattr(lib, self._prefix + "_create")(C.byref(self._cfg), C.byref(self._w), _stream(), C.byref(h))
        _lib.check(rc, self._prefix + "_create")
        self._h = h

    def _logits(self, ptr):
        """Copy of the engine-owned logits buffer (valid only until the next engine call)."""
        view = torch.as_tensor(_DevicePtrView(ptr.value, self.vocab), device="cuda")
        return view.clone()

    def reset_cache(self):
        _lib.check(getattr(_lib.load(), self._prefix + "_reset_cache")(self._h))

    @property
    def seq_len(self):
        n = C.c_uint32()
        _lib.check(getattr(_lib.load(), self._prefix + "_seq_len")(self._h, C.byref(n)))
        return n.value

    def prefill(self, tokens):
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        ptr = C.c_void_p()
        rc = getattr(_lib.load(), self._prefix + "_prefill")(self._h, toks.ctypes.data_as(C.c_void_p), toks.size,
                                                             _stream(), C.byref(ptr))
        _lib.check(rc, self._prefix + "_prefill")
        return self._logits(ptr)

    def decode_next(self, token):
        ptr = C.c_void_p()
        rc = getattr(_lib.load(), self._prefix + "_decode_next")(self._h, int(token), _stream(), C.byref(ptr))
        _lib.check(rc, self._prefix + "_decode_next")
        return self._logits(ptr)

    def decode_greedy(self, first_token, n_steps):
        out = np.empty(n_steps, dtype=np.uint32)
        rc = getattr(_lib.load(), self._prefix + "_decode_greedy")(self._h, int(first_token), n_steps, _stream(),
                                                                   out.ctypes.data_as(C.c_void_p))
        _lib.check(rc, self._prefix + "_decode_greedy")
        return out

    def close(self):
        if getattr(self, "_h", None):
            getattr(_lib.load(), self._prefix + "_free")(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Gpt2(_Engine):
    """gpt2(C): init / prefill / decode_next (src/models/gpt2.zig:236,423,443)."""
    _prefix = "zq_gpt2"

    def set_decode_mode(self, mode):
        """DECODE_AUTO / DECODE_LAUNCH_SEQUENCE / DECODE_PERSISTENT (one cooperative kernel per token)."""
        _lib.check(_lib.load().zq_gpt2_set_decode_mode(self._h, int(mode)), "zq_gpt2_set_decode_mode")

    @property
    def decode_mode(self):
        mode = C.c_int()
        _lib.check(_lib.load().zq_gpt2_decode_mode(self._h, C.byref(mode)))
        return mode.value


class Gemma3(_Engine):
    """gemma3(C): init / prefill / decode_next (src/models/gemma3.zig:283,551,789)."""
    _prefix = "zq_gemma3"

    def seq_len_of(self, seq):
        n = C.c_uint32()
        _lib.check(_lib.load().zq_gemma3_seq_len_of(self._h, int(seq), C.byref(n)))
        return n.value

    def set_decode_mode(self, mode):
        """DECODE_AUTO / DECODE_LAUNCH_SEQUENCE / DECODE_PERSISTENT (one cooperative kernel per token)."""
        _lib.check(_lib.load().zq_gemma3_set_decode_mode(self._h, int(mode)), "zq_gemma3_set_decode_mode")

    def profile_step(self, token):
        """One decode step with per-phase cycle stamps (the device-side counterpart of gemma3.ProfileStats,
        src/models/gemma3.zig:35-92). Returns an int64 array [n_ctas][3 + 10 * layers] of SM cycle counts at the
        phase boundaries (layout: include/zq.h, zq_gemma3_profile_step)."""
        cap = 3 + 10 * self._cfg.layer
        buf = np.zeros(4096 * cap, dtype=np.int64)
        n = C.c_uint32()
        rc = _lib.load().zq_gemma3_profile_step(self._h, int(token), _stream(), buf.ctypes.data_as(C.c_void_p), cap,
                                                C.byref(n))
        _lib.check(rc, "zq_gemma3_profile_step")
        return buf[:n.value * cap].reshape(n.value, cap)

    @property
    def decode_mode(self):
        mode = C.c_int()
        _lib.check(_lib.load().zq_gemma3_decode_mode(self._h, C.byref(mode)))
        return mode.value


class Gemma3Batch:
    """Several independent sequences in one engine: prefill each, then advance all of them per call
    (the linears run as exact int8 GEMMs over the sequences)."""

    def __init__(self, host_model, n_seq):
        lib = _lib.load()
        self._cfg = host_model.config_struct()
        self._w = host_model.weights_struct()
        self.vocab, self.n_seq = self._cfg.vocab, int(n_seq)
        h = C.c_void_p()
        _lib.check(lib.zq_gemma3_create_batch(C.byref(self._cfg), C.byref(self._w), self.n_seq, _stream(), C.byref(h)),
                   "zq_gemma3_create_batch")
        self._h = h

    def prefill(self, seq, tokens):
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        ptr = C.c_void_p()
        rc = _lib.load().zq_gemma3_prefill_seq(self._h, int(seq), toks.ctypes.data_as(C.c_void_p), toks.size, _stream(),
                                               C.byref(ptr))
        _lib.check(rc, "zq_gemma3_prefill_seq")
        return torch.as_tensor(_DevicePtrView(ptr.value, self.vocab), device="cuda").clone()

    def decode_next(self, tokens):
        """tokens: one per sequence -> logits [n_seq][vocab] (a copy)."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        if toks.size != self.n_seq:
            raise ValueError("need %d tokens, got %d" % (self.n_seq, toks.size))
        ptr = C.c_void_p()
        rc = _lib.load().zq_gemma3_decode_next_batch(self._h, toks.ctypes.data_as(C.c_void_p), _stream(), C.byref(ptr))
        _lib.check(rc, "zq_gemma3_decode_next_batch")
        view = torch.as_tensor(_DevicePtrView(ptr.value, self.n_seq * self.vocab), device="cuda")
        return view.clone().view(self.n_seq, self.vocab)

    def seq_len(self, seq):
        n = C.c_uint32()
        _lib.check(_lib.load().zq_gemma3_seq_len_of(self._h, int(seq), C.byref(n)))
        return n.value

    def reset_cache(self):
        """Every sequence restarts at position 0 (its cache rows are overwritten by the next prefill)."""
        _lib.check(_lib.load().zq_gemma3_reset_cache(self._h))

    def close(self):
        if getattr(self, "_h", None):
            _lib.load().zq_gemma3_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
