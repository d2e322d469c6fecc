"""GGUF v2/v3 container: reader with the behaviour of zig-nn's parser, and a v3 writer.

Reader (mirrors src/gguf/gguf.zig):
  header  magic "GGUF", version 2 or 3, tensor count, metadata count         gguf.zig:329-351
  metadata  key string, u32 value type, value; arrays kept as raw bytes      gguf.zig:426-540
  tensor info  name, n_dims <= 4, u64 dims (innermost first), type, offset   gguf.zig:542-574
  data section  starts at the next multiple of general.alignment (32)        gguf.zig:353-398
  get_tensor_raw_bytes  2-D: out_dim = dims[1], in_dim = dims[0]; borrowed   gguf.zig:147-176
  load_tensor_f32  f32 as is, f16 widened, block types decoded               gguf.zig:179-193

zig-nn only reads GGUF; the writer exists so that the synthetic GPT-2 / Gemma-3 models of this package
can be stored under the tensor names zig-nn's loaders ask for (src/models/gpt2.zig:70-181,
src/models/gemma3.zig:129-226) and read back — by this package or by zig-nn itself.

Host-only module. Decoding a *quantised* tensor to f32 (load_tensor_f32 on a q4_0 / q4_1 / q8_0 tensor)
runs the CUDA decoder and therefore needs the library and a GPU; f32 and f16 tensors need neither.
"""
import struct

import numpy as np

from . import ggml

GGUF_MAGIC = 0x46554747  # "GGUF" little-endian
DEFAULT_ALIGNMENT = 32

# metadata value types (gguf.zig:11-26)
T_UINT8, T_INT8, T_UINT16, T_INT16, T_UINT32, T_INT32, T_FLOAT32, T_BOOL, T_STRING, T_ARRAY, T_UINT64, T_INT64, \
    T_FLOAT64 = range(13)
_SCALAR_FMT = {T_UINT8: "<B", T_INT8: "<b", T_UINT16: "<H", T_INT16: "<h", T_UINT32: "<I", T_INT32: "<i",
               T_FLOAT32: "<f", T_BOOL: "<B", T_UINT64: "<Q", T_INT64: "<q", T_FLOAT64: "<d"}


class GGUFError(Exception):
    pass


class InvalidMagic(GGUFError):
    pass


class UnsupportedVersion(GGUFError):
    pass


class UnexpectedEof(GGUFError):
    pass


class UnsupportedValueType(GGUFError):
    pass


class TooManyDimensions(GGUFError):
    pass


class TensorNotFound(GGUFError, KeyError):
    pass


class UnsupportedQuantType(GGUFError):
    pass


class ArrayValue:
    """A metadata array, kept as raw bytes and decoded on demand (gguf.zig:29-33)."""

    def __init__(self, elem_type, count, raw):
        self.elem_type, self.count, self.raw = elem_type, count, raw

    def strings(self):
        if self.elem_type != T_STRING:
            raise GGUFError("array elements are not strings")
        out, pos = [], 0
        for _ in range(self.count):
            (n,) = struct.unpack_from("<Q", self.raw, pos)
            pos += 8
            out.append(bytes(self.raw[pos:pos + n]).decode("utf-8", errors="replace"))
            pos += n
        return out

    def values(self):
        if self.elem_type == T_STRING:
            return self.strings()
        if self.elem_type not in _SCALAR_FMT:
            raise GGUFError("nested arrays are kept as raw bytes only")
        fmt = _SCALAR_FMT[self.elem_type]
        vals = [v[0] for v in struct.iter_unpack(fmt, bytes(self.raw))]
        return [bool(v) for v in vals] if self.elem_type == T_BOOL else vals


class TensorInfo:
    def __init__(self, name, dims, type_, offset):
        self.name, self.dimensions, self.type_, self.offset = name, tuple(dims), type_, offset
        self.n_dims = len(dims)

    def num_elements(self):
        n = 1
        for d in self.dimensions:
            n *= d
        return n


class RawTensorRef:
    """Borrowed bytes of one tensor plus its geometry (gguf.zig:147-153)."""

    def __init__(self, data, type_, n_elem, out_dim, in_dim):
        self.data, self.type_, self.n_elem, self.out_dim, self.in_dim = data, type_, n_elem, out_dim, in_dim


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, n):
        if self.pos + n > len(self.buf):
            raise UnexpectedEof("need %d bytes at offset %d of %d" % (n, self.pos, len(self.buf)))
        b = self.buf[self.pos:self.pos + n]
        self.pos += n
        return b

    def unpack(self, fmt):
        return struct.unpack(fmt, bytes(self.take(struct.calcsize(fmt))))[0]

    def string(self):
        n = self.unpack("<Q")
        return bytes(self.take(n)).decode("utf-8", errors="replace")


def _read_value(cur, vtype):
    if vtype == T_STRING:
        return cur.string()
    if vtype == T_ARRAY:
        elem = cur.unpack("<I")
        count = cur.unpack("<Q")
        start = cur.pos
        if elem in _SCALAR_FMT:
            cur.take(count * struct.calcsize(_SCALAR_FMT[elem]))
        else:  # strings, nested arrays; unknown element types raise
            for _ in range(count):
                _read_value(cur, elem)
        return ArrayValue(elem, count, cur.buf[start:cur.pos])
    if vtype in _SCALAR_FMT:
        v = cur.unpack(_SCALAR_FMT[vtype])
        return bool(v) if vtype == T_BOOL else v
    raise UnsupportedValueType("metadata value type %d" % vtype)


class GGUFFile:
    """A parsed GGUF file. Tensor bytes are views into the file buffer (a numpy uint8 array or memmap)."""

    def __init__(self, buf, path=""):
        self.file_buf = buf if isinstance(buf, np.ndarray) else np.frombuffer(buf, dtype=np.uint8)
        self.file_path = path
        cur = _Cursor(self.file_buf)
        if cur.unpack("<I") != GGUF_MAGIC:
            raise InvalidMagic(path)
        self.version = cur.unpack("<I")
        if self.version < 2 or self.version > 3:
            raise UnsupportedVersion("GGUF version %d" % self.version)
        n_tensors = cur.unpack("<Q")
        n_kv = cur.unpack("<Q")
        self.metadata = []  # (key, value type, value) in file order
        for _ in range(n_kv):
            key = cur.string()
            vtype = cur.unpack("<I")
            self.metadata.append((key, vtype, _read_value(cur, vtype)))
        self.alignment = DEFAULT_ALIGNMENT
        for key, vtype, v in self.metadata:
            if key == "general.alignment":  # the first such key decides; other value types mean 32
                if vtype in (T_UINT32, T_UINT64):
                    self.alignment = int(v)
                break
        if self.alignment == 0:
            raise GGUFError("general.alignment is 0")
        self.tensors = []
        for _ in range(n_tensors):
            name = cur.string()
            n_dims = cur.unpack("<I")
            if n_dims > 4:
                raise TooManyDimensions("%s has %d dimensions" % (name, n_dims))
            dims = [cur.unpack("<Q") for _ in range(n_dims)]
            type_ = cur.unpack("<I")
            offset = cur.unpack("<Q")
            self.tensors.append(TensorInfo(name, dims, type_, offset))
        self._by_name = {t.name: t for t in reversed(self.tensors)}  # first of equal names wins
        a = self.alignment
        self.data_offset = (cur.pos + a - 1) // a * a

    # ---- metadata ----
    def get_metadata(self, key):
        for k, _, v in self.metadata:
            if k == key:
                return v
        return None

    def _typed(self, key, types):
        for k, t, v in self.metadata:
            if k == key:
                return v if t in types else None
        return None

    def get_metadata_string(self, key):
        return self._typed(key, (T_STRING,))

    def get_metadata_u32(self, key):
        return self._typed(key, (T_UINT32,))

    def get_metadata_u64(self, key):
        return self._typed(key, (T_UINT64,))

    def get_metadata_f32(self, key):
        return self._typed(key, (T_FLOAT32,))

    def get_array_strings(self, key):
        v = self._typed(key, (T_ARRAY,))
        return None if v is None or v.elem_type != T_STRING else v.strings()

    # ---- tensors ----
    def get_tensor_info(self, name):
        return self._by_name.get(name)

    def get_tensor_raw_bytes(self, name):
        info = self.get_tensor_info(name)
        if info is None:
            raise TensorNotFound(name)
        n_elem = info.num_elements()
        if ggml.block_size(info.type_) == 0:
            raise UnsupportedQuantType("%s: ggml type %d" % (name, info.type_))
        nbytes = ggml.tensor_bytes(info.type_, n_elem)
        start = self.data_offset + info.offset
        if start + nbytes > self.file_buf.size:
            raise UnexpectedEof("%s: %d bytes at %d of %d" % (name, nbytes, start, self.file_buf.size))
        out_dim = info.dimensions[1] if info.n_dims >= 2 else info.dimensions[0]
        in_dim = info.dimensions[0] if info.n_dims >= 2 else 1
        return RawTensorRef(self.file_buf[start:start + nbytes], info.type_, n_elem, out_dim, in_dim)

    def load_tensor_f32(self, name):
        """The tensor as a flat f32 array (a copy). Quantised tensors are decoded on the GPU."""
        ref = self.get_tensor_raw_bytes(name)
        if ref.type_ == ggml.F32:
            return np.frombuffer(ref.data.tobytes(), dtype="<f4").astype(np.float32)
        if ref.type_ == ggml.F16:
            return np.frombuffer(ref.data.tobytes(), dtype="<f2").astype(np.float32)
        from . import api  # needs the CUDA library
        rows = ref.out_dim if ref.in_dim % ggml.BLOCK_SIZE == 0 and ref.in_dim > 1 else 1
        qw = api.QuantWeight(np.ascontiguousarray(ref.data), ref.type_, rows, ref.n_elem // rows)
        try:
            return qw.dequantize().reshape(-1).cpu().numpy()
        finally:
            qw.close()

    def load_tensor_f32_transposed(self, name):
        """2-D tensor stored (cols, rows) -> row-major (rows, cols) (gguf.zig:196-221)."""
        info = self.get_tensor_info(name)
        if info is None:
            raise TensorNotFound(name)
        if info.n_dims != 2:
            raise GGUFError("%s is not 2-D" % name)
        cols, rows = info.dimensions[0], info.dimensions[1]
        return np.ascontiguousarray(self.load_tensor_f32(name).reshape(cols, rows).T).reshape(-1)


def parse(path):
    """Map the file and parse it (gguf.zig:306-322). Tensor data is not read until asked for."""
    return GGUFFile(np.memmap(path, dtype=np.uint8, mode="r"), path)


def parse_from_buffer(buf, path=""):
    return GGUFFile(buf, path)


# ---- writer ---------------------------------------------------------------------------------------

def _w_string(out, s):
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _w_value(out, vtype, v):
    out += struct.pack("<I", vtype)
    if vtype == T_STRING:
        _w_string(out, v)
    elif vtype == T_ARRAY:
        elem, items = v
        out += struct.pack("<IQ", elem, len(items))
        for it in items:
            if elem == T_STRING:
                _w_string(out, it)
            else:
                out += struct.pack(_SCALAR_FMT[elem], it)
    else:
        out += struct.pack(_SCALAR_FMT[vtype], v)


def write(path, metadata, tensors, alignment=DEFAULT_ALIGNMENT):
    """Write a GGUF v3 file.

    metadata: list of (key, value type, value); arrays as (T_ARRAY, (element type, [items])).
    tensors: list of (name, dims innermost-first, ggml type, bytes-like). Tensor data is laid out in the
    given order, each tensor starting on an `alignment` boundary of the data section.
    """
    head = bytearray()
    meta = list(metadata)
    if alignment != DEFAULT_ALIGNMENT and not any(k == "general.alignment" for k, _, _ in meta):
        meta.append(("general.alignment", T_UINT32, alignment))
    head += struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(meta))
    for key, vtype, v in meta:
        _w_string(head, key)
        _w_value(head, vtype, v)
    offsets, off = [], 0
    for name, dims, type_, data in tensors:
        n_elem = 1
        for d in dims:
            n_elem *= d
        nbytes = ggml.tensor_bytes(type_, n_elem)
        if nbytes == 0 or len(memoryview(data).cast("B")) != nbytes:
            raise GGUFError("%s: %d bytes given, %d expected" % (name, len(memoryview(data).cast("B")), nbytes))
        if len(dims) > 4:
            raise TooManyDimensions(name)
        offsets.append(off)
        off = (off + nbytes + alignment - 1) // alignment * alignment
    for (name, dims, type_, _), o in zip(tensors, offsets):
        _w_string(head, name)
        head += struct.pack("<I", len(dims))
        for d in dims:
            head += struct.pack("<Q", d)
        head += struct.pack("<IQ", type_, o)
    data_offset = (len(head) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (data_offset - len(head)))
        pos = 0
        for (_, _, _, data), o in zip(tensors, offsets):
            if o > pos:
                f.write(b"\0" * (o - pos))
            b = memoryview(data).cast("B")
            f.write(b)
            pos = o + len(b)
    return data_offset
