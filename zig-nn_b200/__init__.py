"""zig-nn's quantised-inference hot path on B200: GGUF Q4_0 / Q4_1 / Q8_0 linears and the small
ops between them, as hand-written sm_100a CUDA kernels behind a C ABI (include/zq.h).

The directory is named ``zig-nn_b200``; import it as ``zignn_b200`` (see zignn_b200.py at the
repository root). ``ggml``, ``gguf``, ``structs``, ``hostmodel`` and ``sharding`` are host-only; everything in ``api``
needs libzq.so and a GPU and raises if either is missing.
"""
from . import ggml, gguf, hostmodel, sharding, structs  # noqa: F401

__all__ = ["ggml", "gguf", "hostmodel", "sharding", "structs", "api", "_lib"]


def __getattr__(name):
    if name in ("api", "_lib"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
