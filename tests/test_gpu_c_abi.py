"""The C ABI used from plain C: tests/c_abi/client.c is compiled with gcc against include/zq.h, linked with
libzq.so and the CUDA runtime, and run. It builds a q8_0 matrix by hand whose product is known in
closed form and checks both activation modes, the epilogue, argmax and the error statuses."""
import os
import shutil
import subprocess

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cuda_home():
    for p in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if p and os.path.exists(os.path.join(p, "include", "cuda_runtime_api.h")):
            return p
    return None


def _compile(tmp_path):
    cuda = _cuda_home()
    gcc = shutil.which("gcc")
    if not cuda or not gcc:
        pytest.skip("needs gcc and a CUDA toolkit")
    libdir = os.path.join(REPO, "zig-nn_b200")
    if not os.path.exists(os.path.join(libdir, "libzq.so")):
        pytest.skip("libzq.so not built")
    exe = str(tmp_path / "client")
    cmd = [gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-I" + os.path.join(REPO, "include"),
           "-I" + os.path.join(cuda, "include"), os.path.join(REPO, "tests", "c_abi", "client.c"), "-o", exe,
           "-L" + libdir, "-lzq", "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-lm",
           "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_c_client_compiles_and_links(tmp_path):
    """No GPU needed: the header is valid C99 and every symbol the client uses is exported."""
    _compile(tmp_path)


@pytest.mark.gpu
def test_c_client_runs(tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    exe = _compile(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "c abi client ok" in r.stdout
