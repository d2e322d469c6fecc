"""Builds libzq.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a, and the module image of the f32
forward kernels that zig-nn's CUDA backend loads by name (cuda_kernels.fatbin / cuda_kernels.cubin: what
`nvcc -ptx -arch=sm_90 ... cuda_kernels.cu` produces by hand in the reference, src/backend/cuda_kernels.cu:2,
here as a build step and for sm_100a; cuModuleLoadData takes either file's bytes).

    python zig-nn_b200/build.py [--force] [--verbose]
"""
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libzq.so")
MODULE_SRC = os.path.join(CSRC, "module", "cuda_kernels.cu")
MODULE_FATBIN = os.path.join(HERE, "cuda_kernels.fatbin")
MODULE_CUBIN = os.path.join(HERE, "cuda_kernels.cubin")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(REPO, "include"),
    "-I", CSRC,
]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libzq.so cannot be built")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hdrs.append(os.path.join(REPO, "include", "zq.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src, verbose):
    obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
    if os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), _deps_mtime()):
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return obj, r.stderr


def build_module_image(force=False):
    """cuda_kernels.fatbin and cuda_kernels.cubin: the sm_100a image of csrc/module/cuda_kernels.cu."""
    for out, flag in ((MODULE_FATBIN, "-fatbin"), (MODULE_CUBIN, "-cubin")):
        if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(MODULE_SRC):
            continue
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", flag, "-o", out, MODULE_SRC]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for the module image:\n%s\n%s" % (r.stdout, r.stderr))
    return MODULE_FATBIN


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    build_module_image(force)
    if force:
        for f in os.listdir(OBJ):
            os.remove(os.path.join(OBJ, f))
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if (not os.path.exists(LIB)) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
