"""Builds liblwb200.so (CUDA kernels for sm_100a + the C ABI) in-tree with nvcc.

    python -m lazyweights_b200.build [--force]

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is installed.  The library lands next
to this file; the Python package loads it with ctypes and fails loudly if it is missing.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "liblwb200.so")
SOURCES = ["lw_host.cpp", "lw_blocks.cpp", "lw_pairs.cpp", "lw_kernels.cu", "lw_gemv1.cu", "lw_gemvm.cu", "lw_decw.cu", "lw_decc.cu", "lw_gemm_t5.cu", "lw_capi.cu", "lw_runtime.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC,-O3,-Wall,-pthread", "-Xptxas", "-v"]


def _nvcc():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found: set NVCC or add the CUDA toolkit to PATH")


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "lwb200.h"),
                                                                os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compiles the library if any source is newer than it.  Returns the library path."""
    if not force and not _stale():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    def compile_one(src):
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        with open(os.path.join(objdir, os.path.splitext(src)[0] + ".log"), "w") as f:
            f.write(r.stdout + r.stderr)
        return src, obj, r

    objs = []
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:   # one nvcc per source, side by side
        for src, obj, r in pool.map(compile_one, SOURCES):
            if r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError("nvcc failed on " + src)
            if verbose:
                sys.stderr.write(r.stderr)
            objs.append(obj)
    r = subprocess.run([nvcc, "-shared", "-o", LIB] + objs + ["-lcudart", "-lpthread", "-ldl"], capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
