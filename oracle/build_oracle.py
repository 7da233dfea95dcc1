"""Builds the oracle's native parts.  TEST INFRASTRUCTURE ONLY.

  oracle/liblw_oracle.so   the C restatement (lw_oracle_c.c), gcc -O2 -pthread
  oracle/_ref/huff_csim    the REFERENCE's own C++ decoder test bench (hw/huff/tb/csim_main.cpp with
                           hw/huff/huff_engine.h), compiled from the sources where they lie in a reference
                           checkout; only built when $LW_REFERENCE names such a checkout.  Nothing of the
                           reference is copied into this repository.
"""
import ctypes as C
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liblw_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_BIN = os.path.join(REF_DIR, "huff_csim")
FMT = {"Q4_K": 1, "Q5_K": 2, "Q6_K": 3, "IQ4_XS": 4}


def _newer(src, dst):
    return not os.path.exists(dst) or os.path.getmtime(src) > os.path.getmtime(dst)


def build():
    src = os.path.join(HERE, "lw_oracle_c.c")
    if _newer(src, LIB):
        # -ffp-contract=off: the dequantisation must round the product before the subtraction
        subprocess.run(["gcc", "-O2", "-std=c11", "-ffp-contract=off", "-fPIC", "-shared", "-pthread", src, "-o", LIB],
                       check=True)
    ref = os.environ.get("LW_REFERENCE", "")
    tb = os.path.join(ref, "hw", "huff", "tb", "csim_main.cpp")
    if ref and os.path.exists(tb) and shutil.which("g++") and _newer(tb, REF_BIN):
        os.makedirs(REF_DIR, exist_ok=True)
        subprocess.run(["g++", "-O2", "-std=c++17", "-pthread", "-I", os.path.join(ref, "hw", "huff"), tb, "-o",
                        REF_BIN], check=True)
    return LIB


def lib():
    build()
    L = C.CDLL(LIB)
    L.orc_decode.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    L.orc_dequant.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    L.orc_pack.restype = C.c_longlong
    L.orc_pack.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.orc_matvec.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                             C.c_int]
    return L


if __name__ == "__main__":
    print(build())
