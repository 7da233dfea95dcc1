"""Shared helpers of the tests: library build, tolerance definition, seeded cases."""
import os

import numpy as np

from oracle import lw_oracle as orc

GEMV_TOL = 1e-3          # max |y - y_ref| / max |y_ref|, the reference check's definition (kernels/llmrt.cu:2868-2874)
FORMATS = ["Q4_K", "Q5_K", "Q6_K", "IQ4_XS"]
GOLDEN_FILES = {"Q4_K": "Q4_K_128x1024", "Q5_K": "Q5_K_128x512", "Q6_K": "Q6_K_192x512", "IQ4_XS": "IQ4_XS_64x1536"}


def build_library():
    from lazyweights_b200 import build
    return build.build()


def rel_err(y, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.abs(np.asarray(y, np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def golden(golden_dir, ty):
    return np.load(os.path.join(golden_dir, GOLDEN_FILES[ty] + ".npz"))


def seeded_case(ty, n, k, seed):
    """codes, side bytes, symbols, float32 weights from the oracle, for sizes the oracle handles in seconds."""
    rng = np.random.default_rng(seed)
    q = orc.synth_codes(ty, n, k, rng)
    side = orc.synth_side(ty, n, k, rng)
    return q, side, orc.symbols_of(ty, q), orc.dequant(ty, q, side), rng
