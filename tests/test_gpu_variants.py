"""The two alternative readers of the batch-1 kernel against the shipping one: the fixed-width twin (no Huffman
decoding) and the comparator (limit-register) decoder.  Both run the same integer sums in the same order, so their
results must equal the table decoder's bit for bit - what the reference demands of its packed twins
(kernels/llmrt.cu:895) - and meet the oracle's product within the usual bar."""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import lw_oracle as orc
from tests import helpers

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SHAPES = [("Q4_K", 256, 2048), ("Q5_K", 192, 1024), ("Q6_K", 320, 1024), ("IQ4_XS", 128, 2560), ("Q6_K", 64, 256),
          ("Q4_K", 1024, 4096)]


@pytest.fixture(scope="module")
def lw():
    helpers.build_library()
    import torch
    assert torch.cuda.is_available()
    import lazyweights_b200 as pkg
    yield pkg
    assert pkg.lib().lw_kernel_error() == 0


@pytest.mark.parametrize("ty,n,k", SHAPES)
def test_twin_equals_coded_product(lw, ty, n, k):
    import torch
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=3 * n + k)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
        assert mat.twin_bytes("m") == -1
        assert mat.make_twin("m")
        bits = {"Q4_K": 4, "IQ4_XS": 4, "Q5_K": 5, "Q6_K": 6}[ty]
        assert mat.twin_bytes("m") >= n * k * bits // 8                  # fixed-width codes plus the unit scales
        for dt in (np.float16, np.float32):
            x = torch.from_numpy(rng.standard_normal(k).astype(dt)).cuda()
            coded = mat.linear("m", x).cpu().numpy()
            twin = mat.linear_twin("m", x).cpu().numpy()[0]
            assert np.array_equal(twin, coded)
            assert helpers.rel_err(twin, orc.gemv_f64(w, x.cpu().numpy().astype(np.float32)[None])[0]) <= helpers.GEMV_TOL
        mat.drop_twin("m")
        with pytest.raises(lw.LwError):
            mat.linear_twin("m", x)


WORKER = r"""
import sys, numpy as np, torch
sys.path.insert(0, %r)
import lazyweights_b200 as lw
from tests import helpers
out = sys.argv[1]
res = {}
for ty, n, k in %r:
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=5 * n + k)
    # a patch of rare codes: long code words, groups that need the exact fallback
    hi = 15 if ty in ("Q4_K", "IQ4_XS") else (31 if ty == "Q5_K" else 63)
    q[:64, :128] = rng.integers(0, hi + 1, (64, 128))
    from oracle import lw_oracle as orc
    sym = orc.symbols_of(ty, q)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
        x = torch.from_numpy(rng.standard_normal(k).astype(np.float32)).cuda()
        res["%%s_%%d_%%d" %% (ty, n, k)] = mat.linear("m", x).cpu().numpy()
assert lw.lib().lw_kernel_error() == 0
np.savez(out, **res)
"""


def test_limit_register_decoder_equals_table_decoder(lw, tmp_path):
    """The comparator decoder is selected when the library is loaded (LW_GEMV1_LOOKUP=limit), so each decoder runs in
    a process of its own; the two result files must be identical."""
    script = WORKER % (ROOT, SHAPES[:5])
    outs = {}
    for mode in ("table", "limit"):
        env = dict(os.environ)
        env.pop("LW_GEMV1_LOOKUP", None)
        if mode == "limit":
            env["LW_GEMV1_LOOKUP"] = "limit"
        path = str(tmp_path / (mode + ".npz"))
        r = subprocess.run([sys.executable, "-c", script, path], env=env, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        outs[mode] = np.load(path)
    assert sorted(outs["table"].files) == sorted(outs["limit"].files) and len(outs["table"].files) == 5
    for key in outs["table"].files:
        assert np.array_equal(outs["table"][key], outs["limit"][key]), key
        ty, n, k = key.rsplit("_", 2)
        q, side, sym, w, rng = helpers.seeded_case(ty, int(n), int(k), seed=5 * int(n) + int(k))
        hi = 15 if ty in ("Q4_K", "IQ4_XS") else (31 if ty == "Q5_K" else 63)
        q[:64, :128] = rng.integers(0, hi + 1, (64, 128))
        w = orc.dequant(ty, q, side)
        x = rng.standard_normal(int(k)).astype(np.float32)
        assert helpers.rel_err(outs["limit"][key], orc.gemv_f64(w, x[None])[0]) <= helpers.GEMV_TOL
