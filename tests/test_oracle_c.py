"""The C restatement of the oracle (also the timed CPU baseline) against the reference-made golden vectors, and the
reference's own C++ decoder (oracle/_ref/huff_csim, built from a reference checkout when one is present)."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from oracle import build_oracle
from oracle import lw_oracle as orc
from tests import helpers


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


@pytest.mark.parametrize("ty", helpers.FORMATS)
def test_c_oracle_matches_golden(golden_dir, ty):
    L = build_oracle.lib()
    g = helpers.golden(golden_dir, ty)
    n, ks = g["sym"].shape
    k = g["q"].shape[1]
    blob = np.concatenate([g["blob"], np.zeros(16, np.uint8)])
    sym = np.empty((n, ks), np.uint8)
    L.orc_decode(_p(blob), n, ks, 3, _p(sym))
    assert np.array_equal(sym, g["decoded"])
    w = np.empty((n, k), np.float32)
    q, side = np.ascontiguousarray(g["q"]), np.ascontiguousarray(g["side"])
    L.orc_dequant(build_oracle.FMT[ty], _p(q), _p(side), n, k, _p(w))
    assert np.array_equal(w, g["w"])                                                  # bit-exact float32
    x = np.ascontiguousarray(g["x"].astype(np.float32))
    y = np.empty((x.shape[0], n), np.float32)
    L.orc_matvec(build_oracle.FMT[ty], _p(blob), _p(side), n, k, _p(x), x.shape[0], _p(y), 4)
    assert helpers.rel_err(y, g["y"]) <= 1e-5


@pytest.mark.parametrize("ty", helpers.FORMATS)
def test_c_packer_reproduces_reference_blobs(golden_dir, ty):
    g = helpers.golden(golden_dir, ty)
    blob, bits, _ = orc.encode_huf8_native(g["sym"])
    assert blob == g["blob"].tobytes()
    assert blob == orc.encode_huf8(g["sym"])[0]


@pytest.mark.parametrize("name", ["single", "uniform256", "two", "skewed"])
def test_c_packer_edge_blobs(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "edge_%s.npz" % name))
    assert orc.encode_huf8_native(g["sym"])[0] == g["blob"].tobytes()


def test_reference_cpp_decoder_agrees(tmp_path):
    """The reference's C++ ref_decode (hw/huff/tb/csim_main.cpp:45-62), run as a binary, on an oracle-written
    bundle.  Skipped where no reference checkout was available to build it from."""
    build_oracle.build()
    if not os.path.exists(build_oracle.REF_BIN):
        pytest.skip("oracle/_ref/huff_csim not built (no reference checkout)")
    rng = np.random.default_rng(2)
    w = orc.BundleWriter(str(tmp_path / "b"))
    cases = {}
    for ty, n, k in (("Q4_K", 64, 1024), ("Q6_K", 128, 256)):
        q, side = orc.synth_codes(ty, n, k, rng), orc.synth_side(ty, n, k, rng)
        w.add_matrix("m_" + ty, ty, q, side)
        cases["m_" + ty] = (ty, q)
    w.close()
    for name, (ty, q) in cases.items():
        dump = str(tmp_path / (name + ".bin"))
        r = subprocess.run([build_oracle.REF_BIN, str(tmp_path / "b"), "--threads", "2", "--only", name,
                            "--dump-ref", name, dump], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr
        sym = orc.symbols_of(ty, q)
        got = np.fromfile(dump, np.uint8).reshape(sym.shape)
        assert np.array_equal(got, sym)
        assert '"mismatch": 0' in r.stdout or "mismatch" not in r.stdout or '"mismatch":0' in r.stdout
