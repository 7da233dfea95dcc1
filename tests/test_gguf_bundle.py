"""The GGUF -> bundle builder and the block split / join behind it (host only).

Pins: `tests/golden/<TYPE>_*.npz` hold GGUF block bytes with the reference's own split output and dequantised weights;
`tests/golden/gguf_bundles.json` holds, for three synthetic GGUF files (tests/golden/synth_gguf.py), the name, encoding,
shape, size and SHA-256 of every tensor the reference's builder functions write (recorded by make_gguf_golden.py)."""
import hashlib
import json
import os
import sys

import numpy as np
import pytest

from tests import helpers

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import synth_gguf  # noqa: E402


@pytest.fixture(scope="module")
def kq():
    helpers.build_library()
    from lazyweights_b200 import kquant
    return kquant


@pytest.mark.parametrize("ty", helpers.FORMATS)
def test_split_join_dequant_match_reference(kq, golden_dir, ty):
    g = helpers.golden(golden_dir, ty)
    n, k = g["q"].shape
    blocks = g["blocks"].reshape(-1, kq.BLOCK_BYTES[ty])
    q, side, bits = kq.split(ty, blocks)
    assert bits == kq.CODE_BITS[ty]
    assert np.array_equal(q.reshape(n, k), g["q"]) and np.array_equal(side.reshape(n, -1), g["side"])
    assert np.array_equal(kq.join(ty, q, side), blocks)                               # lossless
    assert np.array_equal(kq.dequant(ty, g["q"], g["side"]), g["w"])                  # bit-exact float32
    import gguf
    assert np.array_equal(kq.dequant(getattr(gguf.GGMLQuantizationType, ty), g["q"], g["side"]), g["w"])


def test_join_refuses_codes_outside_the_format(kq):
    import lazyweights_b200 as lw
    q = np.full((1, 256), 16, np.uint8)
    with pytest.raises(lw.LwError):
        kq.join("Q4_K", q, np.zeros((1, 16), np.uint8))
    assert kq.join("Q5_K", q, np.zeros((1, 16), np.uint8)).shape == (1, 176)


def test_split_join_random_roundtrip(kq):
    rng = np.random.default_rng(0)
    for ty in helpers.FORMATS:
        b = rng.integers(0, 256, (37, kq.BLOCK_BYTES[ty]), dtype=np.uint8)
        q, side, _ = kq.split(ty, b)
        assert q.max() < (1 << kq.CODE_BITS[ty])
        assert np.array_equal(kq.join(ty, q, side), b)


@pytest.mark.parametrize("case", sorted(synth_gguf.CASES))
def test_builder_writes_what_the_reference_writes(kq, golden_dir, tmp_path, case):
    import lazyweights_b200 as lw
    from lazyweights_b200 import gguf_bundle
    want = json.load(open(os.path.join(golden_dir, "gguf_bundles.json")))[case]
    path = str(tmp_path / (case + ".gguf"))
    synth_gguf.write(path, **synth_gguf.CASES[case])
    out = str(tmp_path / case)
    summary = gguf_bundle.build_bundle(path, out, check=True)
    cfg, ts = lw.bundle.read_manifest(out)
    for key, val in want["cfg"].items():
        assert int(float(cfg[key])) == val, key
    raw = open(os.path.join(out, "weights.bin"), "rb").read()
    got = [[t["name"], t["enc"], t["N"], t["K"], t["nbytes"],
            hashlib.sha256(raw[t["offset"]:t["offset"] + t["nbytes"]]).hexdigest()] for t in ts]
    assert [g[:5] for g in got] == [w[:5] for w in want["tensors"]]                   # names, order, shapes, sizes
    assert got == want["tensors"]                                                     # and every byte
    assert lw.lib().lw_validate_bundle(out.encode()) == 0, lw._native.last_error()    # the runtime would take it
    assert summary["embed_max_abs_err"] <= 1e-6


def test_unpermute_is_the_inverse_of_the_conversion_permute():
    from lazyweights_b200 import gguf_bundle
    rows = np.arange(8 * 128)
    inv = gguf_bundle.unpermute_index(rows.size, 8)
    assert np.array_equal(gguf_bundle.permute_rows(rows, 8)[inv], rows)
