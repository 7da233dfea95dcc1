"""CPU-side checks: the library builds, loads and exports the declared C ABI; its host codec (encoder, validator,
threaded decoder, bundle reader) agrees with the reference-made golden vectors; GPU entry points refuse to run
without a device instead of falling back."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import lw_oracle as orc
from tests import helpers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lwlib():
    helpers.build_library()
    from lazyweights_b200 import _native
    return _native


def test_library_exports_every_declared_symbol(lwlib):
    header = open(os.path.join(ROOT, "include", "lwb200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b((?:rt|lw)_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 19
    raw = ctypes.CDLL(lwlib.LIB_PATH)
    missing = [n for n in sorted(declared) if not hasattr(raw, n)]
    assert not missing, missing
    assert declared == set(lwlib.exported_names())          # the Python binding covers the whole header


@pytest.mark.parametrize("ty", helpers.FORMATS)
def test_encoder_is_byte_exact(lwlib, golden_dir, ty):
    from lazyweights_b200 import bundle
    g = helpers.golden(golden_dir, ty)
    blob, bits, hist = bundle.encode_huf8(g["sym"])
    assert blob == g["blob"].tobytes() and bits == int(g["nbits"]) and np.array_equal(hist, g["hist"])
    bundle.validate_huf8(blob, *g["sym"].shape)
    assert np.array_equal(bundle.cpu_decode_huf8(blob, *g["sym"].shape, threads=3), g["decoded"])


@pytest.mark.parametrize("name", ["single", "uniform256", "two", "skewed"])
def test_edge_blobs(lwlib, golden_dir, name):
    from lazyweights_b200 import bundle
    g = np.load(os.path.join(golden_dir, "edge_%s.npz" % name))
    blob, bits, _ = bundle.encode_huf8(g["sym"])
    assert blob == g["blob"].tobytes() and bits == int(g["nbits"])
    bundle.validate_huf8(blob, *g["sym"].shape)
    assert np.array_equal(bundle.cpu_decode_huf8(blob, *g["sym"].shape), g["sym"])


def test_encoder_matches_oracle_on_random_tables(lwlib):
    from lazyweights_b200 import bundle
    rng = np.random.default_rng(21)
    for trial in range(6):
        nsym = int(rng.integers(2, 257))
        p = rng.dirichlet(np.full(nsym, 0.05 + trial * 0.3))
        sym = rng.choice(nsym, (64, 256 * (1 + trial % 2)), p=p).astype(np.uint8)
        blob, bits, _ = bundle.encode_huf8(sym)
        oblob, obits, _ = orc.encode_huf8(sym)
        assert blob == oblob and bits == obits


def test_shape_errors(lwlib):
    from lazyweights_b200 import bundle
    with pytest.raises(AssertionError):
        bundle.encode_huf8(np.zeros((63, 256), np.uint8))
    with pytest.raises(lwlib.LwError) as e:
        bundle.validate_huf8(b"\0" * 100, 64, 256)
    assert e.value.status == lwlib.LW_ERR_FORMAT


def test_validator_rejects_corruption(lwlib, golden_dir):
    """Fault injection on the host: corrupted bytes must be caught before anything reaches a GPU."""
    from lazyweights_b200 import bundle
    g = helpers.golden(golden_dir, "Q6_K")
    n, k = g["sym"].shape
    good = bytearray(g["blob"].tobytes())
    tiles = (n // 64) * (k // 256)

    def status(b):
        try:
            bundle.validate_huf8(bytes(b), n, k)
            return 0
        except lwlib.LwError as err:
            return err.status

    assert status(good) == 0
    bad = bytearray(good); bad[1] = 12                       # table entry with length 12
    assert status(bad) == lwlib.LW_ERR_FORMAT
    bad = bytearray(good); bad[0] ^= 1                       # wrong symbol in one table entry
    assert status(bad) == lwlib.LW_ERR_FORMAT
    bad = bytearray(good); bad[4096 + 4 * 5] ^= 4            # one lane offset moved
    assert status(bad) == lwlib.LW_ERR_FORMAT
    bad = bytearray(good); bad[4096:4100] = (7).to_bytes(4, "little")   # first lane not at bit 0
    assert status(bad) == lwlib.LW_ERR_FORMAT
    assert status(good[:-4]) == lwlib.LW_ERR_FORMAT          # payload one word short
    assert status(good + b"\0\0\0\0") == lwlib.LW_ERR_FORMAT
    assert status(good[:4096 + tiles * 128 + 4]) == lwlib.LW_ERR_FORMAT
    # (a flipped payload bit is not detectable in general: the result is another valid stream)
    bad = bytearray(good); bad[4096 + 4 * 40:4096 + 4 * 41] = (2 ** 32 - 64).to_bytes(4, "little")
    assert status(bad) == lwlib.LW_ERR_FORMAT               # a lane that starts beyond the payload


def test_writer_and_manifest(lwlib, tmp_path):
    from lazyweights_b200 import bundle
    rng = np.random.default_rng(9)
    q = orc.synth_codes("Q4_K", 64, 512, rng)
    side = orc.synth_side("Q4_K", 64, 512, rng)
    w = bundle.Writer(str(tmp_path / "b"))
    w.cfg("hidden", 512)
    w.add_kquant("l0.o", "Q4_K", q, side)
    w.close()
    assert bundle.read_manifest(str(tmp_path / "b")) == orc.read_manifest(str(tmp_path / "b"))
    # identical bytes to a bundle written by the oracle's writer
    o = orc.BundleWriter(str(tmp_path / "o"))
    o.cfg("hidden", 512)
    o.add_matrix("l0.o", "Q4_K", q, side)
    o.close()
    for f in ("manifest.txt", "weights.bin"):
        assert open(tmp_path / "b" / f, "rb").read() == open(tmp_path / "o" / f, "rb").read()


def test_gpu_entry_points_fail_loudly_without_device(lwlib, golden_dir, tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from lazyweights_b200 import bundle, runtime
    g = helpers.golden(golden_dir, "Q5_K")
    with pytest.raises(lwlib.LwError) as e:
        bundle.decode_huf8(g["blob"].tobytes(), *g["sym"].shape)
    assert e.value.status == lwlib.LW_ERR_NO_DEVICE
    w = bundle.Writer(str(tmp_path / "b"))
    w.add_kquant("m", "Q5_K", g["q"], g["side"])
    w.close()
    with pytest.raises(lwlib.LwError):
        runtime.Bundle(str(tmp_path / "b"))


def test_encoder_bytes_do_not_depend_on_the_threads(monkeypatch):
    """The encoder packs ranges of tiles side by side (LW_THREADS host threads) and ORs the words two ranges share:
    one thread, a few, and more threads than tiles must give the same bytes."""
    helpers.build_library()
    import lazyweights_b200 as lw
    rng = np.random.default_rng(8)
    sym = np.clip(np.rint(rng.laplace(100.0, 6.0, (192, 768))), 0, 255).astype(np.uint8)   # 3 x 3 tiles, long and short words
    blobs = []
    for threads in ("1", "2", "5", "64"):
        monkeypatch.setenv("LW_THREADS", threads)
        blob, _, bits = lw.bundle.encode_huf8(sym)
        blobs.append(bytes(blob))
    assert all(b == blobs[0] for b in blobs[1:])
    assert np.array_equal(orc.decode_huf8(blobs[0], *sym.shape), sym)
