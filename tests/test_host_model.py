"""Host-side validation of model bundles (no GPU): a manifest whose cfg and tensor shapes disagree must be refused
before anything is uploaded; rt_open runs the same check.  Also the plan limits of the fused kernels' launchers are
exercised through the library's test switches in the GPU suite; here only the argument checks of the switches."""
import os
import shutil

import pytest

from tests import helpers

SHAPE = dict(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, inter=1024, vocab=512, eps=1e-5, theta=1e4)


@pytest.fixture(scope="module")
def bundle_dir(tmp_path_factory):
    helpers.build_library()
    from lazyweights_b200 import modelgen
    d = tmp_path_factory.mktemp("model") / "m"
    modelgen.write_model(str(d), SHAPE, "Q4_K", "Q6_K", seed=3)
    return str(d)


def _doctor(src, dst, edit):
    shutil.copytree(src, dst)
    path = os.path.join(dst, "manifest.txt")
    lines = open(path).read().splitlines()
    open(path, "w").write("\n".join(edit(lines)) + "\n")
    return dst


def _status(path):
    import lazyweights_b200 as lw
    return lw.lib().lw_validate_bundle(os.fsencode(path))


def test_good_bundle_validates(bundle_dir):
    assert _status(bundle_dir) == 0


@pytest.mark.parametrize("what", ["vocab", "hidden", "inter", "heads", "norm", "rope", "missing", "truncated", "embed_cols"])
def test_doctored_manifests_are_refused(bundle_dir, tmp_path, what):
    import lazyweights_b200 as lw

    def edit(lines):
        out = []
        for ln in lines:
            p = ln.split()
            if what == "vocab" and p[:2] == ["cfg", "vocab"]:
                p[2] = "1024"                                   # lm_head has 512 rows
            elif what == "hidden" and p[:2] == ["cfg", "hidden"]:
                p[2] = "1024"
            elif what == "inter" and p[:2] == ["cfg", "inter"]:
                p[2] = "2048"
            elif what == "heads" and p[:2] == ["cfg", "n_heads"]:
                p[2] = "8"                                      # qkv would need more rows than it has
            elif what == "norm" and p[0] == "t" and p[1] == "l1.ln2":
                p[4] = "256"
            elif what == "rope" and p[0] == "t" and p[1] == "sin":
                p[4] = "32"
            elif what == "missing" and p[0] == "t" and p[1] in ("l0.down", "l0.down.kqs"):
                continue
            elif what == "truncated" and p[0] == "t" and p[1] == "lm_head":
                p[7] = str(int(p[7]) + (1 << 30))               # offset beyond the end of weights.bin
                p[7] = str(int(p[7]) // 256 * 256)
            elif what == "embed_cols" and p[0] == "t" and p[1] == "embed":
                p[4] = "256"
            out.append(" ".join(p))
        return out

    bad = _doctor(bundle_dir, str(tmp_path / what), edit)
    assert _status(bad) == -3, lw._native.last_error()
    assert lw._native.last_error()


def test_debug_switch_arguments():
    import lazyweights_b200 as lw
    L = lw.lib()
    assert L.lw_debug_set(b"max_units", 64) == 0
    assert L.lw_debug_set(b"max_units", 1) == -2 and L.lw_debug_set(b"max_units", 4096) == -2
    assert L.lw_debug_set(b"wait_limit", 1000) == 0 and L.lw_debug_set(b"wait_limit", 0) == -2
    assert L.lw_debug_set(b"drop_unit", 3) == 0 and L.lw_debug_set(b"nonsense", 1) == -2
    assert L.lw_debug_set(b"reset", 0) == 0


def test_array_addresses_of_the_host_buffer_calls():
    """The host-buffer wrappers hand NumPy arrays to the C ABI by address; the quick route (a ctypes view of the buffer)
    and its fallback for read-only arrays must give the address NumPy itself reports."""
    import numpy as np
    helpers.build_library()
    from lazyweights_b200 import runtime
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    assert runtime._address(a) == a.ctypes.data
    assert runtime._address(a[1:]) == a.ctypes.data + 16            # a contiguous view starts at its own first byte
    frozen = a.copy()
    frozen.setflags(write=False)
    assert runtime._address(frozen) == frozen.ctypes.data
