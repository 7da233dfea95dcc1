"""Paths that ordinary products do not reach: very tall matrices (several launches per product), waits that run out,
token ids outside the embedding, a handle used from the wrong device.  Nothing here faults or hangs a GPU: the waits
that run out are bounded by a small poll limit and the kernels return."""
import numpy as np
import pytest

from oracle import lw_oracle as orc
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture()
def lw():
    helpers.build_library()
    import torch
    assert torch.cuda.is_available()
    import lazyweights_b200 as pkg
    pkg.lib().lw_kernel_error()
    yield pkg
    pkg.lib().lw_debug_set(b"reset", 0)
    assert pkg.lib().lw_kernel_error() == 0


@pytest.mark.parametrize("ty,n,k", [("Q6_K", 4096, 2048), ("Q4_K", 2048, 4096), ("Q5_K", 4096, 2048)])
def test_products_over_several_launches(lw, ty, n, k):
    """With the per-block unit list capped at a few units a product runs as many launches over ranges of tile rows,
    the way a matrix with more tile rows than one list holds does; results must not change."""
    import torch
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=n + 3 * k)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
        x = torch.from_numpy(rng.standard_normal((8, k)).astype(np.float16)).cuda()
        want1, want8 = mat.linear("m", x[0]).cpu().numpy(), mat.linear("m", x).cpu().numpy()
        before = lw.lib().lw_launch_count()
        mat.linear("m", x[0])
        one = lw.lib().lw_launch_count() - before
        assert lw.lib().lw_debug_set(b"max_units", 4) == 0                # 256 or 512 tiles (of 512 weights for the one-row product), at most 148 per launch
        before = lw.lib().lw_launch_count()
        got1 = mat.linear("m", x[0]).cpu().numpy()
        assert lw.lib().lw_launch_count() - before > one                  # really several launches
        got8 = mat.linear("m", x).cpu().numpy()
        assert np.array_equal(got1, want1) and np.array_equal(got8, want8)
        assert helpers.rel_err(got8, orc.gemv_f64(w, x.cpu().numpy().astype(np.float32))) <= helpers.GEMV_TOL


def test_wait_probe_gives_up_and_library_recovers(lw):
    import torch
    assert lw.lib().lw_debug_wait_probe(1000) == 3                        # both kinds of wait ran out and returned
    assert lw.lib().lw_kernel_error() == 1                                # reported ...
    assert lw.lib().lw_kernel_error() == 0                                # ... and cleared
    q, side, sym, w, rng = helpers.seeded_case("Q6_K", 256, 1024, seed=5)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    with lw.CodedMatrix(blob, 256, sym.shape[1], "Q6_K", side) as mat:
        x = rng.standard_normal(1024).astype(np.float32)
        y = mat.linear("m", torch.from_numpy(x).cuda()).cpu().numpy()
        assert helpers.rel_err(y, orc.gemv_f64(w, x[None])[0]) <= helpers.GEMV_TOL


@pytest.mark.parametrize("ty,n,k", [("Q6_K", 4096, 1024), ("Q4_K", 2048, 2048)])
def test_lost_copy_ends_the_kernel_and_next_product_is_right(lw, ty, n, k):
    """A copy that never arrives: block 0 skips one unit of its list, the waits for it run out after 2000 polls, the
    kernel returns with the error word set (its result is void), and the next product of the same matrix - whose
    tile-row counters the failed launch left non-zero - is correct again."""
    import torch
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=n + k)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
        x = torch.from_numpy(rng.standard_normal(k).astype(np.float32)).cuda()
        want = mat.linear("m", x).cpu().numpy()
        L = lw.lib()
        assert L.lw_debug_set(b"wait_limit", 2000) == 0 and L.lw_debug_set(b"drop_unit", 1) == 0
        mat.linear("m", x)
        torch.cuda.synchronize()                                          # the kernel came back by itself
        assert L.lw_debug_set(b"reset", 0) == 0
        assert L.lw_kernel_error() == 1
        for _ in range(2):
            got = mat.linear("m", x).cpu().numpy()
            assert np.array_equal(got, want)
        assert L.lw_kernel_error() == 0


def test_token_ids_outside_the_embedding_are_refused(lw, tmp_path):
    from lazyweights_b200 import modelgen
    from tests.test_runtime import SHAPE
    modelgen.write_model(str(tmp_path / "m"), SHAPE, "Q4_K", "Q4_K", seed=3)
    with lw.Bundle(str(tmp_path / "m"), max_ctx=64, max_batch=8) as b:
        for bad in ([SHAPE["vocab"]], [-1], [0, 1, 1 << 30]):
            with pytest.raises(lw.LwError) as e:
                b.forward(np.array(bad, np.int32))
            assert e.value.status == -2
        assert b.pos == 0
        ok = b.forward(np.array([1, 2, 3], np.int32))                     # nothing was launched by the refused calls
        assert np.isfinite(ok).all() and b.pos == 3


def test_handle_is_bound_to_its_device(lw):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    q, side, sym, w, rng = helpers.seeded_case("Q6_K", 128, 512, seed=1)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    torch.cuda.set_device(0)
    with lw.CodedMatrix(blob, 128, sym.shape[1], "Q6_K", side) as mat:
        x1 = torch.zeros(512, device="cuda:1")
        torch.cuda.set_device(1)
        try:
            with pytest.raises(lw.LwError) as e:
                mat.linear("m", x1)
            assert e.value.status == -2
        finally:
            torch.cuda.set_device(0)
