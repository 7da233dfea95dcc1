"""lw_linear_static: the product for callers that may not allocate (a serving loop whose memory is already handed out,
a plug-in under a host that owns the device heap).  It must give what lw_linear gives, call after call, from the
scratch array built into the library.  Collected last on purpose: a failure here cannot hide any other test."""
import numpy as np
import pytest

from oracle import lw_oracle as orc
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ty,n,k", [("Q6_K", 256, 1024), ("Q4_K", 192, 2048)])
def test_static_scratch_matches_lw_linear(ty, n, k):
    helpers.build_library()
    import torch
    import lazyweights_b200 as lw
    assert torch.cuda.is_available()
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=4242)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
        for m_rows in (1, 5):
            x = torch.from_numpy(rng.standard_normal((m_rows, k)).astype(np.float16)).cuda()
            ref = mat.linear("m", x).cpu().numpy()
            out = torch.full((m_rows, n), float("nan"), dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            before = torch.cuda.memory_allocated()
            first = mat.linear_static("m", x, out).cpu().numpy().copy()
            out.fill_(float("nan"))
            second = mat.linear_static("m", x, out).cpu().numpy()          # second call: the scratch is reused as is
            assert torch.cuda.memory_allocated() == before
            for got in (first, second):
                assert np.isfinite(got).all()
                assert helpers.rel_err(got, ref) <= 1e-6                   # same kernels, same order of sums
                assert helpers.rel_err(got, orc.gemv_f64(w, x.cpu().numpy().astype(np.float32))) <= helpers.GEMV_TOL
        with pytest.raises(lw.LwError) as e:                               # more than eight rows is refused, not grown
            mat.linear_static("m", torch.zeros((9, k), dtype=torch.float16, device="cuda"),
                              torch.empty((9, n), dtype=torch.float32, device="cuda"))
        assert e.value.status == -2
    assert lw.lib().lw_kernel_error() == 0
