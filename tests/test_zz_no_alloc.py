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
            host = torch.empty((2, m_rows, n), dtype=torch.float32).pin_memory()
            mat.linear_static("m", x, out)                                 # first call on the device: address look-up
            torch.cuda.synchronize()
            # free device memory as the driver sees it: a cudaMalloc anywhere in the call (this library's, or a
            # library's it calls) would lower it, which torch's allocator statistics cannot show
            free_before = torch.cuda.mem_get_info()[0]
            out.fill_(float("nan"))
            mat.linear_static("m", x, out)
            host[0].copy_(out)
            out.fill_(float("nan"))
            mat.linear_static("m", x, out)                                 # again: the scratch is reused as is
            host[1].copy_(out)
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before
            first, second = host[0].numpy(), host[1].numpy()
            for got in (first, second):
                assert np.isfinite(got).all()
                assert helpers.rel_err(got, ref) <= 1e-6                   # same kernels, same order of sums
                assert helpers.rel_err(got, orc.gemv_f64(w, x.cpu().numpy().astype(np.float32))) <= helpers.GEMV_TOL
        with pytest.raises(lw.LwError) as e:                               # more than eight rows is refused, not grown
            mat.linear_static("m", torch.zeros((9, k), dtype=torch.float16, device="cuda"),
                              torch.empty((9, n), dtype=torch.float32, device="cuda"))
        assert e.value.status == -2
    assert lw.lib().lw_kernel_error() == 0
