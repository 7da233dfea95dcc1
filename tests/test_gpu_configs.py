"""Parity at the benchmark's own configurations (full sizes), through the C ABI on a real GPU.

The oracle is too slow to dequantise whole 14336 x 4096 matrices in a test, so every case checks sampled rows:
fp16 weights bit-exact against the oracle's float32 block arithmetic, products within 1e-3 (the reference check's
max-norm definition, kernels/llmrt.cu:2868-2874) of a float64 product of the oracle's exact float32 weights.
"""
import numpy as np
import pytest

from oracle import lw_oracle as orc
from tests import helpers
from tests.test_runtime import ref_forward

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lw():
    helpers.build_library()
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import lazyweights_b200 as pkg
    yield pkg
    assert pkg.lib().lw_kernel_error() == 0


def _bits16(a):
    return np.ascontiguousarray(a).view(np.uint16)


CASES = [
    ("Q6_K", 14336, 4096, (1, 8, 33)),      # the single-matrix configuration: batch 1, batch 8, tensor-core path
    ("IQ4_XS", 3072, 3072, (1, 8)),         # Phi-3-mini shapes: o projection, FFN up, verify pass of eight tokens
    ("IQ4_XS", 8192, 3072, (1, 8)),
    ("Q5_K", 4096, 4096, (1, 8, 32)),       # mixed-format decoder: attention q / o, k / v
    ("Q5_K", 1024, 4096, (1, 8)),
    ("Q4_K", 4096, 14336, (1, 8)),          # FFN down of the Q4_K decoder (28 tile columns)
]


@pytest.mark.parametrize("ty,n,k,ms", CASES)
def test_full_size_sampled_rows(lw, ty, n, k, ms):
    import torch
    rng = np.random.default_rng(n + k)
    q, side = orc.synth_codes(ty, n, k, rng), orc.synth_side(ty, n, k, rng)
    sym = orc.symbols_of(ty, q)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    rows = np.sort(rng.choice(n, 96, replace=False))
    w_ref = orc.dequant(ty, q[rows], side[rows])
    with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
        w16 = mat.decode_weights("m")[torch.from_numpy(rows).cuda()].cpu().numpy()
        assert np.array_equal(_bits16(w16), _bits16(w_ref.astype(np.float16)))
        for m in ms:
            x = rng.standard_normal((m, k)).astype(np.float16)
            y = mat.linear("m", torch.from_numpy(x).cuda()).cpu().numpy()
            ref = x.astype(np.float64) @ w_ref.astype(np.float64).T
            assert np.abs(y[:, rows] - ref).max() <= helpers.GEMV_TOL * np.abs(ref).max(), (ty, n, k, m)
            if m in (8, 32, 33):                                   # the host-buffer call, all three paths
                for path in (1, 2):
                    yh = mat.matmul("m", x.astype(np.float32), path)
                    assert np.abs(yh[:, rows] - ref).max() <= helpers.GEMV_TOL * np.abs(ref).max(), (ty, m, path)


@pytest.mark.parametrize("ty,n,k", [("Q6_K", 512, 4096), ("Q4_K", 256, 4096), ("Q5_K", 256, 2048), ("IQ4_XS", 256, 3072)])
@pytest.mark.parametrize("m", [1, 8])
def test_heavy_tailed_activations(lw, ty, n, k, m):
    """One 100x outlier in every sub-block is the worst case of the 16-bit block fixed point the fused kernels use for
    the activations (one scale per sub-block): the product must still meet the 1e-3 bar."""
    import torch
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=17 * m + k)
    sub = 16 if ty == "Q6_K" else 32
    x = rng.standard_normal((m, k)).astype(np.float32)
    pos = np.arange(0, k, sub)[None, :] + rng.integers(0, sub, (m, k // sub))
    x[np.arange(m)[:, None], pos] *= 100.0
    blob, _, _ = lw.bundle.encode_huf8(sym)
    with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
        y = mat.linear("m", torch.from_numpy(x).cuda()).cpu().numpy()
        assert helpers.rel_err(y, orc.gemv_f64(w, x)) <= helpers.GEMV_TOL
        # and a single outlier in the whole row (every other sub-block keeps its own fine scale)
        x2 = rng.standard_normal((m, k)).astype(np.float32)
        x2[:, k // 3] = 1000.0
        y2 = mat.linear("m", torch.from_numpy(x2).cuda()).cpu().numpy()
        assert helpers.rel_err(y2, orc.gemv_f64(w, x2)) <= helpers.GEMV_TOL


REAL = dict(n_layers=2, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, inter=14336, vocab=32000, eps=1e-5, theta=1e6)


@pytest.mark.parametrize("fmt_attn,fmt_ffn", [("Q4_K", "Q4_K"), ("Q5_K", "Q6_K")])
def test_decoder_at_real_width(lw, tmp_path, fmt_attn, fmt_ffn):
    """Two layers of the Mistral-7B shape (d 4096, 32 / 8 heads, FFN 14336, vocabulary 32000): last-token logits of a
    six-token pass and of a following single-token pass against the float64 NumPy model on the oracle's weights."""
    from lazyweights_b200 import modelgen
    W = modelgen.write_model(str(tmp_path / "m"), REAL, fmt_attn, fmt_ffn, seed=11, return_weights=True)
    ids = np.random.default_rng(4).integers(0, REAL["vocab"], 7).astype(np.int32)
    ref = ref_forward(W, ids, REAL)
    with lw.Bundle(str(tmp_path / "m"), max_ctx=32, max_batch=8) as b:
        got6 = b.forward(ids[:6])
        got7 = b.forward(ids[6:])
        assert helpers.rel_err(got6, ref[5]) <= 5e-3
        assert helpers.rel_err(got7, ref[6]) <= 5e-3
        assert int(got7.argmax()) == int(ref[6].argmax())
        assert b.kernel_error() == 0
