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
            # the twin has the unit structure of the bundle's own code: same sums in the same order (a Q5_K / Q6_K
            # matrix with whole 512-weight tiles is otherwise read through its pair layout, whose units are wider)
            assert lw.lib().lw_debug_set(b"pairs", 0) == 0
            coded = mat.linear("m", x).cpu().numpy()
            assert lw.lib().lw_debug_set(b"pairs", 1) == 0
            twin = mat.linear_twin("m", x).cpu().numpy()[0]
            assert np.array_equal(twin, coded)
            assert helpers.rel_err(mat.linear("m", x).cpu().numpy(), coded) <= 1e-5
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
        env["LW_PAIRS"] = "0"   # both decoders read the bundle's own code (a pair layout has its own table reader)
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


DECODE_WORKER = r"""
import sys, numpy as np, torch
sys.path.insert(0, %r)
import lazyweights_b200 as lw
from tests import helpers
from oracle import lw_oracle as orc
for ty, n, k in %r:
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=3 * n + k)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
        assert np.array_equal(mat.decode_codes("m", expand=True).cpu().numpy(), q), ty
        assert np.array_equal(mat.decode_codes("m", expand=False).cpu().numpy(), sym), ty
        got = mat.decode_weights("m").cpu().numpy()
        assert np.array_equal(got.view(np.uint16), w.astype(np.float16).view(np.uint16)), ty
assert lw.lib().lw_kernel_error() == 0
print("ok")
"""


def test_decode_kernels_with_plain_stores(lw):
    """The decode kernels normally send their rows through shared memory and tensor copies; LW_TILE_OUT=0 (read once per
    process) keeps the 32-byte stores, which are also what a driver without the tensor-map encoder gets.  Same bits."""
    shapes = [("Q4_K", 128, 1024), ("Q5_K", 128, 1024), ("Q6_K", 192, 1536), ("IQ4_XS", 64, 2560), ("Q6_K", 64, 256)]
    env = dict(os.environ)
    env["LW_TILE_OUT"] = "0"
    r = subprocess.run([sys.executable, "-c", DECODE_WORKER % (ROOT, shapes)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


def test_decode_kernels_replayed_from_a_graph(lw):
    """Both decode kernels captured into a CUDA graph (their tensor maps travel as kernel parameters) and replayed into
    cleared buffers: same bits as the oracle."""
    import torch
    for ty, n, k in (("Q6_K", 256, 1024), ("Q4_K", 128, 1024)):
        q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=11 * n + k)
        blob, _, _ = lw.bundle.encode_huf8(sym)
        with lw.CodedMatrix(blob, n, sym.shape[1], ty, side) as mat:
            codes = torch.empty((n, k), dtype=torch.uint8, device="cuda")
            halves = torch.empty((n, k), dtype=torch.float16, device="cuda")
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                mat.decode_codes("m", expand=True, out=codes)              # first calls outside the capture
                mat.decode_weights("m", out=halves)
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    mat.decode_codes("m", expand=True, out=codes)
                    mat.decode_weights("m", out=halves)
                codes.zero_()
                halves.zero_()
                g.replay()
                stream.synchronize()
            assert np.array_equal(codes.cpu().numpy(), q), ty
            assert np.array_equal(halves.cpu().numpy().view(np.uint16), w.astype(np.float16).view(np.uint16)), ty
            del g
        assert lw.lib().lw_kernel_error() == 0


def test_batched_launch_equals_single_products(lw, tmp_path):
    """lw_linear_batch: several products in one launch (same format and plan), mixed formats (launched one by one),
    several matrices of one handle; results equal the single-product entry point's bit for bit."""
    import torch
    rng = np.random.default_rng(8)
    mats, entries, want = [], [], []
    for j, (ty, n, k) in enumerate([("Q6_K", 1024, 1024), ("Q6_K", 512, 1024), ("Q6_K", 2048, 512), ("Q6_K", 1024, 1024),
                                    ("Q4_K", 512, 2048), ("Q4_K", 256, 1024)]):
        q, side = orc.synth_codes(ty, n, k, rng), orc.synth_side(ty, n, k, rng)
        sym = orc.symbols_of(ty, q)
        blob, _, _ = lw.bundle.encode_huf8(sym)
        m = lw.CodedMatrix(blob, n, sym.shape[1], ty, side)
        x = torch.from_numpy(rng.standard_normal(k).astype(np.float16)).cuda()
        y = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
        mats.append(m)
        entries.append((m, "m", x, y))
        want.append(m.linear("m", x).cpu().numpy())
        assert helpers.rel_err(want[-1], orc.gemv_f64(orc.dequant(ty, q, side), x.cpu().numpy().astype(np.float32)[None])[0]) <= helpers.GEMV_TOL
    before = lw.lib().lw_launch_count()
    batch = lw.ProductBatch(entries)
    batch.launch()
    launches = lw.lib().lw_launch_count() - before
    plans = [(m.info("m")["fmt"], m.plan("m")["group"], m.plan("m")["index_bits"]) for m in mats]
    if len(set(plans[:4])) == 1:
        assert launches < len(entries)                                  # the like matrices went out together
    assert launches <= len(entries)
    for (m, _, _, y), w in zip(entries, want):
        assert np.array_equal(y.cpu().numpy(), w)
    for _, _, _, y in entries:
        y.fill_(float("nan"))
    batch.launch()                                                      # again: counters and scratch are left clean
    for (m, _, _, y), w in zip(entries, want):
        assert np.array_equal(y.cpu().numpy(), w)
    for m in mats:
        m.close()
    # several matrices of ONE handle share its scratch
    wr = lw.bundle.Writer(str(tmp_path / "b"))
    cases = {}
    for i in range(3):
        q, side = orc.synth_codes("Q5_K", 256, 1024, rng), orc.synth_side("Q5_K", 256, 1024, rng)
        wr.add_kquant("l%d.up" % i, "Q5_K", q, side)
        cases["l%d.up" % i] = (q, side)
    wr.close()
    with lw.Bundle(str(tmp_path / "b")) as b:
        x = torch.from_numpy(rng.standard_normal(1024).astype(np.float32)).cuda()
        ys = [torch.empty(256, dtype=torch.float32, device="cuda") for _ in cases]
        lw.ProductBatch([(b, name, x, y) for name, y in zip(cases, ys)]).launch()
        for (name, (q, side)), y in zip(cases.items(), ys):
            assert np.array_equal(y.cpu().numpy(), b.linear(name, x).cpu().numpy())
            assert helpers.rel_err(y.cpu().numpy(), orc.gemv_f64(orc.dequant("Q5_K", q, side), x.cpu().numpy()[None])[0]) <= helpers.GEMV_TOL


@pytest.mark.parametrize("ty,n,k", [("Q6_K", 512, 1024), ("Q4_K", 256, 2048), ("Q5_K", 256, 1024), ("IQ4_XS", 512, 1536),
                                     ("Q6_K", 1792, 512)])
def test_tensor_memory_gemm_path(lw, tmp_path, ty, n, k):
    """The decode + tcgen05 GEMM (decoded weights go from registers to tensor memory): every row count class from one
    row to 64, through the host-buffer entry point with path 3 and, for 9..64 rows, as the default path."""
    rng = np.random.default_rng(n + k)
    q, side = orc.synth_codes(ty, n, k, rng), orc.synth_side(ty, n, k, rng)
    hi = 15 if ty in ("Q4_K", "IQ4_XS") else (31 if ty == "Q5_K" else 63)
    q[:64, :128] = rng.integers(0, hi + 1, (64, 128))                   # a unit of rare codes: the fallback classes
    w = orc.dequant(ty, q, side)
    wr = lw.bundle.Writer(str(tmp_path / "b"))
    wr.add_kquant("l0.up", ty, q, side)
    wr.close()
    with lw.Bundle(str(tmp_path / "b")) as b:
        assert lw.lib().lw_debug_set(b"wait_limit", 200000) == 0        # a lost signal ends the kernel within a second
        for m in (1, 8, 9, 16, 17, 33, 48, 64):
            X = rng.standard_normal((m, k)).astype(np.float32)
            ref = orc.gemv_f64(w, X)
            try:
                got = b.matmul("l0.up", X, 3)
            except lw.LwError as e:
                # the unit of rare codes is several times the usual size: with many rows its staging ring may not fit
                # beside the activations; the default path then takes the decode + GEMM route by itself
                assert e.status == -5 and m > 32
                assert helpers.rel_err(b.matmul("l0.up", X, 0), ref) <= helpers.GEMV_TOL, (ty, m)
                continue
            assert helpers.rel_err(got, ref) <= helpers.GEMV_TOL, (ty, m)
            if m >= 8:
                before = lw.lib().lw_launch_count()
                auto = b.matmul("l0.up", X, 0)
                if m == 8:                                              # eight rows: the fused kernel is the faster one
                    assert helpers.rel_err(auto, ref) <= helpers.GEMV_TOL
                    assert lw.lib().lw_launch_count() - before == 2     # the fused product and the sum of its partial products
                    continue
                assert np.array_equal(auto, got)                        # the default path for 9 .. 64 rows is this kernel
                assert lw.lib().lw_launch_count() - before == 3         # range factors of fp32 rows, the GEMM, the sum of its planes
        assert b.kernel_error() == 0
        lw.lib().lw_debug_set(b"reset", 0)


@pytest.mark.parametrize("ty,n,k", [("Q4_K", 256, 2048), ("Q6_K", 512, 1024)])
def test_rows_beyond_half_range(lw, tmp_path, ty, n, k):
    """fp32 activations far outside fp16's range (the input of a down projection in an unnormalised model) through the
    paths that feed the tensor cores fp16: every row is brought into range by a power of two and the product scaled
    back, so the result is finite and as accurate as for ordinary rows; rows that fit are converted as they are."""
    rng = np.random.default_rng(n * 7 + k)
    q, side = orc.synth_codes(ty, n, k, rng), orc.synth_side(ty, n, k, rng)
    w = orc.dequant(ty, q, side)
    wr = lw.bundle.Writer(str(tmp_path / "b"))
    wr.add_kquant("l0.down", ty, q, side)
    wr.close()
    with lw.Bundle(str(tmp_path / "b")) as b:
        for m in (8, 33, 70):
            X = rng.standard_normal((m, k)).astype(np.float32)
            X[0] *= 3.0e5                                               # every entry of this row overflows fp16
            X[1, 5] = -7.0e7                                            # one outlier
            X[m - 1] *= 1.0e-3
            ref = orc.gemv_f64(w, X)
            for path in (0, 2) + ((3,) if m <= 64 else ()):
                got = b.matmul("l0.down", X, path)
                assert np.isfinite(got).all(), (ty, m, path)
                for r in range(m):                                      # row by row: the rows differ by 1e11 in size
                    assert helpers.rel_err(got[r], ref[r]) <= helpers.GEMV_TOL, (ty, m, path, r)
        assert b.kernel_error() == 0


@pytest.mark.parametrize("ty,n,k,narrow", [("Q6_K", 512, 1024, False), ("Q5_K", 256, 2048, False), ("Q6_K", 192, 1536, False),
                                            ("Q6_K", 256, 1024, True)])
def test_pair_layout_product(lw, tmp_path, ty, n, k, narrow):
    """Q6_K / Q5_K matrices whose rows are whole 512-weight tiles carry a pair layout that the one-row products read
    (two weights per table lookup): same product as through the bundle's own code, both against the oracle; single
    launch, batched launch and the allocation-free entry point."""
    import torch
    rng = np.random.default_rng(n + 3 * k)
    q, side = orc.synth_codes(ty, n, k, rng), orc.synth_side(ty, n, k, rng)
    hi = 31 if ty == "Q5_K" else 63
    if narrow:   # few different pairs: the pair code fits 11 bits and the kernel keeps 8 copies of a 2048-window table
        q = np.clip(np.rint(rng.normal(32.0, 1.5, q.shape)), 0, 63).astype(np.uint8)
    else:
        q[:64, :256] = rng.integers(0, hi + 1, (64, 256))               # rare pairs: the longest codes of the pair code
    w = orc.dequant(ty, q, side)
    wr = lw.bundle.Writer(str(tmp_path / "b"))
    wr.add_kquant("a", ty, q, side)
    wr.add_kquant("b", ty, q[::-1].copy(), side[::-1].copy())
    wr.close()
    with lw.Bundle(str(tmp_path / "b")) as b:
        assert b.pair_bytes("a") > 0
        for dt in (np.float32, np.float16):
            x = rng.standard_normal(k).astype(dt)
            xd = torch.from_numpy(x).cuda()
            ref = orc.gemv_f64(w, x.astype(np.float32)[None])[0]
            y_pair = b.linear("a", xd).cpu().numpy()
            assert lw.lib().lw_debug_set(b"pairs", 0) == 0
            y_code = b.linear("a", xd).cpu().numpy()
            assert lw.lib().lw_debug_set(b"pairs", 1) == 0
            assert helpers.rel_err(y_pair, ref) <= helpers.GEMV_TOL and helpers.rel_err(y_code, ref) <= helpers.GEMV_TOL
            assert helpers.rel_err(y_pair, y_code) <= 1e-5              # same integer sums, another order of float adds
        x = torch.from_numpy(rng.standard_normal(k).astype(np.float32)).cuda()
        ya, yb = (torch.empty(n, dtype=torch.float32, device="cuda") for _ in range(2))
        lw.ProductBatch([(b, "a", x, ya), (b, "b", x, yb)]).launch()
        assert np.array_equal(ya.cpu().numpy(), b.linear("a", x).cpu().numpy())
        assert helpers.rel_err(yb.cpu().numpy(), orc.gemv_f64(w[::-1], x.cpu().numpy()[None])[0]) <= helpers.GEMV_TOL
        X = rng.standard_normal((3, k)).astype(np.float32)              # the several-row kernel reads the pair layout too
        assert helpers.rel_err(b.matmul("a", X), orc.gemv_f64(w, X)) <= helpers.GEMV_TOL
        assert np.array_equal(b.decode("a"), q)                         # decode to codes: two codes per lookup,
        assert lw.lib().lw_debug_set(b"pairs", 0) == 0
        assert np.array_equal(b.decode("a"), q)                         # and through the bundle's own code
        assert lw.lib().lw_debug_set(b"pairs", 1) == 0
        assert b.kernel_error() == 0
