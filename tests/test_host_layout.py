"""The load-time device layout, checked on the CPU: the batch-1 kernel's grouped bit arithmetic is replayed in Python
on the words the host produced, unit by unit, with the unit class the host assigned; it must return every symbol.
Also: the scales stored behind every work unit equal the oracle's sub-block scales."""
import os

import numpy as np
import pytest

from tests import helpers
from oracle import lw_oracle as orc

M32 = 0xFFFFFFFF


def _funnel(lo, hi, s):
    return (((hi << 32) | lo) >> (s & 31)) & M32


def _replay_chain(words, base, lane, lut, pad, index_bits, nsym, group, cls):
    """symbols of one chain, decoded the way the kernel does for unit class `cls` (lw_ring.cuh: GroupChain).  The
    kernel keeps 16 copies of a 1024-window table and 8 of a 2048-window one; with 8 it starts one bit into the
    chain's pad, which puts the window one bit lower in the shifted word."""
    w = lambda i: int(words[base + 32 * i + lane])
    bp0 = 1 if index_bits == 11 else 0
    pad -= bp0
    w0, w1, w2, nxt, bp = w(0), w(1), w(2), 3, bp0
    out = []
    if cls == 2:                                   # symbol by symbol, single-copy table of all 2048 windows
        for _ in range(nsym):
            e = int(lut[(_funnel(w0, w1, bp) >> pad) & 2047])
            out.append(e & 255)
            bp += e >> 8
            if bp >= 32:
                bp, w0, w1, w2, nxt = bp - 32, w1, w2, w(nxt), nxt + 1
        return out
    g = group if cls == 0 else 2
    a = b = off = 0
    for i in range(nsym):
        if i % g == 0:
            a, b, off = _funnel(w0, w1, bp), _funnel(w1, w2, bp), 0
        assert off < 32 or cls != 0 or True
        t = _funnel(a, b, off)                     # the kernel's funnel shift takes the offset modulo 32
        e = int(lut[(t >> pad) & ((1 << index_bits) - 1)])
        out.append(e & 255)
        off += e >> 8
        if i % g == g - 1 or i == nsym - 1:
            bp += off
            if bp >= 32:                           # ONE refill per group
                bp, w0, w1, w2, nxt = bp - 32, w1, w2, w(nxt), nxt + 1
    return out


def _tail_block(ty, q, rng, rows, cols):
    tails = {"Q4_K": [0, 1, 2, 14, 15], "IQ4_XS": [0, 1, 2, 14, 15], "Q5_K": [0, 1, 2, 3, 4, 5, 27, 28, 29, 30, 31],
             "Q6_K": list(range(0, 11)) + list(range(54, 64))}[ty]
    q[rows, cols] = rng.choice(tails, q[rows, cols].shape)


@pytest.mark.parametrize("ty,n,k", [("Q6_K", 128, 512), ("Q4_K", 64, 1024), ("Q5_K", 64, 512), ("IQ4_XS", 64, 1024)])
@pytest.mark.parametrize("force", [None, ("max", "10"), ("max", "11"), ("3", "11")])
@pytest.mark.parametrize("recode", ["1", "0"])
def test_grouped_decoder_replayed_on_cpu(monkeypatch, ty, n, k, force, recode):
    """recode 1: the loader's default, the matrix re-coded with words of at most 10 bits where the bundle's code has
    11-bit words; 0: the bundle's own code (whose long words make symbol-by-symbol units under a 10-bit table)."""
    helpers.build_library()
    import lazyweights_b200 as lw
    monkeypatch.setenv("LW_RECODE", recode)
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=17 + n + k)
    _tail_block(ty, q, rng, slice(0, 64), slice(64, 128))        # long codes back to back in one unit
    sym = orc.symbols_of(ty, q)
    if force:
        gmax = "4" if ty in ("Q4_K", "IQ4_XS") else "6"
        monkeypatch.setenv("LW_GEMV1_G", gmax if force[0] == "max" else force[0])
        monkeypatch.setenv("LW_GEMV1_IDX", force[1])
    blob, _, _ = lw.bundle.encode_huf8(sym)
    lay = lw.bundle.host_layout(blob, n, sym.shape[1], ty, side)
    lut = lay["lut"]                                              # the blob's table, or the re-coded layout's
    own = np.frombuffer(blob, np.uint16, 2048)
    if recode == "0" or (own >> 8).max() <= 10:
        assert np.array_equal(lut, own) and lay["max_len"] == (own >> 8).max()
    else:
        assert lay["max_len"] <= 10 and (lut >> 8).max() <= 10 and not np.array_equal(lut, own)
    split, pad, group, ib = lay["split"], lay["pad"], lay["group"], lay["index_bits"]
    assert group >= 3 and ib in (10, 11) and pad == 6 and split == (2 if ty == "Q5_K" else 4)
    if force:
        assert str(ib) == force[1]
    nsym = 256 // split
    KT, G = sym.shape[1] // 256, 2 * split
    seen = set()
    for t in range((n // 64) * KT):
        tr, tc = divmod(t, KT)
        for seg in range(split):
            cls = int(lay["unit_class"][t * split + seg])
            seen.add(cls)
            for half in range(2):
                base = int(lay["group_base"][t * G + 2 * seg + half])
                for lane in range(0, 32, 5 if cls == 0 else 1):          # every lane of the fallback units
                    got = _replay_chain(lay["words"], base, lane, lut, pad, ib, nsym, group, cls)
                    row = tr * 64 + half * 32 + lane
                    want = sym[row, tc * 256 + seg * nsym: tc * 256 + (seg + 1) * nsym]
                    assert got == want.tolist(), (t, seg, half, lane, cls)
    if force and force[0] == "max":
        assert seen - {0}, "forcing the largest group must leave some units on a fallback class"


@pytest.mark.parametrize("ty,n,k", [("Q6_K", 64, 512), ("Q4_K", 64, 1024), ("Q5_K", 64, 512), ("IQ4_XS", 64, 1024)])
def test_unit_scales_follow_the_chains(ty, n, k):
    helpers.build_library()
    import lazyweights_b200 as lw
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=5)
    blob, _, _ = lw.bundle.encode_huf8(sym)
    lay = lw.bundle.host_layout(blob, n, sym.shape[1], ty, side)
    split, sw = lay["split"], lay["unit_side_words"]
    assert sw == (96 if ty in ("Q6_K", "IQ4_XS") else 192)
    s_ref, o_ref = orc.sub_scales(ty, side.reshape(n * k // 256, -1))     # [blocks, sub-blocks]
    nsub = s_ref.shape[1]
    s_ref, o_ref = s_ref.reshape(n, -1), o_ref.reshape(n, -1)             # [row, sub-block along the row]
    KT, G = sym.shape[1] // 256, 2 * split
    subs_per_tile = (512 if ty in ("Q4_K", "IQ4_XS") else 256) // (16 if ty == "Q6_K" else 32)
    words = lay["words"]
    for t in range(KT * (n // 64)):
        tr, tc = divmod(t, KT)
        for seg in range(split):
            end = int(lay["group_base"][t * G + 2 * seg + 2])            # the scales are the unit's last words
            sb = words[end - sw:end]
            for r in range(64):
                sub0 = tc * subs_per_tile + seg * 4
                if ty in ("Q4_K", "Q5_K"):
                    dd = np.array([sb[r]], np.uint32).view(np.float16).astype(np.float32)
                    sc = np.array([sb[64 + r]], np.uint32).view(np.uint8).astype(np.float32)
                    mn = np.array([sb[128 + r]], np.uint32).view(np.uint8).astype(np.float32)
                    s, o = dd[0] * sc, dd[1] * mn
                else:
                    d = sb.view(np.float16)[128 + r].astype(np.float32)
                    b = np.array([sb[r]], np.uint32).view(np.int8 if ty == "Q6_K" else np.uint8).astype(np.float32)
                    s, o = d * (b - (32 if ty == "IQ4_XS" else 0)), np.zeros(4, np.float32)
                assert np.array_equal(s.astype(np.float32), s_ref[tr * 64 + r, sub0:sub0 + 4])
                assert np.array_equal(o.astype(np.float32), o_ref[tr * 64 + r, sub0:sub0 + 4])


def _replay_pair_chain(words, base, lane, table, pad, index_bits, nsym, group):
    """pair symbols (value bytes) of one chain of a pair layout, read the way the kernel's reload readers do.  A
    12-bit code (pad 6, 4 copies of a 4096-window table): every group loads three words at the word its bit position has
    reached and starts 4 - log2(copies) bits into the pad.  An 11-bit code is laid out without pad: a group loads two
    words, which always hold the 33 bits three symbols can take."""
    two_words = pad == 0
    bp0 = 0 if two_words else 4 - 2
    shift = pad - bp0
    bp, out = bp0, []
    a = b = off = 0
    for i in range(nsym):
        if i % group == 0:
            q = base + 32 * (bp >> 5) + lane
            w0, w1 = int(words[q]), int(words[q + 32])
            if two_words:
                a, b, off = _funnel(w0, w1, bp), w1 >> (bp & 31), 0
            else:
                a, b, off = _funnel(w0, w1, bp), _funnel(w1, int(words[q + 64]), bp), 0
        assert off < 32
        e = int(table[(_funnel(a, b, off) >> shift) & ((1 << index_bits) - 1)])
        assert e >> 28, "window without a code"
        out.append(e & 0xFFFF)
        off += e >> 28
        if i % group == group - 1 or i == nsym - 1:
            bp += off
    return out


@pytest.mark.parametrize("ty,n,k", [("Q6_K", 128, 1024), ("Q5_K", 64, 512), ("Q6_K", 64, 1536)])
def test_pair_layout_replayed_on_cpu(ty, n, k):
    """The pair layout of Q6_K / Q5_K: every chain decodes (on the CPU, with the kernel's bit arithmetic) to the value
    bytes of its row's code pairs, and the scales behind every unit are the oracle's sub-block scales."""
    helpers.build_library()
    import lazyweights_b200 as lw
    q, side, sym, w, rng = helpers.seeded_case(ty, n, k, seed=5 + n + k)
    _tail_block(ty, q, rng, slice(0, 64), slice(64, 192))         # long codes back to back in one unit
    q[32:40, :] = rng.integers(0, 64 if ty == "Q6_K" else 32, (8, k))   # rows of rare pairs: the longest codes
    lay = lw.bundle.host_pairs(q, ty, side)
    L = lay["index_bits"]                                         # rows of rare pairs: more than 2048 different pairs
    assert L == (12 if ty == "Q6_K" else 11)
    assert lay["split"] == 4 and lay["pad"] == (0 if L == 11 else 6) and lay["group"] == 3 and lay["max_len"] <= L
    bias = 32 if ty == "Q6_K" else 0
    KT = k // 512
    for t in range((n // 64) * KT):
        tr, tc = divmod(t, KT)
        for seg in range(4):
            for half in range(2):
                base = int(lay["group_base"][t * 8 + 2 * seg + half])
                for lane in range(0, 32, 3):
                    got = _replay_pair_chain(lay["words"], base, lane, lay["table"], lay["pad"], L, 64, 3)
                    row = tr * 64 + half * 32 + lane
                    c = q[row, tc * 512 + seg * 128: tc * 512 + (seg + 1) * 128].astype(np.int64) - bias
                    want = ((c[0::2] & 255) | ((c[1::2] & 255) << 8)).tolist()
                    assert got == want, (t, seg, half, lane)
    # scales: rows r of unit (t, seg) against the oracle's per-sub-block scales
    sc, mn = orc.sub_scales(ty, side.reshape(n * k // 256, -1))          # [blocks, sub-blocks]
    sc, mn = sc.reshape(n, -1), mn.reshape(n, -1)                         # [row, sub-block along the row]
    nsub = 8 if ty == "Q6_K" else 4
    sw = lay["unit_side_words"]
    for t in range((n // 64) * KT):
        tr, tc = divmod(t, KT)
        for seg in range(4):
            end = int(lay["group_base"][t * 8 + 2 * seg + 2])             # the scales are the unit's last words
            sd = lay["words"][end - sw:end]
            for r in (0, 17, 63):
                row = tr * 64 + r
                sub0 = (tc * 512 + seg * 128) // (16 if ty == "Q6_K" else 32)
                if ty == "Q6_K":
                    d = np.frombuffer(sd.tobytes(), np.float16)[256 + r].astype(np.float32)
                    ints = np.frombuffer(np.array([sd[r], sd[64 + r]], np.uint32).tobytes(), np.int8).astype(np.float32)
                    got = d * ints
                    assert np.array_equal(got, sc[row, sub0:sub0 + nsub]), (t, seg, r)
                else:
                    dd = np.frombuffer(np.array([sd[r]], np.uint32).tobytes(), np.float16).astype(np.float32)
                    s6 = np.frombuffer(np.array([sd[64 + r]], np.uint32).tobytes(), np.uint8).astype(np.float32)
                    m6 = np.frombuffer(np.array([sd[128 + r]], np.uint32).tobytes(), np.uint8).astype(np.float32)
                    assert np.array_equal(dd[0] * s6, sc[row, sub0:sub0 + nsub]), (t, seg, r)
                    assert np.array_equal(dd[1] * m6, mn[row, sub0:sub0 + nsub]), (t, seg, r)


def test_pair_code_width_follows_the_data():
    """Pairs of 6-bit codes get an 11-bit code when at most 2048 different pairs occur and the limit costs little
    (here: codes from a narrow spread), else a 12-bit one; the layout replays to the same codes."""
    helpers.build_library()
    import lazyweights_b200 as lw
    q, side, sym, w, rng = helpers.seeded_case("Q6_K", 64, 1024, seed=3)
    q = np.clip(np.rint(rng.normal(32.0, 1.5, q.shape)), 0, 63).astype(np.uint8)
    lay = lw.bundle.host_pairs(q, "Q6_K", side)
    assert lay["index_bits"] == 11 and lay["max_len"] <= 11 and lay["pad"] == 0
    for lane in (0, 9, 31):
        got = _replay_pair_chain(lay["words"], int(lay["group_base"][3]), lane, lay["table"], lay["pad"], 11, 64, 3)
        c = q[32 + lane, 128:256].astype(np.int64) - 32
        assert got == ((c[0::2] & 255) | ((c[1::2] & 255) << 8)).tolist()
