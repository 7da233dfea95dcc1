"""CPU oracle for the coded-weight hot path.  TEST INFRASTRUCTURE ONLY.

A NumPy restatement of the reference algorithms for: Huffman table construction, the huf8 / huf4p blob
(encode and decode), the split of llama.cpp K-quant blocks into codes and side bytes, the block
dequantisation arithmetic and the matrix-vector product.  Nothing in the shipped package imports this
file; only the tests, the smoke check and the CPU-baseline leg of the benchmark do, and only as the checker.

Parity pin: every function here is checked against vectors produced by the reference's own Python code
(``tests/golden/*.npz``, written by ``tests/golden/make_golden.py`` from the reference imported in place).

Reference locations restated here (paths inside the reference project):
  lazyweights/huffman.py:8-26        code_lengths            -> huffman_lengths
  lazyweights/lanecodecs.py:28-38    limited_lengths         -> limited_lengths
  lazyweights/lanecodecs.py:41-62    canonical_codes, bitrev -> canonical_codes, bit_reverse
  lazyweights/bundle.py:33-43        lane_order(_inv)        -> to_stream_order, from_stream_order
  lazyweights/bundle.py:46-54        build_lut               -> build_lut
  lazyweights/bundle.py:57-85        encode_huf8             -> encode_huf8
  lazyweights/bundle.py:88-106       decode_huf8             -> decode_huf8
  lazyweights/bundle.py:114-148      Writer, read_manifest   -> BundleWriter, read_manifest
  scripts/kq_code.py:37-81           split, join             -> split_blocks, join_blocks
  scripts/a2_kq_bundle.py:50-82      sub_sm, fq, dequant     -> sub_scales, grid_value, dequant
  scripts/a2_kq_bundle.py:108        pair symbols            -> pair_symbols, unpair_symbols
  hw/huff/huff_engine.h:39-77        build_canon, lookup<1>  -> comparator_tables, comparator_lookup
"""
import heapq
import os

import numpy as np

TILE_ROWS, TILE_SYMS, MAX_LEN, LANES = 64, 256, 11, 32
LUT_SIZE = 1 << MAX_LEN
BLOB_ALIGN = 256

KQ_TYPES = ("Q4_K", "Q5_K", "Q6_K", "IQ4_XS")
SIDE_BYTES = {"Q4_K": 16, "Q5_K": 16, "Q6_K": 18, "IQ4_XS": 8}
BLOCK_BYTES = {"Q4_K": 144, "Q5_K": 176, "Q6_K": 210, "IQ4_XS": 136}
SUB_WIDTH = {"Q4_K": 32, "Q5_K": 32, "Q6_K": 16, "IQ4_XS": 32}
PAIRED = {"Q4_K": True, "Q5_K": False, "Q6_K": False, "IQ4_XS": True}
IQ4_GRID = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)


# ----------------------------------------------------------------------------------------------- tables

def huffman_lengths(counts):
    """Plain Huffman depths; ties between equal counts resolve by creation order (leaves by symbol, then
    merged nodes in the order they were made), which is what fixes the lengths the reference gets."""
    counts = np.asarray(counts, np.int64)
    used = np.flatnonzero(counts)
    depth = np.zeros(counts.size, np.int64)
    if used.size == 0:
        return depth
    if used.size == 1:
        depth[used[0]] = 1
        return depth
    parent = {}
    heap = [(int(counts[s]), order, order) for order, s in enumerate(used)]
    heapq.heapify(heap)
    serial = used.size
    while len(heap) > 1:
        wa, _, na = heapq.heappop(heap)
        wb, _, nb = heapq.heappop(heap)
        parent[na] = serial
        parent[nb] = serial
        heapq.heappush(heap, (wa + wb, serial, serial))
        serial += 1
    for leaf, s in enumerate(used):
        d, node = 0, leaf
        while node in parent:
            node = parent[node]
            d += 1
        depth[s] = d
    return depth


def limited_lengths(counts, max_len=MAX_LEN):
    """Halve the counts (floor, never below one for a used symbol) until the Huffman tree is no deeper than
    max_len."""
    counts = np.asarray(counts, np.int64)
    shift = 0
    while True:
        scaled = np.where(counts > 0, np.maximum(counts >> shift, 1), 0)
        depth = huffman_lengths(scaled)
        if depth.max() <= max_len:
            return depth.astype(np.uint8)
        shift += 1


def canonical_codes(lengths):
    """MSB-first canonical code values: shorter codes first, symbol-ascending inside a length."""
    lengths = np.asarray(lengths, np.int64)
    codes = np.zeros(lengths.size, np.int64)
    nxt = 0
    for ln in range(1, int(lengths.max()) + 1):
        members = np.flatnonzero(lengths == ln)
        codes[members] = nxt + np.arange(members.size)
        nxt = (nxt + members.size) << 1
    return codes


def bit_reverse(values, nbits):
    values = np.asarray(values, np.int64)
    nbits = np.broadcast_to(np.asarray(nbits, np.int64), values.shape)
    out = np.zeros_like(values)
    for i in range(int(nbits.max()) if values.size else 0):
        bit = (values >> i) & 1
        out |= np.where(i < nbits, bit << np.maximum(nbits - 1 - i, 0), 0)
    return out


def build_lut(lengths):
    """uint16[2048]: entry = symbol | length << 8 for every 11-bit LSB-first window that starts with the
    symbol's (bit-reversed) code."""
    lengths = np.asarray(lengths, np.int64)
    codes = canonical_codes(lengths)
    lut = np.zeros(LUT_SIZE, np.uint16)
    for s in np.flatnonzero(lengths):
        ln = int(lengths[s])
        rev = int(bit_reverse(np.array([codes[s]]), ln)[0])
        lut[rev + (np.arange(1 << (MAX_LEN - ln)) << ln)] = s | (ln << 8)
    return lut


def lengths_from_lut(lut):
    """Per-symbol code lengths recovered from a blob's table (the blob stores nothing else)."""
    lut = np.asarray(lut, np.uint16)
    lengths = np.zeros(256, np.int64)
    ok = (lut >> 8) > 0
    lengths[(lut[ok] & 255).astype(np.int64)] = (lut[ok] >> 8).astype(np.int64)
    return lengths


def comparator_tables(lut):
    """limit / first / base / sorted of the canonical code, rebuilt from the table alone."""
    lengths = lengths_from_lut(lut)
    limit = np.zeros(MAX_LEN + 1, np.int64)
    first = np.zeros(MAX_LEN + 1, np.int64)
    base = np.zeros(MAX_LEN + 1, np.int64)
    order = []
    code = 0
    for ln in range(1, MAX_LEN + 1):
        members = np.flatnonzero(lengths == ln)
        first[ln], base[ln] = code, len(order)
        order.extend(int(s) for s in members)
        code += members.size
        limit[ln] = code << (MAX_LEN - ln)
        code <<= 1
    return limit, first, base, np.array(order + [0] * (256 - len(order)), np.uint8)


def comparator_lookup(tables, window):
    """(symbol, length) of an 11-bit LSB-first window using only compares against the limits."""
    limit, first, base, order = tables
    v = int(bit_reverse(np.array([window]), MAX_LEN)[0])
    ln = 1 + sum(1 for k in range(1, MAX_LEN) if v >= limit[k])
    return int(order[base[ln] + (v >> (MAX_LEN - ln)) - first[ln]]), ln


# ------------------------------------------------------------------------------------------- stream order

def to_stream_order(sym):
    """[N, Ks] -> flat (tile row, tile column, lane, half, column); lane l holds tile rows l and l + 32."""
    n, ks = sym.shape
    v = sym.reshape(n // TILE_ROWS, 2, LANES, ks // TILE_SYMS, TILE_SYMS)
    return np.ascontiguousarray(v.transpose(0, 3, 2, 1, 4)).reshape(-1)


def from_stream_order(flat, n, ks):
    v = np.asarray(flat).reshape(n // TILE_ROWS, ks // TILE_SYMS, LANES, 2, TILE_SYMS)
    return np.ascontiguousarray(v.transpose(0, 3, 2, 1, 4)).reshape(n, ks)


# ------------------------------------------------------------------------------------------------ blobs

def blob_layout(n, ks):
    tiles = (n // TILE_ROWS) * (ks // TILE_SYMS)
    return tiles, 2 * LUT_SIZE, 2 * LUT_SIZE + tiles * LANES * 4


def encode_huf8(sym):
    """uint8 [N, Ks] symbols -> (blob bytes, payload bits, histogram)."""
    sym = np.ascontiguousarray(sym, np.uint8)
    n, ks = sym.shape
    if n % TILE_ROWS or ks % TILE_SYMS:
        raise ValueError("shape must be a multiple of 64 x 256 symbols")
    hist = np.bincount(sym.reshape(-1), minlength=256)
    lengths = limited_lengths(hist).astype(np.int64)
    rcodes = bit_reverse(canonical_codes(lengths), np.maximum(lengths, 1))
    order = to_stream_order(sym)
    ln = lengths[order]
    end = np.cumsum(ln)
    pos = end - ln
    total = int(end[-1])
    if total >= 1 << 32:
        raise ValueError("payload does not fit 32-bit lane offsets")
    tiles = (n // TILE_ROWS) * (ks // TILE_SYMS)
    starts = pos[::2 * TILE_SYMS].astype(np.uint32).reshape(tiles, LANES)
    nwords = (total + 31) // 32 + 2
    words = np.zeros(nwords + 2, np.uint32)
    val = rcodes[order].astype(np.uint64)
    sh = (pos & 31).astype(np.uint64)
    spread = val << sh                                        # at most 42 bits
    np.bitwise_or.at(words, pos >> 5, (spread & np.uint64(0xFFFFFFFF)).astype(np.uint32))
    np.bitwise_or.at(words, (pos >> 5) + 1, (spread >> np.uint64(32)).astype(np.uint32))
    blob = build_lut(lengths).tobytes() + starts.tobytes() + words[:nwords].tobytes()
    return blob, total, hist


def encode_huf8_native(sym):
    """encode_huf8 with the bit packing done by the C restatement (oracle/lw_oracle_c.c: orc_pack); the tables are the
    ones above.  Byte-identical to encode_huf8, many times faster on benchmark-size matrices."""
    import ctypes as C
    from oracle import build_oracle
    L = build_oracle.lib()
    sym = np.ascontiguousarray(sym, np.uint8)
    n, ks = sym.shape
    if n % TILE_ROWS or ks % TILE_SYMS:
        raise ValueError("shape must be a multiple of 64 x 256 symbols")
    hist = np.bincount(sym.reshape(-1), minlength=256)
    lengths = limited_lengths(hist).astype(np.int64)
    rcodes = np.ascontiguousarray(bit_reverse(canonical_codes(lengths), np.maximum(lengths, 1)), np.uint32)
    total = int((hist * lengths).sum())
    if total >= 1 << 32:
        raise ValueError("payload does not fit 32-bit lane offsets")
    tiles = (n // TILE_ROWS) * (ks // TILE_SYMS)
    starts = np.zeros(tiles * LANES, np.uint32)
    words = np.zeros((total + 31) // 32 + 2, np.uint32)
    len8 = np.ascontiguousarray(lengths, np.uint8)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    got = L.orc_pack(p(sym), n, ks, p(len8), p(rcodes), p(starts), p(words))
    assert got == total
    return build_lut(lengths).tobytes() + starts.tobytes() + words.tobytes(), total, hist


def decode_huf8(blob, n, ks):
    """blob -> uint8 [N, Ks] symbols.  All lanes advance in lock step, one symbol per pass."""
    tiles, off_starts, off_words = blob_layout(n, ks)
    raw = np.frombuffer(blob, np.uint8)
    lut = raw[:off_starts].view(np.uint16)
    bp = raw[off_starts:off_words].view(np.uint32).astype(np.int64)
    words = raw[off_words:off_words + (len(blob) - off_words) // 4 * 4].view(np.uint32).astype(np.uint64)
    words = np.concatenate([words, np.zeros(2, np.uint64)])
    out = np.empty((tiles * LANES, 2 * TILE_SYMS), np.uint8)
    mask = np.uint64(LUT_SIZE - 1)
    for i in range(2 * TILE_SYMS):
        w = bp >> 5
        window = ((words[w] | (words[w + 1] << np.uint64(32))) >> (bp & 31).astype(np.uint64)) & mask
        entry = lut[window.astype(np.int64)]
        out[:, i] = entry & 255
        bp = bp + (entry >> 8)
    return from_stream_order(out.reshape(-1), n, ks)


def pair_symbols(q):
    """4-bit codes [N, K] -> 8-bit symbols [N, K/2]; the even column is the low nibble."""
    q = np.asarray(q, np.uint8)
    return np.ascontiguousarray(q[:, 0::2] | (q[:, 1::2] << 4))


def unpair_symbols(sym):
    sym = np.asarray(sym, np.uint8)
    q = np.empty((sym.shape[0], sym.shape[1] * 2), np.uint8)
    q[:, 0::2] = sym & 15
    q[:, 1::2] = sym >> 4
    return q


def symbols_of(ty, q):
    return pair_symbols(q) if PAIRED[ty] else np.ascontiguousarray(q, np.uint8)


def codes_of(ty, sym):
    return unpair_symbols(sym) if PAIRED[ty] else np.asarray(sym, np.uint8)


# ------------------------------------------------------------------------------------- K-quant blocks

def split_blocks(ty, blocks):
    """GGUF block bytes [nblk, B] -> (codes [nblk, 256] in weight order, side bytes [nblk, S])."""
    b = np.asarray(blocks, np.uint8)
    nb = b.shape[0]
    nib = np.array([0, 4], np.uint8)
    if ty == "Q4_K":
        side, qs = b[:, :16], b[:, 16:144]
        q = (qs.reshape(nb, 4, 1, 32) >> nib.reshape(1, 1, 2, 1)) & 15          # 64-wide groups: low, high
        return q.reshape(nb, 256), side
    if ty == "Q5_K":
        side, qh, qs = b[:, :16], b[:, 16:48], b[:, 48:176]
        lo = ((qs.reshape(nb, 4, 1, 32) >> nib.reshape(1, 1, 2, 1)) & 15).reshape(nb, 8, 32)
        hi = (qh.reshape(nb, 1, 32) >> np.arange(8, dtype=np.uint8).reshape(1, 8, 1)) & 1
        return (lo | (hi << 4)).reshape(nb, 256), side
    if ty == "Q6_K":
        ql, qh, side = b[:, :128], b[:, 128:192], b[:, 192:210]
        lo = ((ql.reshape(nb, 2, 1, 64) >> nib.reshape(1, 1, 2, 1)) & 15).reshape(nb, 2, 4, 32)
        hi = (qh.reshape(nb, 2, 1, 32) >> np.array([0, 2, 4, 6], np.uint8).reshape(1, 1, 4, 1)) & 3
        return (lo | (hi << 4)).reshape(nb, 256), side
    if ty == "IQ4_XS":
        side, qs = b[:, :8], b[:, 8:136]
        q = (qs.reshape(nb, 8, 1, 16) >> nib.reshape(1, 1, 2, 1)) & 15          # 32-wide groups
        return q.reshape(nb, 256), side
    raise ValueError(ty)


def join_blocks(ty, q, side):
    """Inverse of split_blocks."""
    q = np.asarray(q, np.uint8)
    side = np.asarray(side, np.uint8)
    nb = q.shape[0]
    if ty in ("Q4_K", "IQ4_XS"):
        g = q.reshape(nb, 4, 2, 32) if ty == "Q4_K" else q.reshape(nb, 8, 2, 16)
        return np.concatenate([side, (g[:, :, 0] | (g[:, :, 1] << 4)).reshape(nb, 128)], axis=1)
    if ty == "Q5_K":
        g = q.reshape(nb, 8, 32)
        qh = np.zeros((nb, 32), np.uint8)
        for j in range(8):
            qh |= (g[:, j] >> 4) << j
        lo = (g & 15).reshape(nb, 4, 2, 32)
        return np.concatenate([side, qh, (lo[:, :, 0] | (lo[:, :, 1] << 4)).reshape(nb, 128)], axis=1)
    if ty == "Q6_K":
        g = q.reshape(nb, 2, 4, 32)
        lo = (g & 15).reshape(nb, 2, 2, 64)
        ql = (lo[:, :, 0] | (lo[:, :, 1] << 4)).reshape(nb, 128)
        qh = np.zeros((nb, 2, 32), np.uint8)
        for j in range(4):
            qh |= (g[:, :, j] >> 4) << (2 * j)
        return np.concatenate([ql, qh.reshape(nb, 64), side], axis=1)
    raise ValueError(ty)


def _half_at(side, off):
    return np.ascontiguousarray(side[:, off:off + 2]).view(np.float16).astype(np.float32)[:, 0]


def sub_scales(ty, side):
    """side bytes [nblk, S] -> (scale, offset) float32 [nblk, sub-blocks]: weight = scale * f(q) - offset."""
    side = np.asarray(side, np.uint8)
    if ty in ("Q4_K", "Q5_K"):
        d, dmin = _half_at(side, 0), _half_at(side, 2)
        p = side[:, 4:16].astype(np.int32)
        sc = np.empty((side.shape[0], 8), np.int32)
        mn = np.empty((side.shape[0], 8), np.int32)
        for j in range(8):
            if j < 4:
                sc[:, j] = p[:, j] & 63
                mn[:, j] = p[:, j + 4] & 63
            else:
                sc[:, j] = (p[:, j + 4] & 15) | ((p[:, j - 4] >> 6) << 4)
                mn[:, j] = (p[:, j + 4] >> 4) | ((p[:, j] >> 6) << 4)
        return d[:, None] * sc.astype(np.float32), dmin[:, None] * mn.astype(np.float32)
    if ty == "Q6_K":
        s = _half_at(side, 16)[:, None] * side[:, :16].view(np.int8).astype(np.float32)
        return s, np.zeros_like(s)
    if ty == "IQ4_XS":
        hi = np.ascontiguousarray(side[:, 2:4]).view(np.uint16).astype(np.int32)     # [nblk, 1]
        lo = side[:, 4:8].astype(np.int32)
        ls = np.empty((side.shape[0], 8), np.int32)
        for j in range(8):
            ls[:, j] = ((lo[:, j // 2] >> (4 * (j & 1))) & 15) | (((hi[:, 0] >> (2 * j)) & 3) << 4)
        s = _half_at(side, 0)[:, None] * (ls - 32).astype(np.float32)
        return s, np.zeros_like(s)
    raise ValueError(ty)


def grid_value(ty, q):
    q = np.asarray(q)
    if ty == "IQ4_XS":
        return IQ4_GRID[q]
    return q.astype(np.float32) - np.float32(32 if ty == "Q6_K" else 0)


def dequant(ty, q, side):
    """float32 [N, K]: scale * f(q) - offset, the product and the difference each rounded to float32."""
    n, k = q.shape
    s, o = sub_scales(ty, np.asarray(side, np.uint8).reshape(n * k // 256, -1))
    f = grid_value(ty, q).reshape(n * k // 256, s.shape[1], -1)
    return (s[:, :, None] * f - o[:, :, None]).astype(np.float32).reshape(n, k)


def dequant_f16(ty, q, side):
    return dequant(ty, q, side).astype(np.float16)


def gemv_f64(w, x):
    """y[m, N] = x[m, K] . w[N, K]^T accumulated in float64 (the tolerance reference)."""
    x = np.atleast_2d(np.asarray(x, np.float64))
    return x @ np.asarray(w, np.float64).T


# ---------------------------------------------------------------------------------------------- bundles

class BundleWriter:
    """manifest.txt + weights.bin; every blob starts on a 256-byte boundary."""

    def __init__(self, path):
        os.makedirs(path, exist_ok=True)
        self.path = path
        self._bin = open(os.path.join(path, "weights.bin"), "wb")
        self._lines = []
        self._off = 0

    def cfg(self, key, value):
        self._lines.append("cfg %s %s" % (key, value))

    def add(self, name, enc, n, k, blob, scale=1.0, zp=0):
        pad = -self._off % BLOB_ALIGN
        self._bin.write(bytes(pad))
        self._off += pad
        self._bin.write(blob)
        self._lines.append("t %s %s %d %d %.9g %d %d %d" % (name, enc, n, k, scale, zp, self._off, len(blob)))
        self._off += len(blob)

    def add_matrix(self, name, ty, q, side):
        """codes [N, K] + side bytes -> the coded matrix and its `.kqs` side tensor, as the builder names them."""
        n, k = q.shape
        blob, _, _ = encode_huf8(symbols_of(ty, q))
        self.add(name, "huf4p" if PAIRED[ty] else "huf8", n, k, blob)
        side = np.ascontiguousarray(side, np.uint8).reshape(n, -1)
        self.add(name + ".kqs", "kq_" + ty, n, side.shape[1], side.tobytes())

    def close(self):
        self._bin.close()
        with open(os.path.join(self.path, "manifest.txt"), "w") as f:
            f.write("\n".join(self._lines) + "\n")


def read_manifest(path):
    cfg, tensors = {}, []
    with open(os.path.join(path, "manifest.txt")) as f:
        for line in f:
            p = line.split()
            if not p:
                continue
            if p[0] == "cfg":
                cfg[p[1]] = p[2]
            elif p[0] == "t":
                tensors.append(dict(name=p[1], enc=p[2], N=int(p[3]), K=int(p[4]), scale=float(p[5]),
                                    zp=int(p[6]), offset=int(p[7]), nbytes=int(p[8])))
    return cfg, tensors


# ------------------------------------------------------------------------------- synthetic test inputs

def synth_codes(ty, n, k, rng):
    """Codes with the value distributions the benchmark configurations name."""
    if ty == "Q4_K":
        q = np.clip(np.rint(rng.laplace(8.0, 1.5, (n, k))), 0, 15)
    elif ty == "IQ4_XS":
        q = np.clip(np.rint(rng.laplace(7.5, 1.5, (n, k))), 0, 15)
    elif ty == "Q5_K":
        q = np.clip(np.rint(rng.normal(16.0, 2.5, (n, k))), 0, 31)
    elif ty == "Q6_K":
        q = np.clip(np.rint(rng.normal(32.0, 5.0, (n, k))), 0, 63)
    else:
        raise ValueError(ty)
    return q.astype(np.uint8)


def synth_side(ty, n, k, rng):
    """Side bytes [N, K/256 * S]: fp16 d (and dmin) ~ U(1e-3, 1e-2), every other byte uniform."""
    nb = n * k // 256
    side = rng.integers(0, 256, (nb, SIDE_BYTES[ty]), dtype=np.uint8)
    d = rng.uniform(1e-3, 1e-2, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    if ty in ("Q4_K", "Q5_K"):
        side[:, 0:2] = d
        side[:, 2:4] = rng.uniform(1e-3, 1e-2, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    elif ty == "Q6_K":
        side[:, 0:16] = rng.integers(-64, 64, (nb, 16)).astype(np.int8).view(np.uint8)
        side[:, 16:18] = d
    else:
        side[:, 0:2] = d
    return side.reshape(n, -1)
