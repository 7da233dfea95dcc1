"""Host-side mirror of the reference's bundle module (lazyweights/bundle.py) on top of liblwb200.

Same names and argument meaning as the reference: `encode_huf8(q) -> (blob, bits, hist)` (bundle.py:57),
`decode_huf8(blob, N, K) -> uint8 [N, K]` (bundle.py:88), `Writer` (bundle.py:114), `read_manifest`
(bundle.py:139).  The encoder runs in the library's C++ host code; `decode_huf8` decodes ON THE GPU (it raises
without a CUDA device: there is no CPU decode path behind it).  `cpu_decode_huf8` is the explicit host decoder,
the counterpart of the reference's threaded cpu_decode (kernels/llmrt.cu:2513).
"""
import ctypes as C
import os

import numpy as np

from . import _native as nat

TN, TK, LMAX, LANES = 64, 256, 11, 32
ALIGN = 256
ROPE_ROWS = 4096


def _u8(a):
    a = np.ascontiguousarray(a, np.uint8)
    return a, a.ctypes.data_as(C.c_void_p)


def encode_huf8(q):
    """uint8 [N, K] symbols -> (blob bytes, payload bits, histogram[256])."""
    q, qp = _u8(q)
    if q.ndim != 2:
        raise ValueError("encode_huf8 wants a 2-D uint8 array")
    n, k = q.shape
    assert n % TN == 0 and k % TK == 0, (n, k)
    L = nat.lib()
    bits = C.c_longlong(0)
    size = nat.check(L.lw_encode_huf8(qp, n, k, None, 0, C.byref(bits)))
    out = np.empty(size, np.uint8)
    nat.check(L.lw_encode_huf8(qp, n, k, out.ctypes.data_as(C.c_void_p), size, C.byref(bits)))
    return out.tobytes(), int(bits.value), np.bincount(q.reshape(-1), minlength=256)


def validate_huf8(blob, N, K):
    """Raises LwError unless the blob is well formed (canonical table, lanes contiguous, payload length)."""
    b, bp = _u8(np.frombuffer(blob, np.uint8))
    nat.check(nat.lib().lw_validate_blob(bp, b.size, N, K))


def cpu_decode_huf8(blob, N, K, threads=0):
    b, bp = _u8(np.frombuffer(blob, np.uint8))
    out = np.empty((N, K), np.uint8)
    nat.check(nat.lib().lw_cpu_decode(bp, b.size, N, K, threads or (os.cpu_count() or 1),
                                      out.ctypes.data_as(C.c_void_p)))
    return out


def host_layout(blob, N, Ks, fmt="none", side=None):
    """The device layout of one blob, built on the host (no GPU): dict with split, pad, group, index_bits,
    unit_side_words, max_unit_words, max_len and the arrays group_base (uint32), words (uint32), unit_class (uint8), lut
    (uint16[2048]: the decode table of the code the layout holds - the blob's own unless the loader re-coded it)."""
    b, bp = _u8(np.frombuffer(blob, np.uint8))
    s = np.ascontiguousarray(side, np.uint8).reshape(-1) if side is not None else np.zeros(0, np.uint8)
    sp = s.ctypes.data_as(C.c_void_p) if s.size else None
    info = (C.c_int * 8)()
    n = nat.lib().lw_host_layout(bp, b.size, N, Ks, nat.FMT[fmt], sp, s.size, info, None, 0, None, 0, None, 0)
    if n < 0:
        nat.check(int(n))
    gb, words, uc = np.zeros(info[4], np.uint32), np.zeros(n, np.uint32), np.zeros(info[5], np.uint8)
    n = nat.lib().lw_host_layout(bp, b.size, N, Ks, nat.FMT[fmt], sp, s.size, info, gb.ctypes.data_as(C.c_void_p),
                                 gb.size, words.ctypes.data_as(C.c_void_p), words.size,
                                 uc.ctypes.data_as(C.c_void_p), uc.size)
    if n < 0:
        nat.check(int(n))
    lut = np.zeros(2048, np.uint16)
    max_len = nat.lib().lw_host_layout_table(bp, b.size, N, Ks, nat.FMT[fmt], sp, s.size, lut.ctypes.data_as(C.c_void_p))
    if max_len < 0:
        nat.check(int(max_len))
    return dict(split=info[0], pad=info[1], group=info[2], index_bits=info[3], unit_side_words=info[6],
                max_unit_words=info[7], group_base=gb, words=words, unit_class=uc, lut=lut, max_len=int(max_len))


def host_pairs(codes, fmt, side):
    """The pair layout of Q6_K / Q5_K codes [N, K] (one per weight), built on the host (no GPU): dict with split, pad,
    group, index_bits, max_len, unit_side_words, max_unit_words and the arrays table, group_base, words (uint32)."""
    q = np.ascontiguousarray(codes, np.uint8)
    s = np.ascontiguousarray(side, np.uint8).reshape(-1)
    info = (C.c_int * 8)()
    args = (q.ctypes.data_as(C.c_void_p), q.shape[0], q.shape[1], nat.FMT[fmt], s.ctypes.data_as(C.c_void_p), s.size, info)
    n = nat.lib().lw_host_pairs(*args, None, 0, None, 0, None, 0)
    if n < 0:
        nat.check(int(n))
    tab, gb, words = np.zeros(1 << info[3], np.uint32), np.zeros(info[4], np.uint32), np.zeros(n, np.uint32)
    n = nat.lib().lw_host_pairs(*args, tab.ctypes.data_as(C.c_void_p), tab.size, gb.ctypes.data_as(C.c_void_p), gb.size,
                                words.ctypes.data_as(C.c_void_p), words.size)
    if n < 0:
        nat.check(int(n))
    return dict(split=info[0], pad=info[1], group=info[2], index_bits=info[3], max_len=info[5], unit_side_words=info[6],
                max_unit_words=info[7], table=tab, group_base=gb, words=words)


def decode_huf8(blob, N, K):
    """blob -> uint8 [N, K] symbols, decoded by the CUDA kernel."""
    from .runtime import CodedMatrix
    with CodedMatrix(blob, N, K) as m:
        return m.decode_symbols()


class Writer:
    """manifest.txt + weights.bin, every blob on a 256-byte boundary (reference: bundle.py:114-136)."""

    def __init__(self, path):
        os.makedirs(path, exist_ok=True)
        self.path = path
        self.f = open(os.path.join(path, "weights.bin"), "wb")
        self.lines = []
        self.off = 0

    def cfg(self, k, v):
        self.lines.append("cfg %s %s" % (k, v))

    def add(self, name, enc, N, K, scale, zp, blob):
        pad = (-self.off) % ALIGN
        if pad:
            self.f.write(bytes(pad))
            self.off += pad
        self.f.write(blob)
        self.lines.append("t %s %s %d %d %.9g %d %d %d" % (name, enc, N, K, scale, zp, self.off, len(blob)))
        self.off += len(blob)

    def add_kquant(self, name, ty, q, side):
        """Codes [N, K] of block format `ty` and their side bytes -> coded matrix + `<name>.kqs`, named and
        encoded as the reference's bundle builder does (scripts/a2_kq_bundle.py:104-114, :213-218)."""
        q = np.ascontiguousarray(q, np.uint8)
        n, k = q.shape
        paired = ty in ("Q4_K", "IQ4_XS")
        sym = np.ascontiguousarray(q[:, 0::2] | (q[:, 1::2] << 4)) if paired else q
        blob, nbits, _ = encode_huf8(sym)
        self.add(name, "huf4p" if paired else "huf8", n, k, 1.0, 0, blob)
        side = np.ascontiguousarray(side, np.uint8).reshape(n, -1)
        self.add(name + ".kqs", "kq_" + ty, n, side.shape[1], 1.0, 0, side.tobytes())
        return len(blob), side.size, nbits

    def close(self):
        self.f.close()
        with open(os.path.join(self.path, "manifest.txt"), "w") as f:
            f.write("\n".join(self.lines) + "\n")


def read_manifest(path):
    cfg, ts = {}, []
    with open(os.path.join(path, "manifest.txt")) as f:
        for line in f:
            p = line.split()
            if p and p[0] == "cfg":
                cfg[p[1]] = p[2]
            elif p and p[0] == "t":
                ts.append(dict(name=p[1], enc=p[2], N=int(p[3]), K=int(p[4]), scale=float(p[5]), zp=int(p[6]),
                               offset=int(p[7]), nbytes=int(p[8])))
    return cfg, ts
