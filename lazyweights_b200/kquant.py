"""llama.cpp block formats on the host: GGUF block bytes <-> (codes, side bytes), and the kernels' dequantisation
arithmetic in NumPy.

Mirrors the reference's scripts/kq_code.py (`split` :37, `join` :63) and scripts/a2_kq_bundle.py (`sub_sm` :50, `fq` :71,
`dequant` :76) with the same argument meaning; block types are named by string ("Q4_K", "Q5_K", "Q6_K", "IQ4_XS") or by
gguf-py's GGMLQuantizationType.  split / join run in the library's C++ host code (lw_split_blocks / lw_join_blocks);
`dequant` is the float32 arithmetic the CUDA kernels perform (scale * f(code) - offset, product and difference rounded
separately), used by the bundle builder to check every matrix against gguf-py before it is coded.
"""
import ctypes as C

import numpy as np

from . import _native as nat

BLOCK_BYTES = {"Q4_K": 144, "Q5_K": 176, "Q6_K": 210, "IQ4_XS": 136}
SIDE_BYTES = {"Q4_K": 16, "Q5_K": 16, "Q6_K": 18, "IQ4_XS": 8}
CODE_BITS = {"Q4_K": 4, "Q5_K": 5, "Q6_K": 6, "IQ4_XS": 4}
PAIRED = ("Q4_K", "IQ4_XS")                      # two 4-bit codes per coded symbol
IQ4_GRID = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)


def type_name(ty):
    """'Q4_K' for 'Q4_K' or for gguf.GGMLQuantizationType.Q4_K."""
    name = ty if isinstance(ty, str) else ty.name
    if name not in BLOCK_BYTES:
        raise ValueError("unsupported block type %s" % name)
    return name


def split(ty, blocks):
    """Blocks [n, block bytes] -> (codes [n, 256] uint8 in weight order, side bytes [n, s], code bits)."""
    ty = type_name(ty)
    b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, BLOCK_BYTES[ty])
    n = b.shape[0]
    q = np.empty((n, 256), np.uint8)
    side = np.empty((n, SIDE_BYTES[ty]), np.uint8)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    nat.check(nat.lib().lw_split_blocks(nat.FMT[ty], p(b), n, p(q), p(side)))
    return q, side, CODE_BITS[ty]


def join(ty, q, side):
    """Inverse of split: codes [n, 256] + side bytes [n, s] -> blocks [n, block bytes]."""
    ty = type_name(ty)
    q = np.ascontiguousarray(q, np.uint8).reshape(-1, 256)
    n = q.shape[0]
    side = np.ascontiguousarray(side, np.uint8).reshape(n, SIDE_BYTES[ty])
    out = np.empty((n, BLOCK_BYTES[ty]), np.uint8)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    nat.check(nat.lib().lw_join_blocks(nat.FMT[ty], p(q), p(side), n, p(out)))
    return out


def _f16(side, off):
    return np.ascontiguousarray(side[:, off:off + 2]).view(np.float16).astype(np.float32)[:, 0]


def sub_sm(ty, side):
    """Side bytes [n, s] of n super-blocks -> (scale, offset) [n, sub-blocks] float32, as the kernels form them:
    Q4_K / Q5_K  d * sc, dmin * m (eight 32-weight sub-blocks, 6-bit sc / m);  Q6_K  d * int8 scale (sixteen 16-weight
    sub-blocks);  IQ4_XS  d * (ls - 32) (eight 32-weight sub-blocks)."""
    ty = type_name(ty)
    side = np.asarray(side, np.uint8)
    if ty in ("Q4_K", "Q5_K"):
        d, dmin = _f16(side, 0), _f16(side, 2)
        b = side[:, 4:16].astype(np.int32)
        sc = np.empty((side.shape[0], 8), np.int32)
        mn = np.empty_like(sc)
        for j in range(8):
            if j < 4:
                sc[:, j], mn[:, j] = b[:, j] & 63, b[:, j + 4] & 63
            else:
                sc[:, j] = (b[:, j + 4] & 15) | ((b[:, j - 4] >> 6) << 4)
                mn[:, j] = (b[:, j + 4] >> 4) | ((b[:, j] >> 6) << 4)
        return d[:, None] * sc.astype(np.float32), dmin[:, None] * mn.astype(np.float32)
    if ty == "Q6_K":
        s = _f16(side, 16)[:, None] * np.ascontiguousarray(side[:, :16]).view(np.int8).astype(np.float32)
        return s, np.zeros_like(s)
    hi = np.ascontiguousarray(side[:, 2:4]).view(np.uint16).astype(np.int32)          # IQ4_XS
    lo = side[:, 4:8].astype(np.int32)
    ls = np.empty((side.shape[0], 8), np.int32)
    for j in range(8):
        ls[:, j] = ((lo[:, j // 2] >> (4 * (j % 2))) & 15) | (((hi[:, 0] >> (2 * j)) & 3) << 4)
    s = _f16(side, 0)[:, None] * (ls - 32).astype(np.float32)
    return s, np.zeros_like(s)


def fq(ty, q):
    """Grid value of a code: Q4_K / Q5_K the code, Q6_K code - 32, IQ4_XS the non-linear grid."""
    ty = type_name(ty)
    q = np.asarray(q)
    return IQ4_GRID[q] if ty == "IQ4_XS" else q.astype(np.float32) - np.float32(32 if ty == "Q6_K" else 0)


def dequant(ty, q, side):
    """Kernel arithmetic in float32: w = s * f(q) - o per sub-block.  q [N, K] codes, side [N, K / 256 * s]."""
    ty = type_name(ty)
    n, k = q.shape
    s, o = sub_sm(ty, np.asarray(side, np.uint8).reshape(n * k // 256, -1))
    f = fq(ty, q).reshape(n * k // 256, s.shape[1], -1)
    return (s[:, :, None] * f - o[:, :, None]).reshape(n, k)
