"""GGUF -> runtime bundle: the bundle builder for real llama.cpp files.

    python -m lazyweights_b200.gguf_bundle model.gguf out_dir [--no-check]

Does what the reference's builder does (scripts/a2_kq_bundle.py:117-218) for a GGUF whose matrices are Q4_K, Q5_K, Q6_K
or IQ4_XS blocks, but takes the model shape from the GGUF's own metadata instead of a Hugging Face config directory:
  * every matrix: blocks -> codes + side bytes (kquant.split), llama-architecture q / k rows back from GGUF order to the
    rotate-half order (:147-149, the inverse of llama.cpp's conversion permute), q / k / v of one block type fused into
    `l<i>.qkv` (:159-160) else `l<i>.q / .k / .v`, phi3's fused `ffn_up` = [gate; up] split (:166-169), `lm_head` from
    `output.weight` or the tied embedding (:171);
  * codes coded with one 11-bit-limited Huffman table per matrix (pairs of 4-bit codes as one symbol for Q4_K / IQ4_XS),
    side bytes kept verbatim as `<name>.kqs` (enc `kq_<TYPE>`);
  * embedding as raw8 codes with float32 `embed.rs` / `embed.rsub` per sub-block (:85-101; Q8_0, Q6_K, IQ4_XS exact,
    Q4_K / Q5_K with rsub = dmin m / (d sc)); float32 norms; rotary cos / sin tables of 4096 rows computed in float64
    (:183-185); cfg keys as the runtime reads them (:190-192).
Unless --no-check, every matrix is checked before it is written: the kernels' dequantisation of (codes, side bytes)
must equal gguf-py's `dequantize` bit for bit, and the coded blob must decode (host decoder) to the symbols (:107, :113).
"""
import argparse
import os
import sys

import numpy as np

from . import kquant
from .bundle import ROPE_ROWS, Writer, cpu_decode_huf8, encode_huf8

PERMUTED_ARCHS = ("llama", "mistral")            # conversion permutes q / k rows for these architectures


def permute_rows(w, n_head):
    """HF q / k rows -> GGUF rows, as llama.cpp's conversion does (reference: scripts/kq_quant.py:232-234)."""
    return w.reshape(n_head, 2, w.shape[0] // n_head // 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)


def unpermute_index(n_rows, n_head):
    """Row order that undoes permute_rows: rows_hf = rows_gguf[unpermute_index]."""
    return np.argsort(permute_rows(np.arange(n_rows), n_head))


def embedding_raw8(ty_name, blocks, vocab, dim):
    """Embedding blocks -> raw8 codes [V, D] and float32 rs / rsub [V, D / sub-block]: w = (code - rsub) * rs."""
    if ty_name == "Q8_0":
        b = np.ascontiguousarray(blocks, np.uint8).reshape(-1, 34)
        d = np.ascontiguousarray(b[:, :2]).view(np.float16).astype(np.float32).reshape(vocab, -1)
        codes = (np.ascontiguousarray(b[:, 2:]).view(np.int8).astype(np.int16) + 128).astype(np.uint8)
        return codes.reshape(vocab, dim), d, np.full_like(d, 128)
    q, side, _ = kquant.split(ty_name, blocks)
    s, o = kquant.sub_sm(ty_name, side)
    if ty_name == "IQ4_XS":
        codes = (kquant.IQ4_GRID[q] + 128).astype(np.uint8)
        return codes.reshape(vocab, dim), s.reshape(vocab, -1), np.full((vocab, s.size // vocab), 128, np.float32)
    if ty_name == "Q6_K":
        return q.reshape(vocab, dim), s.reshape(vocab, -1), np.full((vocab, s.size // vocab), 32, np.float32)
    ok = s != 0
    if not np.all(ok | (o == 0)):
        raise ValueError("embedding has a sub-block with scale 0 and a non-zero minimum")
    z = np.where(ok, o / np.where(ok, s, 1), 0)
    return q.reshape(vocab, dim), s.reshape(vocab, -1), z.astype(np.float32).reshape(vocab, -1)


class _Gguf:
    """The parts of a GGUF file the builder needs."""

    def __init__(self, path):
        import gguf
        self.gguf = gguf
        self.reader = gguf.GGUFReader(path)
        self.tensors = {t.name: t for t in self.reader.tensors}
        self.arch = self.field("general.architecture")

    def field(self, key, default=None):
        f = self.reader.fields.get(key)
        return default if f is None else f.contents()

    def hp(self, key, default=None):
        return self.field("%s.%s" % (self.arch, key), default)

    def blocks(self, name):
        t = self.tensors[name]
        ty = t.tensor_type.name
        k, n = (int(x) for x in t.shape[:2])                         # GGUF shapes list the row length first
        return ty, n, k, np.asarray(t.data).reshape(-1)

    def f32(self, name):
        return np.asarray(self.tensors[name].data, np.float32).reshape(-1)


def build_bundle(gguf_path, out_dir, check=True, log=None):
    """Writes the bundle directory; returns a summary dict (cfg, bits per weight, embedding error)."""
    g = _Gguf(gguf_path)
    say = log or (lambda *a: None)
    L = int(g.hp("block_count"))
    D = int(g.hp("embedding_length"))
    H = int(g.hp("attention.head_count"))
    Hk = int(g.hp("attention.head_count_kv", H))
    Dh = int(g.hp("attention.key_length", D // H))
    inter = int(g.hp("feed_forward_length"))
    eps = float(g.hp("attention.layer_norm_rms_epsilon", 1e-5))
    theta = float(g.hp("rope.freq_base", 10000.0))
    tied = "output.weight" not in g.tensors
    permuted = g.arch in PERMUTED_ARCHS

    def matrix(name, heads=None):
        ty, n, k, raw = g.blocks(name)
        if ty not in kquant.BLOCK_BYTES:
            raise ValueError("%s is %s: only Q4_K, Q5_K, Q6_K and IQ4_XS matrices can be coded" % (name, ty))
        q, side, _ = kquant.split(ty, raw.reshape(-1, kquant.BLOCK_BYTES[ty]))
        q, side = q.reshape(n, k), side.reshape(n, -1)
        ref = None
        if check:
            ref = g.gguf.quants.dequantize(raw.reshape(n, -1), g.tensors[name].tensor_type).reshape(n, k)
        if heads is not None and permuted:
            inv = unpermute_index(n, heads)
            q, side = q[inv], side[inv]
            ref = ref[inv] if ref is not None else None
        return ty, q, side, ref

    order = []
    for i in range(L):
        p = "blk.%d." % i
        if p + "attn_qkv.weight" in g.tensors:
            order.append(("l%d.qkv" % i, matrix(p + "attn_qkv.weight")))
        else:
            qkv = [matrix(p + "attn_q.weight", H), matrix(p + "attn_k.weight", Hk), matrix(p + "attn_v.weight")]
            if len({m[0] for m in qkv}) == 1:
                fused = tuple(None if qkv[0][j] is None else np.concatenate([m[j] for m in qkv]) for j in (1, 2, 3))
                order.append(("l%d.qkv" % i, (qkv[0][0],) + fused))
            else:
                order += [("l%d.%s" % (i, nm), m) for nm, m in zip("qkv", qkv)]
        order.append(("l%d.o" % i, matrix(p + "attn_output.weight")))
        if p + "ffn_gate.weight" in g.tensors:
            order += [("l%d.gate" % i, matrix(p + "ffn_gate.weight")), ("l%d.up" % i, matrix(p + "ffn_up.weight"))]
        else:                                                        # phi3: ffn_up holds the gate rows, then the up rows
            ty, q, side, ref = matrix(p + "ffn_up.weight")
            half = q.shape[0] // 2
            cut = lambda a, lo, hi: None if a is None else a[lo:hi]
            order += [("l%d.gate" % i, (ty, q[:half], side[:half], cut(ref, 0, half))),
                      ("l%d.up" % i, (ty, q[half:], side[half:], cut(ref, half, None)))]
        order.append(("l%d.down" % i, matrix(p + "ffn_down.weight")))
    order.append(("lm_head", matrix("token_embd.weight" if tied else "output.weight")))

    ety, V, _, eraw = g.blocks("token_embd.weight")
    eblock = 34 if ety == "Q8_0" else kquant.BLOCK_BYTES.get(ety)
    if eblock is None:
        raise ValueError("embedding type %s is not supported (Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS)" % ety)
    eq, es, ez = embedding_raw8(ety, eraw.reshape(-1, eblock), V, D)
    emb_err = None
    if check:
        eref = g.gguf.quants.dequantize(eraw.reshape(V, -1), g.tensors["token_embd.weight"].tensor_type).reshape(V, D)
        sub = D // es.shape[1]
        emb_err = float(np.abs((eq.astype(np.float32) - np.repeat(ez, sub, 1)) * np.repeat(es, sub, 1) - eref).max())
        say("embed %s: max |w - gguf| %.3g" % (ety, emb_err))

    eos = g.field("tokenizer.ggml.eos_token_id")
    eot = g.field("tokenizer.ggml.eot_token_id")
    eos_ids = sorted({int(x) for x in (eos, eot) if x is not None}) or [2]
    w = Writer(out_dir)
    cfg = dict(n_layers=L, hidden=D, n_heads=H, n_kv_heads=Hk, head_dim=Dh, inter=inter, vocab=V, eps=eps,
               rope_rows=ROPE_ROWS, rope_half=Dh // 2, attn_scale=Dh ** -0.5, enc="kq_huf", tied=int(tied),
               eos=",".join(str(x) for x in eos_ids))
    for k, v in cfg.items():
        w.cfg(k, v)

    def f32(name, v):
        v = np.asarray(v, np.float32)
        v = v.reshape(v.shape[0], -1) if v.ndim == 2 else v.reshape(1, -1)
        w.add(name, "f32", v.shape[0], v.shape[1], 1.0, 0, v.tobytes())

    w.add("embed", "raw8", V, D, 1.0, 0, eq.tobytes())
    f32("embed.rs", es)
    f32("embed.rsub", ez)
    inv = 1.0 / (theta ** (np.arange(0, Dh, 2, dtype=np.float64) / Dh))
    ang = np.arange(ROPE_ROWS, dtype=np.float64)[:, None] * inv[None]
    f32("cos", np.cos(ang))
    f32("sin", np.sin(ang))
    for i in range(L):
        f32("l%d.ln1" % i, g.f32("blk.%d.attn_norm.weight" % i))
        f32("l%d.ln2" % i, g.f32("blk.%d.ffn_norm.weight" % i))
    f32("lnf", g.f32("output_norm.weight"))
    code_bits = side_bits = weights = 0
    for name, (ty, q, side, ref) in order:
        if check and not np.array_equal(kquant.dequant(ty, q, side), ref):
            raise ValueError("%s: dequantisation of (codes, side bytes) differs from gguf-py" % name)
        n, k = q.shape
        paired = ty in kquant.PAIRED
        sym = np.ascontiguousarray((q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8) if paired else q)
        blob, _, _ = encode_huf8(sym)
        if check and not np.array_equal(cpu_decode_huf8(blob, *sym.shape), sym):
            raise ValueError("%s: the coded blob does not decode to its symbols" % name)
        w.add(name, "huf4p" if paired else "huf8", n, k, 1.0, 0, blob)
        w.add(name + ".kqs", "kq_" + ty, n, side.shape[1], 1.0, 0, np.ascontiguousarray(side).tobytes())
        code_bits += 8 * len(blob)
        side_bits += 8 * side.size
        weights += n * k
        say("%s %s %dx%d: %.3f + %.3f bits per weight" % (name, ty, n, k, 8 * len(blob) / (n * k), 8 * side.size / (n * k)))
    w.close()
    return dict(cfg=cfg, matmul_params=weights, code_bpw=code_bits / weights, side_bpw=side_bits / weights,
                embed_type=ety, embed_max_abs_err=emb_err, arch=g.arch)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("gguf")
    ap.add_argument("out")
    ap.add_argument("--no-check", action="store_true")
    a = ap.parse_args()
    print(build_bundle(a.gguf, a.out, check=not a.no_check, log=lambda *s: print(*s, file=sys.stderr)))


if __name__ == "__main__":
    main()
