"""Records what the REFERENCE project's bundle-builder code makes of the synthetic GGUF files of synth_gguf.py.

    python tests/golden/make_gguf_golden.py <path-to-reference-checkout>      (or set LW_REFERENCE)

The reference's functions are imported in place and called in the order its builder's main() calls them
(scripts/a2_kq_bundle.py:139-218: split, un-permute, qkv fusion, phi3 gate / up split, emb8, job = check + encode, Writer);
main() itself cannot run here because it reads a Hugging Face model directory, so the model shape is taken from the
synthetic file's constants.  Output: gguf_bundles.json = per case the manifest's tensor lines (name, enc, N, K, nbytes)
and the SHA-256 of every tensor's bytes in weights.bin, plus the cfg values that do not depend on a tokenizer.
"""
import hashlib
import json
import os
import sys
import tempfile

import numpy as np


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LW_REFERENCE", "")
    if not ref:
        sys.exit("usage: make_gguf_golden.py <reference checkout>   (or set LW_REFERENCE)")
    ref = os.path.abspath(ref)
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, ref)
    sys.path.insert(0, os.path.join(ref, "scripts"))
    sys.path.insert(0, here)
    import gguf
    import a2_kq_bundle as kqb
    from kq_code import split
    from kq_quant import permute
    from lazyweights.bundle import ROPE_ROWS, Writer, read_manifest
    import synth_gguf as sg

    out = {}
    tmp = tempfile.mkdtemp(prefix="gguf_golden_")
    for case, kw in sg.CASES.items():
        path = os.path.join(tmp, case + ".gguf")
        sg.write(path, **kw)
        r = gguf.GGUFReader(path)
        G = {t.name: t for t in r.tensors}
        L, Hq, Hk, Dh = sg.LAYERS, sg.HEADS, sg.KV_HEADS, sg.HEAD_DIM
        permuted = kw["arch"] == "llama"
        tied = "output.weight" not in G

        def mat(gn, hq=None):
            t = G[gn]
            ty = t.tensor_type
            K, N = (int(x) for x in t.shape)
            q, side, _ = split(ty, np.asarray(t.data).reshape(-1, gguf.GGML_QUANT_SIZES[ty][1]))
            q, side = q.reshape(N, K), side.reshape(N, -1)
            refw = gguf.quants.dequantize(np.asarray(t.data), ty).reshape(N, K)
            if hq is not None and permuted:
                inv = np.argsort(permute(np.arange(N), hq))
                q, side, refw = q[inv], side[inv], refw[inv]
            return ty, q, side, refw

        order = []
        for i in range(L):
            p = "blk.%d." % i
            if p + "attn_qkv.weight" in G:
                order.append(("l%d.qkv" % i, mat(p + "attn_qkv.weight")))
            else:
                qkv = [mat(p + "attn_q.weight", Hq), mat(p + "attn_k.weight", Hk), mat(p + "attn_v.weight")]
                if len({x[0] for x in qkv}) == 1:
                    order.append(("l%d.qkv" % i, (qkv[0][0],) + tuple(np.concatenate(x) for x in list(zip(*qkv))[1:])))
                else:
                    order += [("l%d.%s" % (i, n), x) for n, x in zip("qkv", qkv)]
            order.append(("l%d.o" % i, mat(p + "attn_output.weight")))
            if p + "ffn_gate.weight" in G:
                order += [("l%d.gate" % i, mat(p + "ffn_gate.weight")), ("l%d.up" % i, mat(p + "ffn_up.weight"))]
            else:
                ty, q, side, refw = mat(p + "ffn_up.weight")
                half = q.shape[0] // 2
                order += [("l%d.gate" % i, (ty, q[:half], side[:half], refw[:half])),
                          ("l%d.up" % i, (ty, q[half:], side[half:], refw[half:]))]
            order.append(("l%d.down" % i, mat(p + "ffn_down.weight")))
        order.append(("lm_head", mat("token_embd.weight" if tied else "output.weight")))
        et = G["token_embd.weight"]
        eq, es, ez = kqb.emb8(et.tensor_type, et)
        inv = 1.0 / (1e6 ** (np.arange(0, Dh, 2, dtype=np.float64) / Dh))
        ang = np.arange(ROPE_ROWS, dtype=np.float64)[:, None] * inv[None]
        bdir = os.path.join(tmp, case)
        w = Writer(bdir)

        def f32(name, v):
            v = np.asarray(v, np.float32)
            v = v.reshape(v.shape[0], -1) if v.ndim == 2 else v.reshape(1, -1)
            w.add(name, "f32", v.shape[0], v.shape[1], 1.0, 0, v.tobytes())

        w.add("embed", "raw8", eq.shape[0], eq.shape[1], 1.0, 0, eq.tobytes())
        f32("embed.rs", es)
        f32("embed.rsub", ez)
        f32("cos", np.cos(ang))
        f32("sin", np.sin(ang))
        for i in range(L):
            f32("l%d.ln1" % i, np.asarray(G["blk.%d.attn_norm.weight" % i].data, np.float32))
            f32("l%d.ln2" % i, np.asarray(G["blk.%d.ffn_norm.weight" % i].data, np.float32))
        f32("lnf", np.asarray(G["output_norm.weight"].data, np.float32))
        for nm, (ty, q, side, refw) in order:
            _, blob, _ = kqb.job((nm, ty, q, side, refw, False))      # the reference's checks run inside
            N, K = q.shape
            w.add(nm, "huf8" if kqb.BITS[ty] == 8 else "huf4p", N, K, 1.0, 0, blob)
            w.add(nm + ".kqs", "kq_" + ty.name, N, side.shape[1], 1.0, 0, np.ascontiguousarray(side).tobytes())
        w.close()
        _, ts = read_manifest(bdir)
        raw = open(os.path.join(bdir, "weights.bin"), "rb").read()
        out[case] = {"tensors": [[t["name"], t["enc"], t["N"], t["K"], t["nbytes"],
                                  hashlib.sha256(raw[t["offset"]:t["offset"] + t["nbytes"]]).hexdigest()] for t in ts],
                     "cfg": {"n_layers": L, "hidden": sg.HIDDEN, "n_heads": Hq, "n_kv_heads": Hk, "head_dim": Dh,
                             "inter": sg.INTER, "vocab": sg.VOCAB, "rope_rows": ROPE_ROWS, "tied": int(tied)}}
    with open(os.path.join(here, "gguf_bundles.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote gguf_bundles.json:", {k: len(v["tensors"]) for k, v in out.items()})


if __name__ == "__main__":
    main()
