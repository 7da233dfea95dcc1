"""A small seeded GGUF file with llama.cpp block-quantised matrices, written with gguf-py's GGUFWriter: the input of the
bundle-builder tests and of the script that records what the reference's builder code makes of the same file.

Shapes: hidden 512, 4 heads / 2 kv heads of 128, FFN 1024, vocabulary 512, 2 layers.  `arch` "llama": separate q / k / v
(q / k rows stored in llama.cpp's permuted order) and gate / up; `arch` "phi3": fused attn_qkv and ffn_up = [gate; up].
Block bytes are uniform random except the fp16 scales (a valid block for any byte pattern)."""
import numpy as np

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, VOCAB, LAYERS = 512, 4, 2, 128, 1024, 512, 2
BLOCK = {"Q4_K": 144, "Q5_K": 176, "Q6_K": 210, "IQ4_XS": 136, "Q8_0": 34}
D_OFFSETS = {"Q4_K": (0, 2), "Q5_K": (0, 2), "Q6_K": (208,), "IQ4_XS": (0,), "Q8_0": (0,)}


def random_blocks(ty, rows, cols, rng):
    per = 32 if ty == "Q8_0" else 256
    nb = rows * cols // per
    b = rng.integers(0, 256, (nb, BLOCK[ty]), dtype=np.uint8)
    for off in D_OFFSETS[ty]:
        b[:, off:off + 2] = rng.uniform(1e-3, 1e-2, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    if ty in ("Q4_K", "Q5_K"):
        b[:, 4:16] |= 1                      # no sub-block with scale 0 and a non-zero minimum (embedding rule)
    return b.reshape(rows, -1)


def write(path, arch="llama", attn=("Q4_K", "Q4_K", "Q4_K"), ffn="Q6_K", embed="Q6_K", tied=False, seed=0):
    """Writes the file; returns {tensor name: (type name, rows, cols, block bytes [rows, row bytes])}."""
    import gguf
    T = gguf.GGMLQuantizationType
    rng = np.random.default_rng(seed)
    w = gguf.GGUFWriter(path, arch)
    w.add_block_count(LAYERS)
    w.add_embedding_length(HIDDEN)
    w.add_head_count(HEADS)
    w.add_head_count_kv(KV_HEADS)
    w.add_feed_forward_length(INTER)
    w.add_layer_norm_rms_eps(1e-5)
    w.add_rope_freq_base(1e6)
    w.add_context_length(4096)
    w.add_eos_token_id(2)
    made = {}

    def quant(name, ty, rows, cols):
        b = random_blocks(ty, rows, cols, rng)
        w.add_tensor(name, b, raw_shape=b.shape, raw_dtype=getattr(T, ty))
        made[name] = (ty, rows, cols, b)

    def f32(name, n):
        v = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        w.add_tensor(name, v)
        made[name] = ("F32", 1, n, v)

    quant("token_embd.weight", embed, VOCAB, HIDDEN)
    for i in range(LAYERS):
        p = "blk.%d." % i
        f32(p + "attn_norm.weight", HIDDEN)
        if arch == "phi3":
            quant(p + "attn_qkv.weight", attn[0], (HEADS + 2 * KV_HEADS) * HEAD_DIM, HIDDEN)
        else:
            quant(p + "attn_q.weight", attn[0], HEADS * HEAD_DIM, HIDDEN)
            quant(p + "attn_k.weight", attn[1], KV_HEADS * HEAD_DIM, HIDDEN)
            quant(p + "attn_v.weight", attn[2], KV_HEADS * HEAD_DIM, HIDDEN)
        quant(p + "attn_output.weight", attn[0], HIDDEN, HEADS * HEAD_DIM)
        f32(p + "ffn_norm.weight", HIDDEN)
        if arch == "phi3":
            quant(p + "ffn_up.weight", ffn, 2 * INTER, HIDDEN)
        else:
            quant(p + "ffn_gate.weight", ffn, INTER, HIDDEN)
            quant(p + "ffn_up.weight", ffn, INTER, HIDDEN)
        quant(p + "ffn_down.weight", ffn, HIDDEN, INTER)
    f32("output_norm.weight", HIDDEN)
    if not tied:
        quant("output.weight", attn[0], VOCAB, HIDDEN)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return made


CASES = {
    "llama_fused": dict(arch="llama", attn=("Q4_K", "Q4_K", "Q4_K"), ffn="Q6_K", embed="Q6_K", tied=False, seed=1),
    "llama_split": dict(arch="llama", attn=("Q5_K", "Q5_K", "Q6_K"), ffn="IQ4_XS", embed="Q4_K", tied=True, seed=2),
    "phi3": dict(arch="phi3", attn=("IQ4_XS",) * 3, ffn="IQ4_XS", embed="Q8_0", tied=False, seed=3),
}
