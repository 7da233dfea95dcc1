// llama.cpp block formats <-> (codes in weight order, side bytes), and the n-gram draft cache of speculative decoding.
// Host code only (no CUDA).
//
// split / join restate the reference's scripts/kq_code.py:37-81 block by block with scalar index arithmetic.  Block
// layouts (one block = 256 weights):
//   Q4_K   144 B  side = bytes 0..15 (fp16 d, fp16 dmin, 12 scale bytes); 128 nibble bytes: weights 64 g .. 64 g + 31 are
//                 the low nibbles of bytes 32 g .., weights 64 g + 32 .. the high nibbles
//   Q5_K   176 B  side = bytes 0..15; 32 bytes of fifth bits (bit j of byte p = weight 32 j + p); nibbles as Q4_K
//   Q6_K   210 B  128 nibble bytes, 64 bytes of two-bit pieces, side = last 18 bytes (16 int8 scales, fp16 d)
//   IQ4_XS 136 B  side = bytes 0..7 (fp16 d, scales_h, 4 bytes scales_l); groups of 32 weights: low then high nibbles
//                 of 16 bytes
#include <algorithm>
#include <cstring>
#include <unordered_map>
#include <vector>

#include "../../include/lwb200.h"
#include "lw_host.h"

namespace lw {

int block_bytes(int fmt) { return fmt == kFmtQ4K ? 144 : fmt == kFmtQ5K ? 176 : fmt == kFmtQ6K ? 210 : fmt == kFmtIQ4XS ? 136 : 0; }

// Where code w of a block lives: nibble byte, nibble shift, and for the 5- and 6-bit formats the byte and shift of the
// upper bits.
struct CodePlace {
  int lo_byte, lo_shift, hi_byte, hi_shift, hi_mask;
};

static CodePlace place(int fmt, int w) {
  CodePlace p{0, 0, -1, 0, 0};
  if (fmt == kFmtQ4K || fmt == kFmtQ5K) {
    const int base = fmt == kFmtQ4K ? 16 : 48, g = w / 64, r = w % 64;
    p.lo_byte = base + 32 * g + (r & 31);
    p.lo_shift = r < 32 ? 0 : 4;
    if (fmt == kFmtQ5K) {
      p.hi_byte = 16 + (w & 31);
      p.hi_shift = w / 32;
      p.hi_mask = 1;
    }
  } else if (fmt == kFmtQ6K) {
    const int h = w / 128, k = (w % 128) / 32, q = w % 32;
    p.lo_byte = 64 * h + 32 * (k & 1) + q;
    p.lo_shift = 4 * (k >> 1);
    p.hi_byte = 128 + 32 * h + q;
    p.hi_shift = 2 * k;
    p.hi_mask = 3;
  } else {   // IQ4_XS
    const int g = w / 32, r = w % 32;
    p.lo_byte = 8 + 16 * g + (r & 15);
    p.lo_shift = r < 16 ? 0 : 4;
  }
  return p;
}

static void side_range(int fmt, int* off, int* len) {
  *len = side_bytes(fmt);
  *off = fmt == kFmtQ6K ? 192 : 0;
}

int split_blocks(int fmt, const uint8_t* blocks, long long nblk, uint8_t* q, uint8_t* side) {
  const int B = block_bytes(fmt);
  if (!B || !blocks || !q || !side || nblk < 0) {
    set_error("split_blocks: bad argument");
    return kErrArg;
  }
  CodePlace pl[256];
  for (int w = 0; w < 256; ++w) pl[w] = place(fmt, w);
  int so, sl;
  side_range(fmt, &so, &sl);
  for (long long b = 0; b < nblk; ++b) {
    const uint8_t* blk = blocks + b * B;
    uint8_t* qo = q + b * 256;
    for (int w = 0; w < 256; ++w) {
      unsigned v = (blk[pl[w].lo_byte] >> pl[w].lo_shift) & 15u;
      if (pl[w].hi_byte >= 0) v |= ((blk[pl[w].hi_byte] >> pl[w].hi_shift) & pl[w].hi_mask) << 4;
      qo[w] = static_cast<uint8_t>(v);
    }
    std::memcpy(side + b * sl, blk + so, sl);
  }
  return kOk;
}

int join_blocks(int fmt, const uint8_t* q, const uint8_t* side, long long nblk, uint8_t* blocks) {
  const int B = block_bytes(fmt);
  if (!B || !blocks || !q || !side || nblk < 0) {
    set_error("join_blocks: bad argument");
    return kErrArg;
  }
  CodePlace pl[256];
  for (int w = 0; w < 256; ++w) pl[w] = place(fmt, w);
  int so, sl;
  side_range(fmt, &so, &sl);
  const unsigned top = fmt == kFmtQ5K ? 32u : fmt == kFmtQ6K ? 64u : 16u;
  for (long long b = 0; b < nblk; ++b) {
    uint8_t* blk = blocks + b * B;
    const uint8_t* qi = q + b * 256;
    std::memset(blk, 0, B);
    for (int w = 0; w < 256; ++w) {
      const unsigned v = qi[w];
      if (v >= top) {
        set_error("join_blocks: code %u does not fit the format", v);
        return kErrArg;
      }
      blk[pl[w].lo_byte] |= static_cast<uint8_t>((v & 15u) << pl[w].lo_shift);
      if (pl[w].hi_byte >= 0) blk[pl[w].hi_byte] |= static_cast<uint8_t>((v >> 4) << pl[w].hi_shift);
    }
    std::memcpy(blk + so, side + b * sl, sl);
  }
  return kOk;
}

// ---------------------------------------------------------------------------------------------- n-gram draft cache
//
// The drafter of the reference's `spec --drafter ngramcache` mode (kernels/llmrt.cu:2604-2661, itself llama.cpp's
// prompt-lookup n-gram cache run without static / dynamic cache files): a context cache of the n-grams (n = 1..4) of the
// prompt and of every accepted token -> counts of the token that followed; a draft token comes from the longest n-gram
// whose most frequent continuation passes the lax thresholds (sample size, share).  Equal counts are broken by the
// iteration order of the containers, so the containers and hashes are the ones the reference uses (std::unordered_map,
// multiplicative token hash, xor over the n-gram); with the same standard library both draft alike.
struct NgramKey {
  int t[4];
  bool operator==(const NgramKey& o) const { return std::equal(t, t + 4, o.t); }
};
struct TokenHash {
  size_t operator()(int tok) const { return tok * 11400714819323198485llu; }
};
struct NgramKeyHash {
  size_t operator()(const NgramKey& k) const {
    size_t h = TokenHash{}(k.t[0]);
    for (int i = 1; i < 4; ++i) h ^= TokenHash{}(k.t[i]);
    return h;
  }
};

struct NgramCache {
  std::unordered_map<NgramKey, std::unordered_map<int, int32_t>, NgramKeyHash> grams;
  std::vector<int> seq;   // every token seen so far
  static NgramKey key(const int* x, int n) {
    NgramKey k;
    for (int i = 0; i < 4; ++i) k.t[i] = i < n ? x[i] : -1;
    return k;
  }
  // one token at a time, as the reference feeds it (llmrt.cu:3101-3103)
  void push(int tok) {
    seq.push_back(tok);
    const long S = static_cast<long>(seq.size());
    for (long n = 1; n <= 4; ++n)
      for (long i = std::max(S - 1, n); i < S; ++i) ++grams[key(&seq[i - n], static_cast<int>(n))][seq[i]];
  }
  int draft(int* out, int kmax) const {
    static const int min_n[4] = {2, 2, 1, 1}, min_pct[4] = {66, 50, 50, 50};
    const int S = static_cast<int>(seq.size());
    int nd = 0;
    if (S < 2) return 0;
    auto at = [&](int i) { return i < S ? seq[i] : out[i - S]; };
    while (nd < kmax) {
      int tok = -1;
      for (int n = 4; n >= 1 && tok < 0; --n) {
        if (S + nd - n < 0) continue;
        int g[4];
        for (int j = 0; j < n; ++j) g[j] = at(S + nd - n + j);
        const auto it = grams.find(key(g, n));
        if (it == grams.end()) continue;
        int best = 0, sum = 0, arg = -1;
        for (const auto& tc : it->second) {
          if (tc.second > best) {
            best = tc.second;
            arg = tc.first;
          }
          sum += tc.second;
        }
        if (sum < min_n[n - 1] || 100 * best < min_pct[n - 1] * sum) continue;
        tok = arg;
      }
      if (tok < 0) break;
      out[nd++] = tok;
    }
    return nd;
  }
};

}  // namespace lw

using namespace lw;

extern "C" {

int lw_block_bytes(int fmt) { return block_bytes(fmt); }

int lw_split_blocks(int fmt, const uint8_t* blocks, long long nblk, uint8_t* q, uint8_t* side) {
  return split_blocks(fmt, blocks, nblk, q, side);
}

int lw_join_blocks(int fmt, const uint8_t* q, const uint8_t* side, long long nblk, uint8_t* blocks) {
  return join_blocks(fmt, q, side, nblk, blocks);
}

void* lw_ngram_create(void) { return new NgramCache(); }

void lw_ngram_destroy(void* cache) { delete static_cast<NgramCache*>(cache); }

int lw_ngram_push(void* cache, const int* tokens, int n) {
  if (!cache || (n > 0 && !tokens) || n < 0) return kErrArg;
  for (int i = 0; i < n; ++i) static_cast<NgramCache*>(cache)->push(tokens[i]);
  return kOk;
}

int lw_ngram_draft(void* cache, int* out, int kmax) {
  if (!cache || kmax < 0 || (kmax > 0 && !out)) return kErrArg;
  return static_cast<NgramCache*>(cache)->draft(out, kmax);
}

}  // extern "C"
