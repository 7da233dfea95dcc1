#include "lw_host.h"

#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <array>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <queue>
#include <sstream>
#include <thread>

namespace lw {

// ------------------------------------------------------------------------------------------------ errors

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
}

const char* last_error() { return g_err; }

static thread_local int g_status = 0;
int note_status(int rc) {
  g_status = rc;
  return rc;
}
int last_status() { return g_status; }

int default_threads() {
  if (const char* e = getenv("LW_THREADS")) {   // host threads of the loader and the host codec (read at every use)
    const int n = atoi(e);
    if (n >= 1) return std::min(n, 256);
  }
  unsigned n = std::thread::hardware_concurrency();
  return n ? static_cast<int>(n) : 1;
}

template <class F>
static void parallel_for(int n, int threads, F&& body) {
  threads = std::max(1, std::min(threads, n));
  if (threads == 1) {
    for (int i = 0; i < n; ++i) body(i);
    return;
  }
  std::atomic<int> next(0);
  std::vector<std::thread> pool;
  for (int w = 0; w < threads; ++w)
    pool.emplace_back([&] {
      for (int i; (i = next.fetch_add(1)) < n;) body(i);
    });
  for (auto& t : pool) t.join();
}

// ------------------------------------------------------------------------------------------------ tables

// Depth of every used symbol in the Huffman tree.  Two nodes of equal weight are taken in creation order (leaves in
// symbol order, then merged nodes as they are made); that rule decides the lengths, so it must be kept.
void huffman_depths(const int64_t counts[256], int depth[256]) {
  struct Node {
    int64_t w;
    int serial;
    bool operator>(const Node& o) const { return w != o.w ? w > o.w : serial > o.serial; }
  };
  std::fill(depth, depth + 256, 0);
  std::vector<int> leaf_sym;
  for (int s = 0; s < 256; ++s)
    if (counts[s] > 0) leaf_sym.push_back(s);
  const int n = static_cast<int>(leaf_sym.size());
  if (n == 0) return;
  if (n == 1) {
    depth[leaf_sym[0]] = 1;
    return;
  }
  std::priority_queue<Node, std::vector<Node>, std::greater<Node>> heap;
  std::vector<int> parent(2 * n, -1);
  for (int i = 0; i < n; ++i) heap.push({counts[leaf_sym[i]], i});
  int serial = n;
  while (heap.size() > 1) {
    Node a = heap.top();
    heap.pop();
    Node b = heap.top();
    heap.pop();
    parent[a.serial] = parent[b.serial] = serial;
    heap.push({a.w + b.w, serial});
    ++serial;
  }
  for (int i = 0; i < n; ++i) {
    int d = 0;
    for (int v = i; parent[v] >= 0; v = parent[v]) ++d;
    depth[leaf_sym[i]] = d;
  }
}

void limited_lengths(const int64_t counts[256], uint8_t len[256], int limit) {
  limit = std::max(8, std::min(limit, kMaxLen));
  int depth[256];
  for (int shift = 0;; ++shift) {
    int64_t scaled[256];
    for (int s = 0; s < 256; ++s) scaled[s] = counts[s] > 0 ? std::max<int64_t>(counts[s] >> shift, 1) : 0;
    huffman_depths(scaled, depth);
    if (*std::max_element(depth, depth + 256) <= limit) break;
  }
  for (int s = 0; s < 256; ++s) len[s] = static_cast<uint8_t>(depth[s]);
}

static uint32_t reverse_bits(uint32_t v, int n) {
  uint32_t r = 0;
  for (int i = 0; i < n; ++i) r |= ((v >> i) & 1u) << (n - 1 - i);
  return r;
}

void table_from_lengths(const uint8_t len[256], HuffTable& t) {
  std::memset(&t, 0, sizeof t);
  std::memcpy(t.len, len, 256);
  uint32_t code = 0, filled = 0;
  for (int l = 1; l <= kMaxLen; ++l) {
    t.first[l] = code;
    t.base[l] = filled;
    for (int s = 0; s < 256; ++s) {
      if (len[s] != l) continue;
      t.sorted[filled++] = static_cast<uint8_t>(s);
      const uint32_t rev = reverse_bits(code, l);
      for (uint32_t hi = 0; hi < (1u << (kMaxLen - l)); ++hi)
        t.lut[rev | (hi << l)] = static_cast<uint16_t>(s | (l << 8));
      ++code;
      t.max_len = l;
    }
    t.limit[l] = code << (kMaxLen - l);
    code <<= 1;
  }
  t.nsym = static_cast<int>(filled);
}

int table_from_lut(const uint16_t* lut, HuffTable& t) {
  uint8_t len[256] = {0};
  for (int i = 0; i < kLutSize; ++i) {
    const int l = lut[i] >> 8, s = lut[i] & 255;
    if (l > kMaxLen) {
      set_error("table entry %d has length %d", i, l);
      return kErrFormat;
    }
    if (l == 0) continue;
    if (len[s] && len[s] != l) {
      set_error("table gives symbol %d two lengths (%d, %d)", s, len[s], l);
      return kErrFormat;
    }
    len[s] = static_cast<uint8_t>(l);
  }
  table_from_lengths(len, t);
  if (t.nsym == 0) {
    set_error("table has no symbols");
    return kErrFormat;
  }
  // Kraft: a complete code unless it is the one-symbol table (a single length-1 code)
  uint32_t kraft = 0;
  for (int s = 0; s < 256; ++s)
    if (len[s]) kraft += 1u << (kMaxLen - len[s]);
  const bool single = t.nsym == 1 && t.max_len == 1;
  if (!single && kraft != (1u << kMaxLen)) {
    set_error("table is not a complete prefix code (Kraft sum %u / 2048)", kraft);
    return kErrFormat;
  }
  if (std::memcmp(t.lut, lut, sizeof t.lut) != 0) {
    set_error("table is not the canonical table of its code lengths");
    return kErrFormat;
  }
  return kOk;
}

static float grid_of(int fmt, int q) {
  static const float iq4[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
  if (fmt == kFmtIQ4XS) return iq4[q & 15];
  return static_cast<float>(q) - (fmt == kFmtQ6K ? 32.f : 0.f);
}

// 32-bit decode table of the fused kernels: bits 28-31 = code length (recovered by one multiply-high).  Paired
// formats: byte 0 = the grid value of the low nibble as a signed 8-bit integer, byte 1 = that of the high nibble - the
// multiplier operand of a dp2a instruction.  Unpaired formats: the grid value sign-extended over bits 0-27, so that a
// plain 32-bit multiply-add with the activation accumulates the exact sum in its low 28 bits (the length field only
// disturbs bits 28-31) and byte 0 is still the signed 8-bit value.
static uint32_t value_bytes(int fmt, uint32_t sym) {
  if (is_paired(fmt)) {
    const int v0 = static_cast<int>(grid_of(fmt, sym & 15)), v1 = static_cast<int>(grid_of(fmt, sym >> 4));
    return (static_cast<uint32_t>(v0) & 255u) | ((static_cast<uint32_t>(v1) & 255u) << 8);
  }
  if (fmt == kFmtQ5K || fmt == kFmtQ6K)   // one grid value, sign-extended over the 28 bits below the length field
    return static_cast<uint32_t>(static_cast<int>(grid_of(fmt, sym & (fmt == kFmtQ6K ? 63 : 31)))) & 0x0FFFFFFFu;
  return sym;
}

void fat_table(const HuffTable& t, int fmt, uint32_t out[kLutSize]) {
  for (int i = 0; i < kLutSize; ++i) out[i] = (static_cast<uint32_t>(t.lut[i] >> 8) << 28) | value_bytes(fmt, t.lut[i] & 255u);
}

void comparator_table(const HuffTable& t, int fmt, uint32_t out[kCmpTabWords]) {
  std::memset(out, 0, sizeof(uint32_t) * kCmpTabWords);
  for (int l = 1; l <= kMaxLen; ++l) {
    out[l] = t.limit[l];   // = (first[l] + count[l]) << (11 - l): codes of length <= l lie below it
    out[12 + l] = t.base[l] - t.first[l];
  }
  for (int i = 0; i < t.nsym; ++i) out[24 + i] = value_bytes(fmt, t.sorted[i]);
}

void symbol_values(int fmt, uint32_t out[256]) {
  for (uint32_t s = 0; s < 256; ++s) out[s] = value_bytes(fmt, s);
}

// ------------------------------------------------------------------------------------------------ blob

int make_view(const uint8_t* blob, size_t nbytes, int N, int Ks, BlobView& v) {
  if (N <= 0 || Ks <= 0 || N % kTileRows || Ks % kTileSyms) {
    set_error("matrix of %d x %d symbols is not a multiple of 64 x 256", N, Ks);
    return kErrArg;
  }
  v.data = blob;
  v.nbytes = nbytes;
  v.N = N;
  v.Ks = Ks;
  v.KT = Ks / kTileSyms;
  v.T = (N / kTileRows) * v.KT;
  const size_t head = 2 * kLutSize + static_cast<size_t>(v.T) * kLanes * 4;
  if (nbytes < head + 12 || (nbytes - head) % 4) {
    set_error("blob of %zu bytes is too short for %d tiles", nbytes, v.T);
    return kErrFormat;
  }
  return kOk;
}

int encode_huf8(const uint8_t* sym, int N, int Ks, std::vector<uint8_t>& blob, int64_t* nbits, int limit, int threads) {
  if (N <= 0 || Ks <= 0 || N % kTileRows || Ks % kTileSyms) {
    set_error("matrix of %d x %d symbols is not a multiple of 64 x 256", N, Ks);
    return kErrArg;
  }
  const int KT = Ks / kTileSyms, NT = N / kTileRows, T = NT * KT;
  threads = std::max(1, std::min(threads, T));
  // counts, per range of tiles
  std::vector<std::array<int64_t, 256>> part(threads);
  for (auto& h : part) h.fill(0);
  auto tile_range = [&](int w, int& t0, int& t1) {
    t0 = static_cast<int>(static_cast<int64_t>(T) * w / threads);
    t1 = static_cast<int>(static_cast<int64_t>(T) * (w + 1) / threads);
  };
  auto tile_row = [&](int t, int lane, int half) {
    return sym + (static_cast<size_t>(t / KT) * kTileRows + half * 32 + lane) * Ks + static_cast<size_t>(t % KT) * kTileSyms;
  };
  parallel_for(threads, threads, [&](int w) {
    int t0, t1;
    tile_range(w, t0, t1);
    auto& h = part[w];
    for (int t = t0; t < t1; ++t)
      for (int r = 0; r < kTileRows; ++r) {
        const uint8_t* row = tile_row(t, r & 31, r >> 5);
        for (int c = 0; c < kTileSyms; ++c) ++h[row[c]];
      }
  });
  int64_t hist[256] = {0};
  for (auto& h : part)
    for (int s = 0; s < 256; ++s) hist[s] += h[s];
  uint8_t len[256];
  limited_lengths(hist, len, limit);
  HuffTable tab;
  table_from_lengths(len, tab);
  uint32_t rcode[256] = {0};
  {
    uint32_t code = 0;
    for (int l = 1; l <= kMaxLen; ++l) {
      for (int s = 0; s < 256; ++s)
        if (len[s] == l) rcode[s] = reverse_bits(code++, l);
      code <<= 1;
    }
  }
  uint64_t total = 0;
  for (int s = 0; s < 256; ++s) total += static_cast<uint64_t>(hist[s]) * len[s];
  if (total >= (1ull << 32)) {
    set_error("payload of %llu bits does not fit 32-bit lane offsets", static_cast<unsigned long long>(total));
    return kErrTooLarge;
  }
  const size_t nwords = (total + 31) / 32 + 2;
  const size_t head = 2 * kLutSize + static_cast<size_t>(T) * kLanes * 4;
  blob.assign(head + nwords * 4, 0);
  std::memcpy(blob.data(), tab.lut, 2 * kLutSize);
  uint32_t* starts = reinterpret_cast<uint32_t*>(blob.data() + 2 * kLutSize);
  uint32_t* words = reinterpret_cast<uint32_t*>(blob.data() + head);
  // where every range of tiles starts in the stream: the bits of the ranges before it
  std::vector<uint64_t> range_bits(threads + 1, 0);
  for (int w = 0; w < threads; ++w) {
    uint64_t b = 0;
    for (int s = 0; s < 256; ++s) b += static_cast<uint64_t>(part[w][s]) * len[s];
    range_bits[w + 1] = range_bits[w] + b;
  }
  // Lanes follow one another bit by bit, so two ranges can share a word: whole words are stored, the first and the last
  // word of a range are OR-ed in atomically (the words start as zero and the ranges' bits are disjoint).
  parallel_for(threads, threads, [&](int w) {
    int t0, t1;
    tile_range(w, t0, t1);
    if (t0 == t1) return;
    uint64_t pos = range_bits[w];
    size_t wi = pos >> 5;
    const size_t first = wi, last = (range_bits[w + 1] - 1) >> 5;
    int fill = static_cast<int>(pos & 31);
    uint64_t acc = 0;   // the bits of word wi and beyond, bit `fill` is the next free one
    auto put = [&](uint32_t v) {
      if (wi == first || wi == last)
        __atomic_fetch_or(words + wi, v, __ATOMIC_RELAXED);
      else
        words[wi] = v;
      ++wi;
    };
    for (int t = t0; t < t1; ++t)
      for (int lane = 0; lane < kLanes; ++lane) {
        starts[static_cast<size_t>(t) * kLanes + lane] = static_cast<uint32_t>(pos);
        for (int half = 0; half < 2; ++half) {
          const uint8_t* row = tile_row(t, lane, half);
          for (int c = 0; c < kTileSyms; ++c) {
            const int s = row[c], l = len[s];
            acc |= static_cast<uint64_t>(rcode[s]) << fill;
            fill += l;
            pos += l;
            if (fill >= 32) {
              put(static_cast<uint32_t>(acc));
              acc >>= 32;
              fill -= 32;
            }
          }
        }
      }
    if (fill) put(static_cast<uint32_t>(acc));
  });
  if (nbits) *nbits = static_cast<int64_t>(total);
  return kOk;
}

// Grouped decoding (lw_gemv1.cuh) normalises the bit window once per group of g symbols and refills at most one word
// after it.  With bp < 32 the window offset at the start of a group, that is exact iff every symbol of the group
// starts at most 31 bits into the group and bp plus the group's bits stays below 64.  rel[i] = bit offset of symbol i
// inside its chain (rel[n] = chain length); the phase of the groups restarts every `quad` symbols.
static uint8_t scan_chain(const uint16_t* rel, int n, int quad) {
  uint8_t bad = 0;
  for (int g = kScanMinG; g <= kScanMaxG; ++g) {
    bool ok = true;
    // a kernel that keeps fewer copies of its table starts reading one bit into the chain's pad (lw_ring.cuh,
    // GroupChain::init): a group must be exact from either starting offset
    for (uint32_t bp0 = 0; bp0 < 2 && ok; ++bp0) {
      uint32_t bp = bp0;
      for (int q0 = 0; q0 < n && ok; q0 += quad)
        for (int i = q0; i < q0 + quad && ok; i += g) {
          const int last = std::min(i + g, q0 + quad) - 1;   // last symbol of the group
          if (rel[last] - rel[i] > 31) ok = false;
          bp += rel[last + 1] - rel[i];
          if (bp >= 64) ok = false;
          if (bp >= 32) bp -= 32;
        }
    }
    if (!ok) bad |= static_cast<uint8_t>(1u << (g - kScanMinG));
  }
  return bad;
}

int walk_blob(const BlobView& v, const HuffTable& tab, int split, int threads, std::vector<uint32_t>* chain_start,
              std::vector<uint32_t>* lane_end, uint8_t* out, GroupScan* scan) {
  if (split != 1 && split != 2 && split != 4) {
    set_error("split must be 1, 2 or 4");
    return kErrArg;
  }
  const int G = 2 * split, seg = kTileSyms / split;
  const size_t nl = static_cast<size_t>(v.T) * kLanes;
  if (chain_start) chain_start->assign(nl * G, 0);
  std::vector<uint32_t> ends_local;
  std::vector<uint32_t>& ends = lane_end ? *lane_end : ends_local;
  ends.assign(nl, 0);
  const uint32_t* starts = v.lane_start();
  const uint8_t* pay = reinterpret_cast<const uint8_t*>(v.payload());
  const uint64_t pay_bits = static_cast<uint64_t>(v.payload_words() - 2) * 32;   // the two tail words are padding
  std::atomic<int> bad(0);
  if (scan) scan->mask.assign(static_cast<size_t>(v.T) * split, 0);
  parallel_for(v.T, threads, [&](int t) {
    if (bad.load(std::memory_order_relaxed)) return;
    const int tr = t / v.KT, tc = t % v.KT;
    uint16_t rel[kTileSyms + 1];
    for (int lane = 0; lane < kLanes; ++lane) {
      uint64_t bp = starts[static_cast<size_t>(t) * kLanes + lane];
      for (int half = 0; half < 2; ++half) {
        uint64_t chain0 = bp;
        uint8_t longcode = 0;
        uint8_t* row = out ? out + (static_cast<size_t>(tr) * kTileRows + half * 32 + lane) * v.Ks + tc * kTileSyms
                           : nullptr;
        for (int c = 0; c < kTileSyms; ++c) {
          if (chain_start && c % seg == 0)
            (*chain_start)[(static_cast<size_t>(t) * kLanes + lane) * G + half * split + c / seg] =
                static_cast<uint32_t>(bp);
          if (bp >= pay_bits) {
            bad.store(1);
            return;
          }
          uint64_t w;
          std::memcpy(&w, pay + ((bp >> 5) << 2), 8);
          const uint16_t e = tab.lut[(w >> (bp & 31)) & (kLutSize - 1)];
          if ((e >> 8) == 0) {
            bad.store(2);
            return;
          }
          if (row) row[c] = static_cast<uint8_t>(e);
          if (scan) {
            if (c % seg == 0) {
              chain0 = bp;
              longcode = 0;
            }
            rel[c % seg] = static_cast<uint16_t>(bp - chain0);
            if ((e >> 8) > 10) longcode = 0x80;
          }
          bp += e >> 8;
          if (scan && c % seg == seg - 1) {
            rel[seg] = static_cast<uint16_t>(bp - chain0);
            scan->mask[static_cast<size_t>(t) * split + c / seg] |= scan_chain(rel, seg, scan->quad_syms) | longcode;
          }
        }
      }
      ends[static_cast<size_t>(t) * kLanes + lane] = static_cast<uint32_t>(bp);
      if (bp > pay_bits) {
        bad.store(1);
        return;
      }
    }
  });
  if (bad.load() == 1) {
    set_error("a lane runs past the end of the payload");
    return kErrFormat;
  }
  if (bad.load() == 2) {
    set_error("the payload holds a bit pattern the table does not resolve");
    return kErrFormat;
  }
  if (starts[0] != 0) {
    set_error("first lane does not start at bit 0");
    return kErrFormat;
  }
  for (size_t i = 0; i + 1 < nl; ++i)
    if (ends[i] != starts[i + 1]) {
      set_error("lane %zu ends at bit %u but the next lane starts at bit %u", i, ends[i], starts[i + 1]);
      return kErrFormat;
    }
  if ((static_cast<uint64_t>(ends[nl - 1]) + 31) / 32 + 2 != v.payload_words()) {
    set_error("payload has %zu words but the lanes cover %u bits", v.payload_words(), ends[nl - 1]);
    return kErrFormat;
  }
  return kOk;
}

// Scales of tile row `row`, column segment `seg` of tile column tc: the four sub-blocks that a work unit covers.
// sc / mn: one value per byte; dd: fp16 d (low half) and fp16 dmin (reference block formulas: kernels/llmrt.cu:126-149).
static void unit_scales(int fmt, const uint8_t* side_row, int tc, int seg, int split, uint32_t* sc, uint32_t* mn,
                        uint32_t* dd) {
  const int subs_per_tile = (is_paired(fmt) ? 512 : 256) / sub_width(fmt);
  unit_scales_at(fmt, side_row, tc * subs_per_tile + seg * (subs_per_tile / split), sc, mn, dd);
}

// The same for the four sub-blocks sub0 .. sub0 + 3, counted along the row (they must lie in one super-block).
void unit_scales_at(int fmt, const uint8_t* side_row, int sub0, uint32_t* sc, uint32_t* mn, uint32_t* dd) {
  const int sb = side_bytes(fmt);
  const int per_block = 256 / sub_width(fmt);                            // sub-blocks per super-block
  const uint8_t* blk = side_row + static_cast<size_t>(sub0 / per_block) * sb;
  const int j0 = sub0 % per_block;
  *sc = *mn = 0;
  if (fmt == kFmtQ6K) {
    for (int j = 0; j < 4; ++j) *sc |= static_cast<uint32_t>(blk[j0 + j]) << (8 * j);
    *dd = blk[16] | (blk[17] << 8);
  } else if (fmt == kFmtIQ4XS) {
    const uint32_t sh = blk[2] | (blk[3] << 8);
    for (int j = 0; j < 4; ++j) {
      const int jj = j0 + j;
      const uint32_t ls = ((blk[4 + jj / 2] >> (4 * (jj & 1))) & 15u) | (((sh >> (2 * jj)) & 3u) << 4);
      *sc |= ls << (8 * j);
    }
    *dd = blk[0] | (blk[1] << 8);
  } else {
    const uint8_t* q = blk + 4;   // llama.cpp get_scale_min_k4
    for (int j = 0; j < 4; ++j) {
      const int jj = j0 + j;
      uint32_t s6, m6;
      if (jj < 4) {
        s6 = q[jj] & 63u;
        m6 = q[jj + 4] & 63u;
      } else {
        s6 = (q[jj + 4] & 15u) | ((q[jj - 4] >> 6) << 4);
        m6 = (q[jj + 4] >> 4) | ((q[jj] >> 6) << 4);
      }
      *sc |= s6 << (8 * j);
      *mn |= m6 << (8 * j);
    }
    *dd = blk[0] | (blk[1] << 8) | (blk[2] << 16) | (static_cast<uint32_t>(blk[3]) << 24);
  }
}

int relayout(const BlobView& v, int split, int pad, const std::vector<uint32_t>& chain_start,
             const std::vector<uint32_t>& lane_end, int threads, std::vector<uint32_t>& group_base,
             std::vector<uint32_t>& words, uint32_t* max_group_words, uint32_t* max_tile_words, int fmt,
             const uint8_t* side) {
  const int G = 2 * split;
  const size_t ngroups = static_cast<size_t>(v.T) * G;
  const uint32_t side_words = side ? unit_side_words(fmt) : 0;
  if (side && (is_paired(fmt) ? 512 : 256) / sub_width(fmt) != 4 * split) {
    set_error("relayout: a column segment must hold exactly four sub-blocks to carry its scales");
    return kErrArg;
  }
  group_base.assign(ngroups + 1, 0);
  // group gi of a tile = (column segment gi / 2, rows half gi % 2): the two halves of a segment are adjacent, so a
  // warp that decodes rows l and l + 32 over one segment stages one contiguous piece.  In stream order the lane's
  // chains run half-major (row l: all segments, then row l + 32).
  auto chain_bits = [&](size_t t, int lane, int gi, uint32_t* begin) {
    const size_t li = t * kLanes + lane;
    const int ci = (gi & 1) * split + (gi >> 1);
    const uint32_t b = chain_start[li * G + ci];
    const uint32_t e = ci + 1 < G ? chain_start[li * G + ci + 1] : lane_end[li];
    *begin = b;
    return e - b;
  };
  // pass 1: words per chain of every group (its longest chain), then the running base
  std::vector<uint32_t> gw(ngroups);
  uint32_t mg = 0, mt = 0;
  uint64_t total = 0;
  for (size_t t = 0; t < static_cast<size_t>(v.T); ++t) {
    uint32_t tile_words = 0;
    for (int g = 0; g < G; ++g) {
      uint32_t w = 0, b;
      for (int lane = 0; lane < kLanes; ++lane) w = std::max(w, (chain_bits(t, lane, g, &b) + pad + 31) / 32);
      gw[t * G + g] = w;
      tile_words += w * kLanes;
    }
    tile_words += side_words * split;
    mt = std::max(mt, tile_words);
    for (int seg = 0; seg < split; ++seg)
      mg = std::max(mg, (gw[t * G + 2 * seg] + gw[t * G + 2 * seg + 1]) * kLanes + side_words);
    for (int g = 0; g < G; ++g) {
      if (total > 0xFFFFFFFFull) {
        set_error("matrix needs more than 2^32 device words");
        return kErrTooLarge;
      }
      group_base[t * G + g] = static_cast<uint32_t>(total);
      total += static_cast<uint64_t>(gw[t * G + g]) * kLanes + ((g & 1) ? side_words : 0);
    }
  }
  if (total > 0xFFFFFFFFull) {
    set_error("matrix needs more than 2^32 device words");
    return kErrTooLarge;
  }
  group_base[ngroups] = static_cast<uint32_t>(total);
  words.assign(total + kTailWords, 0);
  const uint32_t* pay = v.payload();
  const size_t side_row_bytes = side ? static_cast<size_t>(v.Ks) * (is_paired(fmt) ? 2 : 1) / 256 * side_bytes(fmt) : 0;
  parallel_for(v.T, threads, [&](int t) {
    for (int g = 0; g < G; ++g) {
      uint32_t* dst = words.data() + group_base[static_cast<size_t>(t) * G + g];
      for (int lane = 0; lane < kLanes; ++lane) {
        uint32_t b;
        const uint32_t nbits = chain_bits(t, lane, g, &b) + pad;   // the chain starts with `pad` zero bits
        for (uint32_t i = 0; i * 32 < nbits; ++i) {
          uint32_t w;
          if (i == 0) {
            const uint64_t x = pay[b >> 5] | (static_cast<uint64_t>(pay[(b >> 5) + 1]) << 32);
            w = static_cast<uint32_t>(x >> (b & 31)) << pad;
          } else {
            const uint64_t p = static_cast<uint64_t>(b) + i * 32ull - pad;
            const uint64_t x = pay[p >> 5] | (static_cast<uint64_t>(pay[(p >> 5) + 1]) << 32);
            w = static_cast<uint32_t>(x >> (p & 31));
          }
          const uint32_t left = nbits - i * 32;
          if (left < 32) w &= (1u << left) - 1;
          dst[static_cast<size_t>(i) * kLanes + lane] = w;
        }
      }
      if (side_words && (g & 1)) {   // the unit's scales follow its second group
        uint32_t* sd = dst + static_cast<size_t>(gw[static_cast<size_t>(t) * G + g]) * kLanes;
        uint16_t* sh = reinterpret_cast<uint16_t*>(sd);
        const int tr = t / v.KT, tc = t % v.KT;
        for (int r = 0; r < kTileRows; ++r) {
          uint32_t sc, mn, dd;
          unit_scales(fmt, side + (static_cast<size_t>(tr) * kTileRows + r) * side_row_bytes, tc, g >> 1, split, &sc, &mn, &dd);
          sd[r] = (fmt == kFmtQ4K || fmt == kFmtQ5K) ? dd : sc;
          if (fmt == kFmtQ4K || fmt == kFmtQ5K) {
            sd[64 + r] = sc;
            sd[128 + r] = mn;
          } else {
            sh[128 + r] = static_cast<uint16_t>(dd);
          }
        }
      }
    }
  });
  if (max_group_words) *max_group_words = mg;
  if (max_tile_words) *max_tile_words = mt;
  return kOk;
}

int twin_bits(int fmt) { return fmt == kFmtQ5K ? 5 : fmt == kFmtQ6K ? 6 : 8; }

int build_twin(const uint8_t* sym, int N, int Ks, int fmt, const uint8_t* side, int threads,
               std::vector<uint32_t>& group_base, std::vector<uint32_t>& words, uint32_t* unit_words) {
  if (fmt < kFmtQ4K || fmt > kFmtIQ4XS || !sym || !side || N % kTileRows || Ks % kTileSyms) {
    set_error("build_twin: bad argument");
    return kErrArg;
  }
  const int split = default_split(fmt), G = 2 * split, B = twin_bits(fmt), seg_syms = kTileSyms / split;
  const int KT = Ks / kTileSyms, T = (N / kTileRows) * KT;
  const uint32_t cw = static_cast<uint32_t>(seg_syms * B / 32);            // words per chain (whole words by construction)
  const uint32_t side_words = unit_side_words(fmt), uw = 2 * cw * kLanes + side_words;
  const uint64_t total = static_cast<uint64_t>(T) * split * uw;
  if (total > 0xFFFFFFFFull) {
    set_error("twin needs more than 2^32 device words");
    return kErrTooLarge;
  }
  group_base.assign(static_cast<size_t>(T) * G + 1, 0);
  words.assign(total + kTailWords, 0);
  const size_t side_row_bytes = static_cast<size_t>(Ks) * (is_paired(fmt) ? 2 : 1) / 256 * side_bytes(fmt);
  const uint32_t mask = (1u << B) - 1u;
  parallel_for(T, threads, [&](int t) {
    const int tr = t / KT, tc = t % KT;
    for (int g = 0; g < G; ++g) {
      const int seg = g >> 1, half = g & 1;
      const uint32_t base = (static_cast<uint32_t>(t) * split + seg) * uw + half * cw * kLanes;
      group_base[static_cast<size_t>(t) * G + g] = base;
      for (int lane = 0; lane < kLanes; ++lane) {
        const uint8_t* row = sym + (static_cast<size_t>(tr) * kTileRows + half * 32 + lane) * Ks + tc * kTileSyms + seg * seg_syms;
        uint64_t acc = 0;
        int fill = 0;
        uint32_t wi = 0;
        for (int c = 0; c < seg_syms; ++c) {
          uint32_t v = row[c];
          if (fmt == kFmtQ6K) v = (v - 32u) & mask;   // stored centred, so that a sign extension gives the grid value
          acc |= static_cast<uint64_t>(v & mask) << fill;
          fill += B;
          if (fill >= 32) {
            words[base + static_cast<size_t>(wi++) * kLanes + lane] = static_cast<uint32_t>(acc);
            acc >>= 32;
            fill -= 32;
          }
        }
      }
      if (half) {
        uint32_t* sd = words.data() + base + static_cast<size_t>(cw) * kLanes;
        uint16_t* sh = reinterpret_cast<uint16_t*>(sd);
        for (int r = 0; r < kTileRows; ++r) {
          uint32_t sc, mn, dd;
          unit_scales(fmt, side + (static_cast<size_t>(tr) * kTileRows + r) * side_row_bytes, tc, seg, split, &sc, &mn, &dd);
          sd[r] = (fmt == kFmtQ4K || fmt == kFmtQ5K) ? dd : sc;
          if (fmt == kFmtQ4K || fmt == kFmtQ5K) {
            sd[64 + r] = sc;
            sd[128 + r] = mn;
          } else {
            sh[128 + r] = static_cast<uint16_t>(dd);
          }
        }
      }
    }
  });
  group_base[static_cast<size_t>(T) * G] = static_cast<uint32_t>(total);
  if (unit_words) *unit_words = uw;
  return kOk;
}

// ------------------------------------------------------------------------------------------------ bundle

int read_manifest(const std::string& dir, Manifest& m) {
  std::ifstream f(dir + "/manifest.txt");
  if (!f) {
    set_error("cannot open %s/manifest.txt", dir.c_str());
    return kErrGeneric;
  }
  std::string line;
  while (std::getline(f, line)) {
    std::istringstream is(line);
    std::string tag;
    if (!(is >> tag)) continue;
    if (tag == "cfg") {
      std::string k, val;
      if (is >> k >> val) m.cfg[k] = val;
    } else if (tag == "t") {
      TensorEntry t;
      if (!(is >> t.name >> t.enc >> t.N >> t.K >> t.scale >> t.zp >> t.offset >> t.nbytes)) {
        set_error("bad manifest line: %s", line.c_str());
        return kErrFormat;
      }
      if (t.N < 0 || t.K < 0 || t.offset < 0 || t.nbytes < 0 || t.offset % kBlobAlign) {
        set_error("tensor %s: bad shape, size or alignment", t.name.c_str());
        return kErrFormat;
      }
      m.by_name[t.name] = static_cast<int>(m.tensors.size());
      m.tensors.push_back(t);
    }
  }
  return kOk;
}

int read_blob(int fd, const TensorEntry& t, std::vector<uint8_t>& out) {
  out.resize(static_cast<size_t>(t.nbytes) + 16);   // slack: the decoder reads 8 bytes at a time
  size_t done = 0;
  while (done < static_cast<size_t>(t.nbytes)) {
    const ssize_t r = pread(fd, out.data() + done, t.nbytes - done, t.offset + done);
    if (r <= 0) {
      set_error("tensor %s: weights.bin is shorter than the manifest says", t.name.c_str());
      return kErrFormat;
    }
    done += static_cast<size_t>(r);
  }
  std::memset(out.data() + t.nbytes, 0, 16);
  return kOk;
}

// Everything rt_forward will index with the cfg's sizes is compared with the tensors' shapes here, on the host, so
// that an inconsistent manifest is refused before anything is uploaded or launched.
int validate_model(const Manifest& m) {
  auto geti = [&](const char* k, int def) {
    auto it = m.cfg.find(k);
    return it == m.cfg.end() ? def : atoi(it->second.c_str());
  };
  const int L = geti("n_layers", 0), D = geti("hidden", 0), H = geti("n_heads", 0), Hk = geti("n_kv_heads", H);
  const int Dh = geti("head_dim", H ? D / H : 0), I = geti("inter", 0), V = geti("vocab", 0);
  const int rope_rows = geti("rope_rows", 4096);
  if (L <= 0 || D <= 0 || H <= 0 || Hk <= 0 || Dh <= 0 || I <= 0 || V <= 0 || H % Hk || Dh % 8 || Dh > 128 || rope_rows <= 0) {
    set_error("bundle cfg: bad model shape (head_dim must be a multiple of 8, at most 128)");
    return kErrFormat;
  }
  auto want = [&](const std::string& name, const char* enc, long long n, long long k, bool any_rows) -> int {
    const TensorEntry* t = m.find(name);
    if (!t) {
      set_error("bundle has no tensor %s", name.c_str());
      return kErrFormat;
    }
    if (enc && t->enc != enc) {
      set_error("tensor %s is %s, expected %s", name.c_str(), t->enc.c_str(), enc);
      return kErrFormat;
    }
    if ((!any_rows && t->N != n) || t->K != k) {
      set_error("tensor %s is %d x %d, the cfg wants %lld x %lld", name.c_str(), t->N, t->K, n, k);
      return kErrFormat;
    }
    return kOk;
  };
  auto coded = [&](const std::string& name, long long n, long long k) -> int {
    const TensorEntry* t = m.find(name);
    if (!t || (t->enc != "huf8" && t->enc != "huf4p")) {
      set_error("bundle has no coded matrix %s", name.c_str());
      return kErrFormat;
    }
    if (t->N != n || t->K != k) {
      set_error("matrix %s is %d x %d, the cfg wants %lld x %lld", name.c_str(), t->N, t->K, n, k);
      return kErrFormat;
    }
    if (!m.find(name + ".kqs")) {
      set_error("matrix %s has no side tensor", name.c_str());
      return kErrFormat;
    }
    return kOk;
  };
  int rc;
  const TensorEntry* emb = m.find("embed");
  if (!emb || emb->K != D || emb->N <= 0 || (emb->enc != "f16" && emb->enc != "raw8")) {
    set_error("embed must be an f16 or raw8 tensor with %d columns", D);
    return kErrFormat;
  }
  if (emb->enc == "raw8") {
    const TensorEntry* rs = m.find("embed.rs");
    const TensorEntry* rsub = m.find("embed.rsub");
    if (!rs || !rsub || rs->enc != "f32" || rsub->enc != "f32" || rs->N != emb->N || rsub->N != emb->N || rs->K <= 0 ||
        rs->K > D || D % rs->K || rsub->K != rs->K) {
      set_error("embed.rs / embed.rsub must be f32 [%d, G] with G dividing %d", emb->N, D);
      return kErrFormat;
    }
  }
  if ((rc = want("cos", "f32", rope_rows, Dh / 2, false)) || (rc = want("sin", "f32", rope_rows, Dh / 2, false)) ||
      (rc = want("lnf", "f32", 1, D, false)))
    return rc;
  const long long QKV = static_cast<long long>(H + 2 * Hk) * Dh;
  for (int l = 0; l < L; ++l) {
    const std::string pre = "l" + std::to_string(l) + ".";
    if ((rc = want(pre + "ln1", "f32", 1, D, false)) || (rc = want(pre + "ln2", "f32", 1, D, false))) return rc;
    if (m.find(pre + "qkv")) {
      if ((rc = coded(pre + "qkv", QKV, D))) return rc;
    } else if ((rc = coded(pre + "q", static_cast<long long>(H) * Dh, D)) ||
               (rc = coded(pre + "k", static_cast<long long>(Hk) * Dh, D)) ||
               (rc = coded(pre + "v", static_cast<long long>(Hk) * Dh, D))) {
      return rc;
    }
    if ((rc = coded(pre + "o", D, static_cast<long long>(H) * Dh)) || (rc = coded(pre + "gate", I, D)) ||
        (rc = coded(pre + "up", I, D)) || (rc = coded(pre + "down", D, I)))
      return rc;
  }
  return coded("lm_head", V, D);
}

int format_of_side_enc(const std::string& enc) {
  if (enc == "kq_Q4_K") return kFmtQ4K;
  if (enc == "kq_Q5_K") return kFmtQ5K;
  if (enc == "kq_Q6_K") return kFmtQ6K;
  if (enc == "kq_IQ4_XS") return kFmtIQ4XS;
  return kFmtNone;
}

}  // namespace lw
