// Pair layout of Q6_K / Q5_K matrices (host side; see lw_host.h).  The reference codes these formats one symbol per
// weight (scripts/a2_kq_bundle.py:104-115) and its kernel does one table lookup per weight (kernels/llmrt.cu:972-1024);
// the formats whose symbols are pairs of 4-bit codes get two weights per lookup.  This file gives the unpaired formats
// the same: at load, the decoded codes are re-coded two at a time with a prefix code built from the matrix's own pair
// counts, and laid out in the unit structure of lw::relayout.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <queue>
#include <thread>

#include "lw_host.h"

namespace lw {

namespace {

template <class F>
void for_each_index(int n, int threads, F&& body) {
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

// Huffman code lengths of the symbols with a non-zero count (0 for the others).
void huffman_lengths(const std::vector<int64_t>& counts, std::vector<uint8_t>& len) {
  const int n = static_cast<int>(counts.size());
  len.assign(n, 0);
  struct Node {
    int64_t c;
    int id;
  };
  auto later = [](const Node& a, const Node& b) { return a.c != b.c ? a.c > b.c : a.id > b.id; };
  std::priority_queue<Node, std::vector<Node>, decltype(later)> heap(later);
  std::vector<int> parent;
  parent.reserve(2 * n);
  std::vector<int> leaf_node(n, -1);
  for (int s = 0; s < n; ++s)
    if (counts[s] > 0) {
      leaf_node[s] = static_cast<int>(parent.size());
      heap.push(Node{counts[s], static_cast<int>(parent.size())});
      parent.push_back(-1);
    }
  if (heap.size() == 1) {   // a single symbol still needs one bit
    for (int s = 0; s < n; ++s)
      if (leaf_node[s] >= 0) len[s] = 1;
    return;
  }
  while (heap.size() > 1) {
    const Node a = heap.top();
    heap.pop();
    const Node b = heap.top();
    heap.pop();
    const int id = static_cast<int>(parent.size());
    parent.push_back(-1);
    parent[a.id] = id;
    parent[b.id] = id;
    heap.push(Node{a.c + b.c, id});
  }
  for (int s = 0; s < n; ++s) {
    if (leaf_node[s] < 0) continue;
    int d = 0;
    for (int v = leaf_node[s]; parent[v] >= 0; v = parent[v]) ++d;
    len[s] = static_cast<uint8_t>(std::min(d, 255));
  }
}

// Lengths limited to `limit` bits by the rule the bundle's own code uses (lazyweights/huffman.py: the counts are
// halved, rounding up, and the tree rebuilt until the deepest leaf fits).  Needs at most 2^limit symbols in use.
void limited_lengths_n(std::vector<int64_t> counts, int limit, std::vector<uint8_t>& len) {
  for (;;) {
    huffman_lengths(counts, len);
    int deepest = 0;
    for (uint8_t l : len) deepest = std::max<int>(deepest, l);
    if (deepest <= limit) return;
    for (auto& c : counts)
      if (c > 0) c = (c + 1) / 2;
  }
}

uint32_t reverse_low_bits(uint32_t v, int n) {
  uint32_t r = 0;
  for (int i = 0; i < n; ++i) r |= ((v >> i) & 1u) << (n - 1 - i);
  return r;
}

}  // namespace

int build_pairs(const uint8_t* sym, int N, int K, int fmt, const uint8_t* side, int threads, PairImage& out) {
  if ((fmt != kFmtQ6K && fmt != kFmtQ5K) || !sym || !side || N < kTileRows || N % kTileRows || K < 512 || K % 512) {
    set_error("build_pairs: Q6_K or Q5_K codes [N, K] with N a multiple of 64 and K a multiple of 512");
    return kErrArg;
  }
  const int B = fmt == kFmtQ6K ? 6 : 5, A = 1 << B, NP = A * A;
  const int pf = pair_layout_of(fmt);
  int L = pair_code_bits_max(pf);
  const int Ks = K / 2, KT = Ks / kTileSyms, NT = N / kTileRows, T = NT * KT;
  const int split = default_split(pf), G = 2 * split, seg_syms = kTileSyms / split;
  const uint32_t side_words = unit_side_words(pf);
  out = PairImage();
  out.fmt = pf;
  out.max_len = 0;
  out.KT = KT;
  out.T = T;
  out.split = split;

  // 1. pair counts (per thread, then added)
  threads = std::max(1, threads);
  std::vector<std::vector<int64_t>> part(threads, std::vector<int64_t>(NP, 0));
  {
    std::atomic<int> next(0);
    std::vector<std::thread> pool;
    for (int w = 0; w < threads; ++w)
      pool.emplace_back([&, w] {
        std::vector<int64_t>& h = part[w];
        for (int r; (r = next.fetch_add(1)) < N;) {
          const uint8_t* row = sym + static_cast<size_t>(r) * K;
          for (int i = 0; i < K; i += 2) {
            if (row[i] >= A || row[i + 1] >= A) {
              h[0] = -1;   // a code outside the format: reported below
              return;
            }
            ++h[row[i] | (row[i + 1] << B)];
          }
        }
      });
    for (auto& t : pool) t.join();
  }
  std::vector<int64_t> counts(NP, 0);
  for (auto& h : part) {
    if (h[0] < 0) {
      set_error("build_pairs: a code does not fit the format");
      return kErrFormat;
    }
    for (int p = 0; p < NP; ++p) counts[p] += h[p];
  }

  // 2. the pair code: limited lengths, canonical codes (shorter first, then by symbol), stream order LSB first
  std::vector<uint8_t> len;
  limited_lengths_n(counts, L, len);
  if (L == 12) {
    // 11 bits where no more than 2048 pairs occur and the shorter limit costs at most `slack` per cent of code bits
    // (LW_PAIR_SLACK, default 20): the 2048-window table has 8 copies instead of 4 in the same shared memory, a
    // lookup costs 2.6 instead of 3.8 shared-memory wavefronts and products run 10 % faster (the kernel is bound by
    // shared memory, not by DRAM: measured with 16 % more code bits, 18.3 instead of 20.1 us).
    static const int slack = [] {
      const char* e = getenv("LW_PAIR_SLACK");
      return e ? std::max(0, std::min(100, atoi(e))) : 20;
    }();
    size_t used = 0;
    for (int64_t c : counts) used += c > 0;
    if (used <= 2048) {
      std::vector<uint8_t> len11;
      limited_lengths_n(counts, 11, len11);
      int64_t bits12 = 0, bits11 = 0;
      for (int p = 0; p < NP; ++p) {
        bits12 += counts[p] * len[p];
        bits11 += counts[p] * len11[p];
      }
      if (bits11 * 100 <= bits12 * (100 + slack)) {
        len.swap(len11);
        L = 11;
      }
    }
  }
  out.index_bits = L;
  // an 11-bit code is laid out without pad bits (its reader loads two words per group: lw_ring.cuh), a 12-bit code
  // with the six the table's address bits want
  const int pad = L == 11 ? 0 : 6;
  out.pad = pad;
  std::vector<int> order;
  for (int p = 0; p < NP; ++p)
    if (len[p]) order.push_back(p);
  std::sort(order.begin(), order.end(), [&](int a, int b) { return len[a] != len[b] ? len[a] < len[b] : a < b; });
  std::vector<uint32_t> code(NP, 0);   // bit-reversed: first stream bit = bit 0
  out.tab32.assign(size_t(1) << L, 0);
  uint32_t next_code = 0;
  int prev_len = 0;
  for (int p : order) {
    next_code <<= (len[p] - prev_len);
    prev_len = len[p];
    if (next_code >> len[p]) {
      set_error("build_pairs: code lengths violate the Kraft inequality");
      return kErrGeneric;
    }
    code[p] = reverse_low_bits(next_code, len[p]);
    ++next_code;
    out.max_len = std::max<int>(out.max_len, len[p]);
    const int c0 = p & (A - 1), c1 = p >> B;
    const int v0 = fmt == kFmtQ6K ? c0 - 32 : c0, v1 = fmt == kFmtQ6K ? c1 - 32 : c1;
    const uint32_t entry = (static_cast<uint32_t>(len[p]) << 28) | ((static_cast<uint32_t>(v1) & 255u) << 8) | (static_cast<uint32_t>(v0) & 255u);
    for (uint32_t f = 0; f < (1u << (L - len[p])); ++f) out.tab32[code[p] | (f << len[p])] = entry;
    out.code_bits += counts[p] * len[p];
  }

  // 3. words per chain group (its longest chain), bases
  std::vector<uint32_t> gw(static_cast<size_t>(T) * G, 0);
  for_each_index(T, threads, [&](int t) {
    const int tr = t / KT, tc = t % KT;
    for (int g = 0; g < G; ++g) {
      const int seg = g >> 1, half = g & 1;
      uint32_t w = 0;
      for (int lane = 0; lane < kLanes; ++lane) {
        const uint8_t* row = sym + (static_cast<size_t>(tr) * kTileRows + half * 32 + lane) * K + (static_cast<size_t>(tc) * kTileSyms + seg * seg_syms) * 2;
        uint32_t bits = pad;
        for (int c = 0; c < seg_syms; ++c) bits += len[row[2 * c] | (row[2 * c + 1] << B)];
        w = std::max(w, (bits + 31) / 32);
      }
      gw[static_cast<size_t>(t) * G + g] = w;
    }
  });
  out.group_base.assign(static_cast<size_t>(T) * G + 1, 0);
  uint64_t total = 0;
  for (int t = 0; t < T; ++t) {
    uint32_t tile_words = 0;
    for (int g = 0; g < G; ++g) {
      if (total > 0xFFFFFFFFull) break;
      out.group_base[static_cast<size_t>(t) * G + g] = static_cast<uint32_t>(total);
      const uint32_t w = gw[static_cast<size_t>(t) * G + g] * kLanes + ((g & 1) ? side_words : 0);
      total += w;
      tile_words += w;
      if (g & 1)
        out.max_unit_words = std::max(out.max_unit_words,
                                      (gw[static_cast<size_t>(t) * G + g - 1] + gw[static_cast<size_t>(t) * G + g]) * kLanes + side_words);
    }
    out.max_tile_words = std::max(out.max_tile_words, tile_words);
  }
  if (total > 0xFFFFFFFFull) {
    set_error("pair layout needs more than 2^32 device words");
    return kErrTooLarge;
  }
  out.group_base[static_cast<size_t>(T) * G] = static_cast<uint32_t>(total);
  out.words.assign(total + kTailWords, 0);
  out.unit_class.assign(static_cast<size_t>(T) * split, 0);

  // 4. the chains and the units' scales
  const size_t side_row_bytes = static_cast<size_t>(K) / 256 * side_bytes(fmt);
  for_each_index(T, threads, [&](int t) {
    const int tr = t / KT, tc = t % KT;
    for (int g = 0; g < G; ++g) {
      const int seg = g >> 1, half = g & 1;
      uint32_t* dst = out.words.data() + out.group_base[static_cast<size_t>(t) * G + g];
      for (int lane = 0; lane < kLanes; ++lane) {
        const uint8_t* row = sym + (static_cast<size_t>(tr) * kTileRows + half * 32 + lane) * K + (static_cast<size_t>(tc) * kTileSyms + seg * seg_syms) * 2;
        uint64_t acc = 0;
        int fill = pad;   // the chain starts with `pad` zero bits
        uint32_t wi = 0;
        for (int c = 0; c < seg_syms; ++c) {
          const int p = row[2 * c] | (row[2 * c + 1] << B);
          acc |= static_cast<uint64_t>(code[p]) << fill;
          fill += len[p];
          if (fill >= 32) {
            dst[static_cast<size_t>(wi++) * kLanes + lane] = static_cast<uint32_t>(acc);
            acc >>= 32;
            fill -= 32;
          }
        }
        if (fill > 0) dst[static_cast<size_t>(wi) * kLanes + lane] = static_cast<uint32_t>(acc);
      }
      if (g & 1) {
        uint32_t* sd = dst + static_cast<size_t>(gw[static_cast<size_t>(t) * G + g]) * kLanes;
        uint16_t* sh = reinterpret_cast<uint16_t*>(sd);
        const int sub0 = (tc * kTileSyms + seg * seg_syms) * 2 / sub_width(fmt);
        for (int r = 0; r < kTileRows; ++r) {
          const uint8_t* side_row = side + (static_cast<size_t>(tr) * kTileRows + r) * side_row_bytes;
          uint32_t sc, mn, dd;
          unit_scales_at(fmt, side_row, sub0, &sc, &mn, &dd);
          if (fmt == kFmtQ5K) {
            sd[r] = dd;
            sd[64 + r] = sc;
            sd[128 + r] = mn;
          } else {   // eight sub-blocks of 16 weights per unit
            uint32_t sc2, mn2, dd2;
            unit_scales_at(fmt, side_row, sub0 + 4, &sc2, &mn2, &dd2);
            sd[r] = sc;
            sd[64 + r] = sc2;
            sh[256 + r] = static_cast<uint16_t>(dd);
          }
        }
      }
    }
  });
  return kOk;
}

}  // namespace lw
