// Shared definitions of the coded-weight library: formats, the Huffman table, the host-side view of a blob and
// the device layout of a matrix.  Host and device code both include this file.
//
// On-disk blob (reference: lazyweights/bundle.py:16-21), little-endian:
//   uint16 lut[2048]          index = next 11 stream bits, LSB first -> symbol | length << 8
//   uint32 lane_start[T][32]  absolute bit offset of lane l of tile t; T = (N / 64) * (Ks / 256)
//   uint32 payload[W + 2]     bit b = (payload[b >> 5] >> (b & 31)) & 1
// A tile is 64 rows x 256 symbols; lane l carries tile row l and then tile row l + 32, 256 symbols each.
//
// Device layout (built once at load, lw::relayout): every lane is cut into "chains" of 256 / SPLIT symbols
// (its two rows, each optionally cut into SPLIT column segments).  The 32 chains that cover the same rows half
// and the same column segment form a group; each chain of a group is re-based (it starts with `pad` zero bits, then
// its code bits) and the group's words are interleaved: word i of chain c (= lane) sits at group_base + 32 i + c, so
// one warp reads its 32 next words as one 128-byte line.  A group is padded to its longest chain.  Groups of a tile
// are stored segment-major: group 2 s + h holds rows half h (rows 32 h .. 32 h + 31) over column segment s.
#pragma once
#include <cstddef>
#include <cstdint>

namespace lw {

constexpr int kTileRows = 64;
constexpr int kTileSyms = 256;
constexpr int kMaxLen = 11;
constexpr int kLanes = 32;
constexpr int kLutSize = 1 << kMaxLen;
constexpr int kBlobAlign = 256;
constexpr int kTailWords = 512;   // zero words after the last group: read-ahead of the last chains lands here

// Block formats of the side bytes (reference: kernels/llmrt.cu:113-121, scripts/a2_kq_bundle.py:41-42).
// kFmtQ6KP / kFmtQ5KP are not bundle formats: they name the pair layouts that the loader builds for Q6_K / Q5_K matrices
// (lw::build_pairs: two adjacent codes become one symbol of a code of its own, so that the one-row kernel does one
// table lookup per two weights, as it does for the formats whose symbols are pairs already).  Geometry as Q4_K: tiles of
// 64 rows x 256 symbols = 512 weights.
enum Format : int { kFmtNone = 0, kFmtQ4K = 1, kFmtQ5K = 2, kFmtQ6K = 3, kFmtIQ4XS = 4, kFmtQ6KP = 5, kFmtQ5KP = 6 };

constexpr int side_bytes(int f) { return f == kFmtQ6K ? 18 : f == kFmtIQ4XS ? 8 : 16; }
constexpr int sub_width(int f) { return (f == kFmtQ6K || f == kFmtQ6KP) ? 16 : 32; }
constexpr bool is_paired(int f) { return f == kFmtQ4K || f == kFmtIQ4XS || f == kFmtQ6KP || f == kFmtQ5KP; }
constexpr bool is_pair_layout(int f) { return f == kFmtQ6KP || f == kFmtQ5KP; }
constexpr int pair_layout_of(int f) { return f == kFmtQ6K ? kFmtQ6KP : f == kFmtQ5K ? kFmtQ5KP : kFmtNone; }
// Longest code a pair layout's own code may have = index bits of its table: 1024 pairs of 5-bit codes fit 11 bits; the
// 4096 pairs of 6-bit codes need 12, but a matrix in which at most 2048 different pairs occur gets an 11-bit code where
// that costs at most a fifth more code bits (the 2048-window table has twice the copies for the same shared memory: fewer
// bank conflicts per lookup).
constexpr int pair_code_bits_max(int f) { return f == kFmtQ6KP ? 12 : 11; }
// Column segments per tile row of the device layout: more segments = shorter chains = more of them in flight for the
// same staging memory; a segment must hold whole quads of sub-blocks (four 32-weight sub-blocks of Q5_K = 128 symbols).
constexpr int default_split(int f) { return f == kFmtNone ? 1 : f == kFmtQ5K ? 2 : 4; }
// Scales of one work unit of the batch-1 kernel (64 rows r = 0..63 x one quad of four sub-blocks), stored behind the
// unit's chain words as arrays over the rows:
//   Q6_K    word[r] = the four int8 scales;                      half[2 * 64 + r] = fp16 d
//   IQ4_XS  word[r] = the four 6-bit scales (one per byte);      half[2 * 64 + r] = fp16 d
//   Q4_K / Q5_K  word[r] = fp16 d | fp16 dmin << 16; word[64 + r] = the four 6-bit scales; word[128 + r] = the mins
//   Q6KP    word[r], word[64 + r] = the eight int8 scales of the unit's 128 weights; half[4 * 64 + r] = fp16 d
//   Q5KP    as Q5_K
constexpr int unit_side_words(int f) {
  return f == kFmtNone ? 0 : f == kFmtQ6KP ? 160 : (f == kFmtQ6K || f == kFmtIQ4XS) ? 96 : 192;
}
// Symbols per sub-block (one scale), and per quad of sub-blocks
constexpr int sub_syms(int f) { return is_paired(f) ? sub_width(f) / 2 : sub_width(f); }

// Status codes of the C ABI (0 = success; the reference's -1 / nullptr conventions are kept where it has them).
enum Status : int {
  kOk = 0,
  kErrGeneric = -1,     // not found / not resident (the reference's -1)
  kErrArg = -2,
  kErrFormat = -3,      // malformed bundle or blob
  kErrCuda = -4,
  kErrTooLarge = -5,
  kErrNoDevice = -6,
};

struct HuffTable {
  uint16_t lut[kLutSize];     // as stored in the blob
  uint8_t len[256];           // code length per symbol (0 = unused)
  int nsym = 0;               // symbols in use
  int max_len = 0;
  // canonical comparator form (reference: hw/huff/huff_engine.h:39-52): codes of length l are the MSB-first values
  // first[l] .. first[l] + count[l] - 1; limit[l] = (first[l] + count[l]) << (11 - l); sorted[] lists symbols by
  // (length, symbol); base[l] = index in sorted[] of the first symbol of length l.
  uint32_t limit[kMaxLen + 1];
  uint32_t first[kMaxLen + 1];
  uint32_t base[kMaxLen + 1];
  uint8_t sorted[256];
};

struct BlobView {
  const uint8_t* data = nullptr;
  size_t nbytes = 0;
  int N = 0, Ks = 0;          // rows, symbols per row
  int KT = 0, T = 0;          // tile columns, tiles
  const uint16_t* lut() const { return reinterpret_cast<const uint16_t*>(data); }
  const uint32_t* lane_start() const { return reinterpret_cast<const uint32_t*>(data + 2 * kLutSize); }
  const uint32_t* payload() const { return lane_start() + static_cast<size_t>(T) * kLanes; }
  size_t payload_words() const { return (nbytes - 2 * kLutSize - static_cast<size_t>(T) * kLanes * 4) / 4; }
};

// Device layout of one coded matrix, as host-side arrays ready for upload.
struct DeviceImage {
  int split = 1;                        // chains per row
  int groups_per_tile = 2;              // 2 * split
  std::size_t n_words = 0;              // length of words (incl. tail)
  uint32_t* group_base = nullptr;       // [T * groups_per_tile + 1] word offset of each group (multiple of 32)
  uint32_t* words = nullptr;            // interleaved chain words
  uint32_t max_group_words = 0;         // longest group, in words per chain
  uint32_t max_tile_words = 0;          // largest tile, in words (all groups, all chains)
};

}  // namespace lw
