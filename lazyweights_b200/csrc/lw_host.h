// Host-side (CPU, no CUDA) part of the library: Huffman tables, the blob encoder, blob validation and indexing,
// the load-time re-layout into the device image, the threaded CPU decoder and the bundle directory reader/writer.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "lw_core.h"

namespace lw {

// Thread-local text of the last failure, returned by lw_last_error().
void set_error(const char* fmt, ...);
const char* last_error();
// Status of the last call that could only report failure as NULL (handle constructors).
int note_status(int rc);
int last_status();

// ---- tables (reference: lazyweights/huffman.py:8-26, lazyweights/lanecodecs.py:28-62, lazyweights/bundle.py:46-54)
void huffman_depths(const int64_t counts[256], int depth[256]);
// limit: the longest code allowed (the bundle format's own is kMaxLen = 11; any limit >= 8 fits 256 symbols)
void limited_lengths(const int64_t counts[256], uint8_t len[256], int limit = kMaxLen);
void table_from_lengths(const uint8_t len[256], HuffTable& t);
// Recovers lengths from a stored table and checks that the table is exactly the canonical one for those lengths.
int table_from_lut(const uint16_t* lut, HuffTable& t);
void fat_table(const HuffTable& t, int fmt, uint32_t out[kLutSize]);
// Comparator form for the limit-register decoder (reference: hw/huff/huff_engine.h:39-77, hw/huff/rtl/huff_lane.sv:86-93):
// with v = the 11 window bits reversed (MSB first), len = 1 + #{l in 1..10 : v >= limit[l]} and the symbol is
// sorted[(v >> (11 - len)) + off[len]].  out[0..11] = limit[l] (2048 where no longer code exists), out[12..23] = off[l]
// = base[l] - first[l] (two's complement), out[24..279] = grid value bytes of sorted[i] as in fat_table (no length).
constexpr int kCmpTabWords = 24 + 256;
void comparator_table(const HuffTable& t, int fmt, uint32_t out[kCmpTabWords]);
// Grid value bytes of every 8-bit symbol (the table of a fixed-width twin of a paired format), as in fat_table.
void symbol_values(int fmt, uint32_t out[256]);

// Fixed-width twin of a coded matrix (the role of interleave_packed / interleave_packed_q, kernels/llmrt.cu:1733-1777):
// the decoded symbols packed at a fixed width (8 bits per paired symbol, 5 for Q5_K, 6 for Q6_K stored minus 32 in
// two's complement) into the same unit structure as relayout() builds - chains of 256 / split symbols, 32 chains
// interleaved word by word per group, the unit's scales behind its second group - so that the same kernel body can read
// it without any Huffman decoding.  sym = decoded symbols [N, Ks].
int twin_bits(int fmt);
int build_twin(const uint8_t* sym, int N, int Ks, int fmt, const uint8_t* side, int threads,
               std::vector<uint32_t>& group_base, std::vector<uint32_t>& words, uint32_t* unit_words);

// ---- blob (reference: lazyweights/bundle.py:57-106, kernels/llmrt.cu:2513-2541)
// limit / threads: the code's longest word (kMaxLen = the bundle format's own rule, whose blobs are byte-identical to the
// reference encoder's) and the threads that pack tile ranges side by side (the result does not depend on them).
int encode_huf8(const uint8_t* sym, int N, int Ks, std::vector<uint8_t>& blob, int64_t* nbits, int limit = kMaxLen, int threads = 1);
int make_view(const uint8_t* blob, size_t nbytes, int N, int Ks, BlobView& v);

// Walks every lane once.  chain_start[(t * 32 + l) * (2 * split) + g] = absolute bit offset at which chain g of the
// lane starts; lane_end[t * 32 + l] = bit offset after its 512th symbol.  Checks that every window resolves, that
// each lane ends where the next begins and that the last one ends inside the payload.  If `out` is not null the
// decoded symbols are written to it as [N, Ks].
// If `scan` is not null it also receives, per work unit of the batch-1 kernel, which symbol-group sizes its grouped
// decoder may use.
struct GroupScan {
  int quad_syms = 64;          // in: symbols of a chain after which the group phase restarts (four sub-blocks)
  std::vector<uint8_t> mask;   // out: [T * split] per (tile, column segment): bit (g - kScanMinG) set = groups of g
                               // symbols are unsafe there; bit 7 = the unit holds a code longer than 10 bits
};
constexpr int kScanMinG = 3, kScanMaxG = 6;
int walk_blob(const BlobView& v, const HuffTable& tab, int split, int threads, std::vector<uint32_t>* chain_start,
              std::vector<uint32_t>* lane_end, uint8_t* out, GroupScan* scan = nullptr);

// Re-layout into interleaved chain groups (the role of interleave_huf8, kernels/llmrt.cu:1208-1257).
// Every chain starts with `pad` zero bits (the fused kernels fold the table's entry size into the shift).
// If `side` is not null (block format `fmt`, [N, K / 256 * side_bytes]) every work unit - the two groups of one
// column segment - is followed by unit_side_words(fmt) words with the scales of its 64 rows x 4 sub-blocks, so that
// the unit's one bulk copy brings everything its decoding needs (layout: unit_side_words below).
int relayout(const BlobView& v, int split, int pad, const std::vector<uint32_t>& chain_start,
             const std::vector<uint32_t>& lane_end, int threads, std::vector<uint32_t>& group_base,
             std::vector<uint32_t>& words, uint32_t* max_unit_words, uint32_t* max_tile_words, int fmt = kFmtNone,
             const uint8_t* side = nullptr);

// Scales of four consecutive sub-blocks sub0 .. sub0 + 3 of one row (sub-blocks counted along the row; all four inside
// one 256-weight super-block): sc / mn one value per byte, dd = fp16 d (low half) and fp16 dmin.
void unit_scales_at(int fmt, const uint8_t* side_row, int sub0, uint32_t* sc, uint32_t* mn, uint32_t* dd);

// ---- pair layout (lw_pairs.cpp)
// A second device layout for Q6_K / Q5_K matrices, read by the one-row product only: two adjacent codes of a row become
// one symbol, the pairs get a length-limited prefix code of their own (12 bits for pairs of 6-bit codes, 11 for pairs of
// 5-bit codes; the code is built from the matrix's pair counts like the bundle's code is from its symbol counts), and
// the rows are laid out like a paired format's: tiles of 64 rows x 256 pair symbols, four column segments, chains of
// 64 symbols interleaved by lane, the unit's scales behind its second group.  The kernel then does one table lookup
// and one dp2a per two weights.  The decoded codes are identical by construction; what changes is the entropy code
// that device memory holds (its size is within a per cent of the bundle's: pairs cost no more bits than two singles).
struct PairImage {
  int fmt = kFmtNone;                  // kFmtQ6KP or kFmtQ5KP
  int index_bits = 0, group = 3, split = 4, pad = 6, KT = 0, T = 0, max_len = 0;
  std::vector<uint32_t> tab32;         // [1 << index_bits] length << 28 | value of the second weight << 8 | of the first
  std::vector<uint32_t> group_base;    // [T * 8 + 1]
  std::vector<uint32_t> words;         // interleaved chain words + unit scales (+ zero tail)
  std::vector<uint8_t> unit_class;     // [T * 4], all 0: groups of three are exact for codes of at most 12 bits
  uint32_t max_unit_words = 0, max_tile_words = 0;
  long long code_bits = 0;             // bits of all pair codes (without padding)
};
// sym = decoded codes [N, K] (one per weight), fmt = kFmtQ6K or kFmtQ5K, side = the matrix's side bytes.
// K must be a multiple of 512 and N of 64.
int build_pairs(const uint8_t* sym, int N, int K, int fmt, const uint8_t* side, int threads, PairImage& out);

// ---- bundle directory (reference: lazyweights/bundle.py:114-148)
struct TensorEntry {
  std::string name, enc;
  int N = 0, K = 0;
  double scale = 1.0;
  long long zp = 0;
  long long offset = 0, nbytes = 0;
};

struct Manifest {
  std::map<std::string, std::string> cfg;
  std::vector<TensorEntry> tensors;
  std::map<std::string, int> by_name;
  const TensorEntry* find(const std::string& n) const {
    auto it = by_name.find(n);
    return it == by_name.end() ? nullptr : &tensors[it->second];
  }
};

int read_manifest(const std::string& dir, Manifest& m);
int read_blob(int fd, const TensorEntry& t, std::vector<uint8_t>& out);
// A bundle with a model configuration: every tensor the decoder runtime reads has the shape the cfg implies.
int validate_model(const Manifest& m);
// ---- llama.cpp blocks (reference: scripts/kq_code.py:37-81): [nblk][block_bytes] <-> codes [nblk][256] in weight order
// + side bytes [nblk][side_bytes]
int block_bytes(int fmt);
int split_blocks(int fmt, const uint8_t* blocks, long long nblk, uint8_t* q, uint8_t* side);
int join_blocks(int fmt, const uint8_t* q, const uint8_t* side, long long nblk, uint8_t* blocks);

int format_of_side_enc(const std::string& enc);   // "kq_Q4_K" -> kFmtQ4K, ... ; 0 if unknown
int default_threads();

}  // namespace lw
