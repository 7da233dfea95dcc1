// Instantiations and launcher of the decode-to-codes kernel on the shared decoder; see lw_decc.cuh.
#include "lw_gemv1.h"

#include <cuda.h>

#include <algorithm>

#include "lw_decc.cuh"

namespace lw {

constexpr size_t kSmemLimit = 227 * 1024;
constexpr int kRingSlackWords = 96;

template <int FMT, int G, int IDXBITS, bool EXPAND, bool TILE_OUT>
static int launch_o(const MatDev& M, uint8_t* out, const CUtensorMap& tm, int tr0, int tr1, unsigned int* err, cudaStream_t st) {
  constexpr int SPLIT = default_split(FMT);
  const uint32_t buf_words = (M.max_unit_words + 31u) & ~31u;
  const int tiles = (tr1 - tr0) * M.KT;
  const int blocks = std::max(1, std::min(sm_count(), tiles));
  const int max_units = (((tiles + blocks - 1) / blocks) * SPLIT + 1) & ~1;
  if (max_units > kRingMaxUnits) {   // more tile rows than one block's list holds: two halves
    const int mid = tr0 + (tr1 - tr0) / 2;
    if (mid == tr0) return kErrTooLarge;
    const int rc = launch_o<FMT, G, IDXBITS, EXPAND, TILE_OUT>(M, out, tm, tr0, mid, err, st);
    return rc ? rc : launch_o<FMT, G, IDXBITS, EXPAND, TILE_OUT>(M, out, tm, mid, tr1, err, st);
  }
  const size_t fixed = (size_t(1) << (M.index_bits + ring_log_copies(M.index_bits) + 2)) + kLutSize * 4 + ring_fixed_bytes(max_units) + kRingSlackWords * 4;
  const size_t buf_bytes = static_cast<size_t>(buf_words) * 4;
  if (fixed + buf_bytes > kSmemLimit) return kErrTooLarge;
  // with TILE_OUT every consumer warp also has a 2 KB area for its rows' bytes: about three consumers per four buffers
  const size_t stage = TILE_OUT ? WarpTileStage::kBytes : 0;
  int slots = static_cast<int>(std::min<size_t>(kRingMaxSlots, (kSmemLimit - fixed) / (buf_bytes + stage * 3 / 4)));
  const int warps = std::max(1, std::min(std::min(kRingMaxWarps, max_units), max_units <= slots ? slots : slots * 3 / 4));
  slots = static_cast<int>(std::min<size_t>(kRingMaxSlots, (kSmemLimit - fixed - warps * stage) / buf_bytes));
  if (slots < 1) return kErrTooLarge;
  const size_t smem = fixed + warps * stage + slots * buf_bytes;
  auto kernel = k_decode_codes_ring<FMT, G, IDXBITS, ring_log_copies(IDXBITS), EXPAND, TILE_OUT>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return note_launch("cudaFuncSetAttribute(k_decode_codes_ring)");
  DeccArgs a = {};
  a.r.err = err;
  a.r.wait_limit = debug_knobs().wait_limit;
  a.r.drop_unit = -1;
  a.r.warps = warps;
  a.r.producers = 2;
  a.r.producer_lanes = 4;
  a.r.slots = slots;
  a.r.buf_words = buf_words;
  a.r.nsets = 1;
  a.r.cols_per_set = M.KT;
  a.r.max_units = max_units;
  a.r.tr0 = tr0;
  a.r.ntr = tr1 - tr0;
  a.out = out;
  a.row_bytes = EXPAND ? 2 * M.Ks : M.Ks;
  kernel<<<blocks, (warps + 2) * 32, smem, st>>>(M, a, tm);
  return note_launch("k_decode_codes_ring");
}

template <int FMT, int G, int IDXBITS, bool EXPAND>
static int launch_t(const MatDev& M, uint8_t* out, int tr0, int tr1, unsigned int* err, cudaStream_t st) {
  alignas(64) CUtensorMap tm = {};
  if (tile_output_enabled() && make_row_tile_map(&tm, out, EXPAND ? 2 * static_cast<size_t>(M.Ks) : M.Ks, M.N)) {
    const int rc = launch_o<FMT, G, IDXBITS, EXPAND, true>(M, out, tm, tr0, tr1, err, st);
    if (rc != kErrTooLarge) return rc;
  }
  return launch_o<FMT, G, IDXBITS, EXPAND, false>(M, out, tm, tr0, tr1, err, st);
}

template <int FMT>
static int launch_bundle_code(const MatDev& M, uint8_t* out, bool expand, unsigned int* err, cudaStream_t st);

template <int FMT, int G, int IDXBITS>
static int launch_e(const MatDev& M, uint8_t* out, bool expand, unsigned int* err, cudaStream_t st) {
  const int NT = M.N / kTileRows;
  if constexpr (is_paired(FMT)) {
    if (expand) return launch_t<FMT, G, IDXBITS, true>(M, out, 0, NT, err, st);
  }
  return launch_t<FMT, G, IDXBITS, false>(M, out, 0, NT, err, st);
}

template <int FMT, int G>
static int launch_x(const MatDev& M, uint8_t* out, bool expand, unsigned int* err, cudaStream_t st) {
  if (M.index_bits == 10) return launch_e<FMT, G, 10>(M, out, expand, err, st);
  return launch_e<FMT, G, 11>(M, out, expand, err, st);
}

template <int FMT>
static int launch_i(const MatDev& M, uint8_t* out, bool expand, unsigned int* err, cudaStream_t st) {
  if constexpr (is_pair_layout(FMT)) {
    const int NT = M.N / kTileRows;
    if constexpr (pair_code_bits_max(FMT) == 12)
      if (M.index_bits == 12) return launch_t<FMT, 3, 12, true>(M, out, 0, NT, err, st);
    return launch_t<FMT, 3, 11, true>(M, out, 0, NT, err, st);
  } else {
    return launch_bundle_code<FMT>(M, out, expand, err, st);
  }
}

template <int FMT>
static int launch_bundle_code(const MatDev& M, uint8_t* out, bool expand, unsigned int* err, cudaStream_t st) {
  switch (M.group) {
    case 3: return launch_x<FMT, 3>(M, out, expand, err, st);
    case 4: return launch_x<FMT, 4>(M, out, expand, err, st);
  }
  if constexpr (!is_paired(FMT)) {
    switch (M.group) {
      case 5: return launch_x<FMT, 5>(M, out, expand, err, st);
      case 6: return launch_x<FMT, 6>(M, out, expand, err, st);
    }
  }
  return kErrTooLarge;
}

// Returns kErrTooLarge where this kernel cannot take the matrix (the caller then uses the warp-per-tile kernel).
int launch_decode_codes_ring(const MatDev& M, uint8_t* out, bool expand, unsigned int* err, cudaStream_t st) {
  if (!err || (!M.symtab32 && !is_pair_layout(M.fmt)) || !gemv1_usable(M) || M.reader != 0 || M.KT > 255) return kErrTooLarge;
  switch (M.fmt) {
    case kFmtQ4K: return launch_i<kFmtQ4K>(M, out, expand, err, st);
    case kFmtQ5K: return launch_i<kFmtQ5K>(M, out, expand, err, st);
    case kFmtIQ4XS: return launch_i<kFmtIQ4XS>(M, out, expand, err, st);
    case kFmtQ6K: return launch_i<kFmtQ6K>(M, out, expand, err, st);
    case kFmtQ6KP: return launch_i<kFmtQ6KP>(M, out, expand, err, st);   // always one code per byte
    case kFmtQ5KP: return launch_i<kFmtQ5KP>(M, out, expand, err, st);
  }
  return kErrTooLarge;
}

}  // namespace lw
