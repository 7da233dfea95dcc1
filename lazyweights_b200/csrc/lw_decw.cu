// Instantiations and launcher of the decode-to-weights kernel; see lw_decw.cuh.
#include "lw_gemv1.h"

#include <cuda.h>

#include <algorithm>

#include "lw_decw.cuh"

namespace lw {

constexpr size_t kSmemLimit = 227 * 1024;
constexpr int kRingSlackWords = 96;

template <int FMT, int G, int IDXBITS, bool TILE_OUT>
static int launch_o(const MatDev& M, __half* out, int tr0, int tr1, unsigned int* err, cudaStream_t st) {
  constexpr int SPLIT = default_split(FMT);
  const uint32_t buf_words = (M.max_unit_words + 31u) & ~31u;
  const int tiles = (tr1 - tr0) * M.KT;
  const int blocks = std::max(1, std::min(sm_count(), tiles));
  const int max_units = (((tiles + blocks - 1) / blocks) * SPLIT + 1) & ~1;
  if (max_units > kGemv1MaxUnits) {   // more tile rows than one block's list holds: two halves
    const int mid = tr0 + (tr1 - tr0) / 2;
    if (mid == tr0) return kErrTooLarge;
    const int rc = launch_o<FMT, G, IDXBITS, TILE_OUT>(M, out, tr0, mid, err, st);
    return rc ? rc : launch_o<FMT, G, IDXBITS, TILE_OUT>(M, out + static_cast<size_t>(mid - tr0) * kTileRows * M.K, mid, tr1, err, st);
  }
  const size_t fixed = (size_t(1) << (M.index_bits + ring_log_copies(M.index_bits) + 2)) + kLutSize * 4 + 2 * kGemv1MaxSlots * 8 +
                       kGemv1MaxSlots * 4 + 16 + max_units * sizeof(UnitMeta) + kRingSlackWords * 4;
  const size_t buf_bytes = static_cast<size_t>(buf_words) * 4;
  if (fixed + buf_bytes > kSmemLimit) return kErrTooLarge;
  // with TILE_OUT every consumer warp also has a 2 KB area for its rows' weights: about three consumers per four buffers
  alignas(64) CUtensorMap tm = {};
  if (TILE_OUT && !make_row_tile_map(&tm, out, static_cast<size_t>(M.K) * 2, static_cast<size_t>(tr1 - tr0) * kTileRows)) return kErrTooLarge;
  const size_t stage = TILE_OUT ? WarpTileStage::kBytes : 0;
  int slots = static_cast<int>(std::min<size_t>(kGemv1MaxSlots, (kSmemLimit - fixed) / (buf_bytes + stage * 3 / 4)));
  const int warps = std::max(1, std::min(std::min(kGemv1MaxWarps, max_units), max_units <= slots ? slots : slots * 3 / 4));
  slots = static_cast<int>(std::min<size_t>(kGemv1MaxSlots, (kSmemLimit - fixed - warps * stage) / buf_bytes));
  if (slots < 1) return kErrTooLarge;
  const size_t smem = fixed + warps * stage + slots * buf_bytes;
  auto kernel = k_decw<FMT, G, IDXBITS, ring_log_copies(IDXBITS), TILE_OUT>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return note_launch("cudaFuncSetAttribute(k_decw)");
  DecwArgs a = {};
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
  kernel<<<blocks, (warps + 2) * 32, smem, st>>>(M, a, tm);
  return note_launch("k_decw");
}

template <int FMT, int G, int IDXBITS>
static int launch_t(const MatDev& M, __half* out, int tr0, int tr1, unsigned int* err, cudaStream_t st) {
  if (tile_output_enabled()) {
    const int rc = launch_o<FMT, G, IDXBITS, true>(M, out, tr0, tr1, err, st);
    if (rc != kErrTooLarge) return rc;
  }
  return launch_o<FMT, G, IDXBITS, false>(M, out, tr0, tr1, err, st);
}

template <int FMT, int G>
static int launch_x(const MatDev& M, __half* out, int tr0, int tr1, unsigned int* err, cudaStream_t st) {
  if (M.index_bits == 10) return launch_t<FMT, G, 10>(M, out, tr0, tr1, err, st);
  return launch_t<FMT, G, 11>(M, out, tr0, tr1, err, st);
}

template <int FMT>
static int launch_bundle_code(const MatDev& M, __half* out, int tr0, int tr1, unsigned int* err, cudaStream_t st);

template <int FMT>
static int launch_i(const MatDev& M, __half* out, int tr0, int tr1, unsigned int* err, cudaStream_t st) {
  if constexpr (is_pair_layout(FMT)) {
    if constexpr (pair_code_bits_max(FMT) == 12)
      if (M.index_bits == 12) return launch_t<FMT, 3, 12>(M, out, tr0, tr1, err, st);
    return launch_t<FMT, 3, 11>(M, out, tr0, tr1, err, st);
  } else {
    return launch_bundle_code<FMT>(M, out, tr0, tr1, err, st);
  }
}

template <int FMT>
static int launch_bundle_code(const MatDev& M, __half* out, int tr0, int tr1, unsigned int* err, cudaStream_t st) {
  switch (M.group) {
    case 3: return launch_x<FMT, 3>(M, out, tr0, tr1, err, st);
    case 4: return launch_x<FMT, 4>(M, out, tr0, tr1, err, st);
  }
  if constexpr (!is_paired(FMT)) {
    switch (M.group) {
      case 5: return launch_x<FMT, 5>(M, out, tr0, tr1, err, st);
      case 6: return launch_x<FMT, 6>(M, out, tr0, tr1, err, st);
    }
  }
  return kErrTooLarge;
}

// Returns kErrTooLarge where this kernel cannot take the product (the caller then uses the warp-per-tile kernel).
int launch_decw(const MatDev& M, __half* out, int tr0, int tr1, unsigned int* err, cudaStream_t st) {
  if (!err || M.KT > 255 || tr1 <= tr0) return kErrTooLarge;
  if (reinterpret_cast<uintptr_t>(out) & 31u) {
    set_kernel_error_text("decode_weights", "the output must be 32-byte aligned");
    return kErrArg;
  }
  switch (M.fmt) {
    case kFmtQ4K: return launch_i<kFmtQ4K>(M, out, tr0, tr1, err, st);
    case kFmtQ5K: return launch_i<kFmtQ5K>(M, out, tr0, tr1, err, st);
    case kFmtIQ4XS: return launch_i<kFmtIQ4XS>(M, out, tr0, tr1, err, st);
    case kFmtQ6K: return launch_i<kFmtQ6K>(M, out, tr0, tr1, err, st);
    case kFmtQ6KP: return launch_i<kFmtQ6KP>(M, out, tr0, tr1, err, st);
    case kFmtQ5KP: return launch_i<kFmtQ5KP>(M, out, tr0, tr1, err, st);
  }
  return kErrTooLarge;
}

}  // namespace lw
