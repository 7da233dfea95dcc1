// Instantiations and launcher of the tcgen05 small-M GEMM on coded weights; see lw_gemm_t5.cuh.
#include "lw_gemv1.h"

#include <algorithm>

#include "lw_gemm_t5.cuh"

namespace lw {

constexpr size_t kSmemLimit = 227 * 1024;
constexpr int kRingSlackWords = 96;
// 8 copies of the decode table: 32 KB (1024 windows) or 64 KB (2048); 4 copies of a pair layout's 4096 windows
constexpr int t5_log_copies(int index_bits) { return index_bits == 12 ? 2 : 3; }
constexpr int kT5MinSlots = 17;   // sixteen consumer warps hold a unit each; the rest is run-ahead of the copies

struct T5Plan {
  int nsets, blocks, max_units, slots, ntok;
  uint32_t buf_words;
  size_t smem;
};

template <int FMT>
static bool plan_t5(const MatDev& M, int m, T5Plan& p) {
  constexpr int TW = is_paired(FMT) ? 512 : 256, SPLIT = default_split(FMT), TU = kT5SetK / TW * SPLIT;
  const int NT = M.N / kTileRows;
  if (m < 1 || m > kT5MaxTokens || NT % 4 || M.K % kT5SetK || !gemv1_usable(M) || M.reader != 0) {
    set_kernel_error_text("gemm (tcgen05)", "needs 1..64 rows, tile rows in fours and K in 512s");
    return false;
  }
  p.ntok = (m + 15) / 16 * 16;
  p.nsets = M.K / kT5SetK;
  const int NRG = NT / 4;
  p.blocks = std::max(p.nsets, std::min(sm_count(), p.nsets * NRG));
  const int nb_min = p.blocks / p.nsets;                           // the smallest number of blocks a column set gets
  p.max_units = ((NRG + nb_min - 1) / nb_min) * TU * 4;
  if (p.max_units > kRingMaxUnits) {
    set_kernel_error_text("gemm (tcgen05)", "too many units per block");
    return false;
  }
  p.buf_words = (M.max_unit_words + 31u) & ~31u;
  const size_t fixed = (size_t(1) << (M.index_bits + t5_log_copies(M.index_bits) + 2)) + (M.index_bits < kMaxLen ? kLutSize * 4 : 0) +
                       static_cast<size_t>(p.ntok) * kT5SetK * 2 +
                       (2 * kT5Teams * kT5ASlots + 4) * 8 + 16 + ring_fixed_bytes(p.max_units) + kRingSlackWords * 4;
  if (fixed + static_cast<size_t>(p.buf_words) * 4 * kT5MinSlots > kSmemLimit) {
    set_kernel_error_text("gemm (tcgen05)", "not enough shared memory for the staging ring");
    return false;
  }
  p.slots = static_cast<int>(std::min<size_t>(kRingMaxSlots, (kSmemLimit - fixed) / (p.buf_words * 4)));
  p.smem = fixed + static_cast<size_t>(p.slots) * p.buf_words * 4;
  return true;
}

template <int FMT, int G, int IDXBITS>
static int launch_t(const MatDev& M, const void* X, bool x_is_half, const float* row_scale, int m, float* planes, unsigned int* err, cudaStream_t st,
                    int* terms) {
  T5Plan p;
  if (!plan_t5<FMT>(M, m, p)) return kErrTooLarge;
  auto kernel = k_gemm_t5<FMT, G, IDXBITS, t5_log_copies(IDXBITS)>;
  static size_t configured_per_device[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  size_t& configured = configured_per_device[dev & 63];
  if (p.smem > configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemLimit)) != cudaSuccess)
      return note_launch("cudaFuncSetAttribute(k_gemm_t5)");
    configured = kSmemLimit;
  }
  GemmT5Args a = {};
  a.x = X;
  a.planes = planes;
  a.x_is_half = x_is_half;
  a.row_scale = row_scale;
  a.m = m;
  a.ntok = p.ntok;
  a.r.err = err;
  a.r.wait_limit = debug_knobs().wait_limit;
  a.r.drop_unit = -1;
  a.r.warps = kT5Consumers;
  a.r.producers = kT5Producers;
  a.r.producer_lanes = 4;
  a.r.slots = p.slots;
  a.r.buf_words = p.buf_words;
  a.r.nsets = p.nsets;
  a.r.cols_per_set = kT5SetK / (is_paired(FMT) ? 512 : 256);
  a.r.max_units = p.max_units;
  a.r.tr0 = 0;
  a.r.ntr = M.N / kTileRows;
  kernel<<<p.blocks, kT5Threads, p.smem, st>>>(M, a);
  *terms = p.nsets;
  return note_launch("k_gemm_t5");
}

template <int FMT>
static int launch_bundle_code(const MatDev& M, const void* X, bool x_is_half, const float* row_scale, int m, float* planes, unsigned int* err,
                              cudaStream_t st, int* terms);

template <int FMT, int G>
static int launch_i(const MatDev& M, const void* X, bool x_is_half, const float* row_scale, int m, float* planes, unsigned int* err, cudaStream_t st,
                    int* terms) {
  if (M.index_bits == 10) return launch_t<FMT, G, 10>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
  return launch_t<FMT, G, 11>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
}

template <int FMT>
static int launch_g(const MatDev& M, const void* X, bool x_is_half, const float* row_scale, int m, float* planes, unsigned int* err, cudaStream_t st,
                    int* terms) {
  if constexpr (is_pair_layout(FMT)) {   // groups of three pair symbols, the layout's own table
    if constexpr (pair_code_bits_max(FMT) == 12)
      if (M.index_bits == 12) return launch_t<FMT, 3, 12>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
    return launch_t<FMT, 3, 11>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
  } else {
    return launch_bundle_code<FMT>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
  }
}

template <int FMT>
static int launch_bundle_code(const MatDev& M, const void* X, bool x_is_half, const float* row_scale, int m, float* planes, unsigned int* err,
                              cudaStream_t st, int* terms) {
  switch (M.group) {
    case 3: return launch_i<FMT, 3>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
    case 4: return launch_i<FMT, 4>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
  }
  if constexpr (!is_paired(FMT)) {
    switch (M.group) {
      case 5: return launch_i<FMT, 5>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
      case 6: return launch_i<FMT, 6>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
    }
  }
  set_kernel_error_text("gemm (tcgen05)", "no kernel for this group size");
  return kErrTooLarge;
}

size_t gemm_t5_plane_floats(const MatDev& M, int m) { return static_cast<size_t>(M.K / kT5SetK) * m * M.N; }

// planes[K / 512][m][N] = partial products of the column sets; *terms = K / 512.  kErrTooLarge (nothing launched) where
// this kernel cannot take the product: more than 64 rows, tile rows not a multiple of four, K not a multiple of 512, or
// too little shared memory left for the staging ring (the 2048-window table with many rows).
int launch_gemm_t5(const MatDev& M, const void* X, bool x_is_half, const float* row_scale, int m, float* planes, unsigned int* err, cudaStream_t st,
                   int* terms) {
  if (!err || !planes || !terms) {
    set_kernel_error_text("gemm (tcgen05)", "null argument");
    return kErrTooLarge;
  }
  switch (M.fmt) {
    case kFmtQ4K: return launch_g<kFmtQ4K>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
    case kFmtQ5K: return launch_g<kFmtQ5K>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
    case kFmtIQ4XS: return launch_g<kFmtIQ4XS>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
    case kFmtQ6K: return launch_g<kFmtQ6K>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
    case kFmtQ6KP: return launch_g<kFmtQ6KP>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
    case kFmtQ5KP: return launch_g<kFmtQ5KP>(M, X, x_is_half, row_scale, m, planes, err, st, terms);
  }
  return kErrTooLarge;
}

}  // namespace lw
