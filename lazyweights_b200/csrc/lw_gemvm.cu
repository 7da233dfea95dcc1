// Instantiations and launcher of the 2..8-row fused kernel; see lw_gemvm.cuh.
#include "lw_gemv1.h"

#include <algorithm>
#include <cstdlib>

#include "lw_gemvm.cuh"

namespace lw {

constexpr size_t kSmemLimit = 227 * 1024;
constexpr int kRingSlackWords = 96;

struct GemvmPlan {
  int warps, producers, slots, nsets, cols_per_set, blocks, max_units;
  uint32_t buf_words;
  size_t smem;
};

template <int FMT, int MR>
static bool plan_gemvm(const MatDev& M, int ntr, GemvmPlan& p) {
  constexpr int TW = is_paired(FMT) ? 512 : 256, SPLIT = default_split(FMT), NSB = TW / sub_width(FMT);
  constexpr bool has_offset = FMT == kFmtQ4K || FMT == kFmtQ5K || FMT == kFmtQ5KP;
  const int staged = std::max(1, 8 / MR);   // tile columns whose activations (all rows) one block keeps in shared memory
  p.nsets = (M.KT + staged - 1) / staged;
  p.cols_per_set = (M.KT + p.nsets - 1) / p.nsets;
  p.buf_words = (M.max_unit_words + 31u) & ~31u;
  const int tiles = ntr * M.KT;
  p.blocks = std::max(p.nsets, std::min(sm_count(), tiles));
  p.max_units = 0;
  for (int set = 0; set < p.nsets; ++set) {
    const int nb_set = (p.blocks - set + p.nsets - 1) / p.nsets, ncol = (M.KT - set + p.nsets - 1) / p.nsets;
    const int set_tiles = ntr * ncol;
    p.max_units = std::max(p.max_units, (set_tiles + nb_set - 1) / nb_set * SPLIT);
  }
  p.max_units = (p.max_units + 1) & ~1;
  if (p.max_units > debug_knobs().max_units) return false;
  const size_t fixed = (size_t(1) << (M.index_bits + ring_log_copies(M.index_bits) + 2)) + kLutSize * 4 +
                       static_cast<size_t>(p.cols_per_set) * (kTileSyms + (has_offset ? 2 : 1) * NSB) * MR * 4 +
                       2 * kGemv1MaxSlots * 8 + kGemv1MaxSlots * 4 + 16 + p.max_units * sizeof(UnitMeta) +
                       kRingSlackWords * 4;
  if (fixed + static_cast<size_t>(p.buf_words) * 4 > kSmemLimit) return false;
  p.slots = static_cast<int>(std::min<size_t>(kGemv1MaxSlots, (kSmemLimit - fixed) / (p.buf_words * 4)));
  p.producers = 2;
  const int wmax = gemvm_threads(MR) / 32 - p.producers;
  p.warps = std::max(1, std::min(wmax, p.max_units <= p.slots ? p.slots : p.slots * 3 / 4));
  p.smem = fixed + static_cast<size_t>(p.slots) * p.buf_words * 4;
  return true;
}

template <int FMT, int G, int IDXBITS, int MR>
static int launch_t(const MatDev& M, const void* X, bool x_is_half, int m, float* P, unsigned int* err, cudaStream_t st) {
  // as in the batch-1 launcher: more tile rows than one block's list can hold are covered by several launches
  const int NT = M.N / kTileRows;
  GemvmPlan p;
  int chunks = 1;
  while (!plan_gemvm<FMT, MR>(M, (NT + chunks - 1) / chunks, p)) {
    if (p.max_units <= debug_knobs().max_units || chunks >= NT) {
      set_kernel_error_text("gemvm", "work unit does not fit shared memory");
      return kErrTooLarge;
    }
    chunks = std::min(NT, std::max(chunks + 1, chunks * p.max_units / debug_knobs().max_units));
  }
  auto kernel = k_gemvm<FMT, G, IDXBITS, ring_log_copies(IDXBITS), MR>;
  static size_t configured_per_device[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  size_t& configured = configured_per_device[dev & 63];
  if (p.smem > configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemLimit)) != cudaSuccess)
      return note_launch("cudaFuncSetAttribute(k_gemvm)");
    configured = kSmemLimit;
  }
  const int per = (NT + chunks - 1) / chunks;
  for (int tr0 = 0; tr0 < NT; tr0 += per) {
    const int ntr = std::min(per, NT - tr0);
    if (ntr != per && !plan_gemvm<FMT, MR>(M, ntr, p)) {
      set_kernel_error_text("gemvm", "work unit does not fit shared memory");
      return kErrTooLarge;
    }
    GemvmArgs a;
    a.x = X;
    a.partials = P;
    a.x_is_half = x_is_half;
    a.pdl = 1;
    a.m = m;
    a.r.err = err;
    a.r.wait_limit = debug_knobs().wait_limit;
    a.r.drop_unit = -1;
    a.r.warps = p.warps;
    a.r.slots = p.slots;
    a.r.producers = p.producers;
    a.r.producer_lanes = 4;
    a.r.buf_words = p.buf_words;
    a.r.nsets = p.nsets;
    a.r.cols_per_set = p.cols_per_set;
    a.r.max_units = p.max_units;
    a.r.tr0 = tr0;
    a.r.ntr = ntr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.blocks);
    cfg.blockDim = dim3((p.warps + p.producers) * 32);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, M, a);
    const int rc = note_launch("k_gemvm");
    if (rc) return rc;
  }
  return kOk;
}

template <int FMT, int G, int IDXBITS>
static int launch_r(const MatDev& M, const void* X, bool x_is_half, int m, float* P, unsigned int* err, cudaStream_t st) {
  if (m <= 4) return launch_t<FMT, G, IDXBITS, 4>(M, X, x_is_half, m, P, err, st);
  return launch_t<FMT, G, IDXBITS, 8>(M, X, x_is_half, m, P, err, st);
}

template <int FMT, int G>
static int launch_i(const MatDev& M, const void* X, bool x_is_half, int m, float* P, unsigned int* err, cudaStream_t st) {
  if (M.index_bits == 10) return launch_r<FMT, G, 10>(M, X, x_is_half, m, P, err, st);
  return launch_r<FMT, G, 11>(M, X, x_is_half, m, P, err, st);
}

template <int FMT>
static int launch_g(const MatDev& M, const void* X, bool x_is_half, int m, float* P, unsigned int* err, cudaStream_t st) {
  if constexpr (is_pair_layout(FMT)) {   // groups of three pair symbols, the layout's own table
    if constexpr (pair_code_bits_max(FMT) == 12)
      if (M.index_bits == 12) return launch_r<FMT, 3, 12>(M, X, x_is_half, m, P, err, st);
    return launch_r<FMT, 3, 11>(M, X, x_is_half, m, P, err, st);
  } else {
    switch (M.group) {
      case 3: return launch_i<FMT, 3>(M, X, x_is_half, m, P, err, st);
      case 4: return launch_i<FMT, 4>(M, X, x_is_half, m, P, err, st);
    }
    if constexpr (!is_paired(FMT)) {
      switch (M.group) {
        case 5: return launch_i<FMT, 5>(M, X, x_is_half, m, P, err, st);
        case 6: return launch_i<FMT, 6>(M, X, x_is_half, m, P, err, st);
      }
    }
    set_kernel_error_text("gemvm", "no kernel for this group size");
    return kErrArg;
  }
}

size_t gemvm_partial_floats(const MatDev& M, int m) {
  return static_cast<size_t>(M.KT) * M.split * m * M.N;
}

int launch_gemvm(const MatDev& M, const void* X, bool x_is_half, int m, float* P, unsigned int* err, cudaStream_t st) {
  if (!err || m < 2 || m > 8) {
    set_kernel_error_text("gemvm", "bad argument");
    return kErrArg;
  }
  switch (M.fmt) {
    case kFmtQ4K: return launch_g<kFmtQ4K>(M, X, x_is_half, m, P, err, st);
    case kFmtQ5K: return launch_g<kFmtQ5K>(M, X, x_is_half, m, P, err, st);
    case kFmtIQ4XS: return launch_g<kFmtIQ4XS>(M, X, x_is_half, m, P, err, st);
    case kFmtQ6KP: return launch_g<kFmtQ6KP>(M, X, x_is_half, m, P, err, st);
    case kFmtQ5KP: return launch_g<kFmtQ5KP>(M, X, x_is_half, m, P, err, st);
    default: return launch_g<kFmtQ6K>(M, X, x_is_half, m, P, err, st);
  }
}

}  // namespace lw
