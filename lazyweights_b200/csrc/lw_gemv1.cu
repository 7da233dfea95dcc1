// Instantiations and launcher of the batch-1 kernel: one persistent block per SM; see lw_gemv1.cuh.
#include "lw_gemv1.h"

#include <algorithm>
#include <cstdlib>
#include <memory>
#include <string>

#include "lw_gemv1.cuh"

namespace lw {

constexpr size_t kSmemLimit = 227 * 1024;
constexpr int kMaxStagedColumns = 8;    // tile columns whose activations one block keeps in shared memory
constexpr int kRingSlackWords = 96;     // read-ahead of the last chains of the last staging buffer lands here

struct Gemv1Plan {
  int warps, helpers, producers, producer_lanes, tile_ring_log2, slots, nsets, cols_per_set, blocks, max_units;
  uint32_t buf_words;
  size_t smem;
};

static int env_int(const char* name, int fallback) {
  const char* e = getenv(name);
  return e ? atoi(e) : fallback;
}

// Tuning switches from the environment, read once (a getenv per launch is host overhead on the direct-launch path).
struct Gemv1Env {
  int ring = env_int("LW_GEMV1_RING", 8), warps = env_int("LW_GEMV1_WARPS", 0), producers = env_int("LW_GEMV1_PRODUCERS", 2),
      helpers = env_int("LW_GEMV1_HELPERS", kGemv1MaxWarps), lanes = env_int("LW_GEMV1_LANES", 4), pdl = env_int("LW_PDL", 1);
};
static const Gemv1Env& gemv1_env() {
  static const Gemv1Env e;
  return e;
}

// Plan for a launch over `ntr` tile rows.  False if a unit does not fit shared memory or a block would be dealt more
// units than its list holds (the caller then covers the rows in several launches).
template <int FMT>
static bool plan_gemv1(const MatDev& M, int ntr, Gemv1Plan& p, int index_bits, int avail_blocks = 0) {
  const int log_copies = ring_log_copies(index_bits);
  constexpr int TW = is_paired(FMT) ? 512 : 256, SPLIT = default_split(FMT);
  constexpr bool has_offset = FMT == kFmtQ4K || FMT == kFmtQ5K || FMT == kFmtQ5KP;
  p.nsets = (M.KT + kMaxStagedColumns - 1) / kMaxStagedColumns;
  p.cols_per_set = (M.KT + p.nsets - 1) / p.nsets;
  // a chain reader looks up to three words past its chain; for all buffers but the last that lands in the next buffer
  // (harmless: those bits are never used), so only the end of the ring needs slack
  p.buf_words = (M.max_unit_words + 31u) & ~31u;
  const int tiles = ntr * M.KT;
  p.blocks = std::max(p.nsets, std::min(avail_blocks > 0 ? avail_blocks : sm_count(), tiles));
  p.max_units = 0;   // the longest list any block gets: blocks b, b + nsets, ... serve the tile columns of set b % nsets
  for (int set = 0; set < p.nsets; ++set) {
    const int nb_set = (p.blocks - set + p.nsets - 1) / p.nsets, ncol = (M.KT - set + p.nsets - 1) / p.nsets;
    const int set_tiles = ntr * ncol;
    p.max_units = std::max(p.max_units, (set_tiles + nb_set - 1) / nb_set * SPLIT);
  }
  p.max_units = (p.max_units + 1) & ~1;
  if (p.max_units > debug_knobs().max_units) return false;
  // The ring in which the segments of a tile meet: 8 tiles (28 warps have 7 tiles in flight); 16 with
  // LW_GEMV1_RING=16 where 36 staging buffers still fit (measured: no difference on the bench matrix).
  size_t fixed = 0;
  for (p.tile_ring_log2 = gemv1_env().ring >= 16 ? 4 : 3; p.tile_ring_log2 >= 3; --p.tile_ring_log2) {
    fixed = (size_t(1) << (index_bits + log_copies + 2)) + kLutSize * 4 +
            static_cast<size_t>(p.cols_per_set) * (kTileSyms + (has_offset ? 2 : 1) * (TW / sub_width(FMT))) * 4 +
            2 * kGemv1MaxSlots * 8 + kGemv1MaxSlots * 4 + 16 + (size_t(1) << p.tile_ring_log2) * (8 + SPLIT * kTileRows * 4) +
            p.max_units * sizeof(UnitMeta) + kRingSlackWords * 4;
    if (fixed + static_cast<size_t>(p.buf_words) * 4 * 36 <= kSmemLimit) break;   // 36 buffers still fit
  }
  p.tile_ring_log2 = std::max(3, p.tile_ring_log2);
  if (fixed + static_cast<size_t>(p.buf_words) * 4 > kSmemLimit) return false;
  // as many staging buffers as fit; about three consumers per four buffers, so that copies run ahead of the decoding
  p.slots = static_cast<int>(std::min<size_t>(kGemv1MaxSlots, (kSmemLimit - fixed) / (p.buf_words * 4)));
  // A block whose whole list fits its buffers needs no run-ahead: one warp per unit.  Otherwise about three
  // consumers per four buffers (measured on the bench matrix: 28 warps 35.6 us, 25 warps 37.9 us, 20 warps 39.0 us).
  p.warps = std::max(1, std::min(kGemv1MaxWarps, p.max_units <= p.slots ? p.slots : p.slots * 3 / 4));
  p.warps = std::min(p.warps, p.max_units);
  p.warps = std::max(1, std::min(std::min(kGemv1MaxWarps, p.slots), gemv1_env().warps > 0 ? gemv1_env().warps : p.warps));
  p.producers = std::max(1, std::min(4, gemv1_env().producers));
  p.helpers = std::max(p.warps, std::min(kGemv1MaxWarps, gemv1_env().helpers));
  p.producer_lanes = std::max(1, std::min(32, gemv1_env().lanes));
  p.smem = fixed + static_cast<size_t>(p.slots) * p.buf_words * 4;
  return true;
}

static Gemv1Args make_args(const Gemv1Plan& p, const void* X, bool x_is_half, float* P, float* Y, unsigned int* err, int tr0,
                           int ntr) {
  Gemv1Args a;
  a.x = X;
  a.partials = P;
  a.y = Y;
  a.x_is_half = x_is_half;
  a.helpers = p.helpers;
  a.tile_ring_log2 = p.tile_ring_log2;
  a.pdl = gemv1_env().pdl != 0;
  a.r.err = err;
  a.r.wait_limit = debug_knobs().wait_limit;
  a.r.drop_unit = debug_knobs().drop_unit;
  a.r.warps = p.warps;
  a.r.slots = p.slots;
  a.r.producers = p.producers;
  a.r.producer_lanes = p.producer_lanes;
  a.r.buf_words = p.buf_words;
  a.r.nsets = p.nsets;
  a.r.cols_per_set = p.cols_per_set;
  a.r.max_units = p.max_units;
  a.r.tr0 = tr0;
  a.r.ntr = ntr;
  return a;
}

static void launch_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int blocks, int threads, size_t smem,
                          cudaStream_t st, bool pdl) {
  cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
}

// Several one-row products in one launch (k_gemv1_batch): the grid's blocks are dealt to the matrices in proportion
// to their tiles.  kErrTooLarge (nothing launched) where a matrix's share of the grid cannot hold its unit list; the
// caller then launches the products one by one.
template <int FMT, int G, int IDXBITS>
static int launch_batch_t(int n, const MatDev* const* mats, const void* const* xs, bool x_is_half, float* const* partials,
                          float* const* ys, unsigned int* err, cudaStream_t st) {
  auto B = std::make_unique<Gemv1Batch>();
  const int grid = sm_count();
  long long total_tiles = 0;
  for (int j = 0; j < n; ++j) total_tiles += static_cast<long long>(mats[j]->T);
  int given = 0;
  int share[kGemv1MaxBatch];
  for (int j = 0; j < n; ++j) {
    const int nsets = (mats[j]->KT + kMaxStagedColumns - 1) / kMaxStagedColumns;
    share[j] = std::max(nsets, static_cast<int>(static_cast<long long>(grid) * mats[j]->T / total_tiles));
    given += share[j];
  }
  for (int j = 0; given < grid; j = (j + 1) % n, ++given) ++share[j];   // the remainder, one block each
  if (given > grid) return kErrTooLarge;
  size_t smem = 0;
  int threads = 0;
  B->count = n;
  B->first[0] = 0;
  for (int j = 0; j < n; ++j) {
    Gemv1Plan p;
    if (!plan_gemv1<FMT>(*mats[j], mats[j]->N / kTileRows, p, IDXBITS, share[j])) return kErrTooLarge;
    B->mat[j] = *mats[j];
    B->arg[j] = make_args(p, xs[j], x_is_half, partials[j], ys[j], err, 0, mats[j]->N / kTileRows);
    B->first[j + 1] = B->first[j] + p.blocks;
    smem = std::max(smem, p.smem);
    threads = (p.helpers + p.producers) * 32;
  }
  static size_t configured_per_device[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  size_t& configured = configured_per_device[dev & 63];
  if (smem > configured) {
    if (cudaFuncSetAttribute(k_gemv1_batch<FMT, G, IDXBITS, ring_log_copies(IDXBITS)>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kSmemLimit)) != cudaSuccess)
      return note_launch("cudaFuncSetAttribute(k_gemv1_batch)");
    configured = kSmemLimit;
  }
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  launch_config(cfg, attr, B->first[n], threads, smem, st, gemv1_env().pdl != 0);
  cudaLaunchKernelEx(&cfg, k_gemv1_batch<FMT, G, IDXBITS, ring_log_copies(IDXBITS)>, *B);
  return note_launch("k_gemv1_batch");
}

template <int FMT, int G>
static int launch_batch_i(int n, const MatDev* const* mats, const void* const* xs, bool x_is_half, float* const* partials,
                          float* const* ys, unsigned int* err, cudaStream_t st) {
  if (mats[0]->index_bits == 10) return launch_batch_t<FMT, G, 10>(n, mats, xs, x_is_half, partials, ys, err, st);
  return launch_batch_t<FMT, G, 11>(n, mats, xs, x_is_half, partials, ys, err, st);
}

template <int FMT>
static int launch_batch_g(int n, const MatDev* const* mats, const void* const* xs, bool x_is_half, float* const* partials,
                          float* const* ys, unsigned int* err, cudaStream_t st) {
  if constexpr (is_pair_layout(FMT)) {   // groups of three; the table of the layout's own code, 2048 or 4096 windows
    if constexpr (pair_code_bits_max(FMT) == 12)
      if (mats[0]->index_bits == 12) return launch_batch_t<FMT, 3, 12>(n, mats, xs, x_is_half, partials, ys, err, st);
    return launch_batch_t<FMT, 3, 11>(n, mats, xs, x_is_half, partials, ys, err, st);
  } else {
    switch (mats[0]->group) {
      case 3: return launch_batch_i<FMT, 3>(n, mats, xs, x_is_half, partials, ys, err, st);
      case 4: return launch_batch_i<FMT, 4>(n, mats, xs, x_is_half, partials, ys, err, st);
    }
    if constexpr (!is_paired(FMT)) {
      switch (mats[0]->group) {
        case 5: return launch_batch_i<FMT, 5>(n, mats, xs, x_is_half, partials, ys, err, st);
        case 6: return launch_batch_i<FMT, 6>(n, mats, xs, x_is_half, partials, ys, err, st);
      }
    }
    return kErrTooLarge;
  }
}

int launch_gemv1_batch(int n, const MatDev* const* mats, const void* const* xs, bool x_is_half, float* const* partials,
                       float* const* ys, unsigned int* err, cudaStream_t st) {
  if (n < 1 || n > kGemv1MaxBatch || !err) return kErrTooLarge;
  for (int j = 0; j < n; ++j) {
    const MatDev& M = *mats[j];
    if (!gemv1_usable(M) || M.reader != 0 || M.fmt != mats[0]->fmt || M.group != mats[0]->group ||
        M.index_bits != mats[0]->index_bits)
      return kErrTooLarge;   // not one kernel instantiation: the caller launches them one by one
    if ((reinterpret_cast<uintptr_t>(ys[j]) | reinterpret_cast<uintptr_t>(partials[j])) & 15u) {
      set_kernel_error_text("gemv1", "the result and the scratch must be 16-byte aligned");
      return kErrArg;
    }
  }
  if (debug_knobs().drop_unit >= 0 || debug_knobs().max_units < kGemv1MaxUnits) return kErrTooLarge;   // test switches: plain launches
  switch (mats[0]->fmt) {
    case kFmtQ4K: return launch_batch_g<kFmtQ4K>(n, mats, xs, x_is_half, partials, ys, err, st);
    case kFmtQ5K: return launch_batch_g<kFmtQ5K>(n, mats, xs, x_is_half, partials, ys, err, st);
    case kFmtIQ4XS: return launch_batch_g<kFmtIQ4XS>(n, mats, xs, x_is_half, partials, ys, err, st);
    case kFmtQ6KP: return launch_batch_g<kFmtQ6KP>(n, mats, xs, x_is_half, partials, ys, err, st);
    case kFmtQ5KP: return launch_batch_g<kFmtQ5KP>(n, mats, xs, x_is_half, partials, ys, err, st);
    default: return launch_batch_g<kFmtQ6K>(n, mats, xs, x_is_half, partials, ys, err, st);
  }
}

template <int FMT, int G, int IDXBITS, int LOG_R, int READER = kReaderTable>
static int launch_t(const MatDev& M, const void* X, bool x_is_half, float* P, float* Y, unsigned int* err,
                    cudaStream_t st) {
  // A block's list holds at most kRingMaxUnits units; a matrix with more tile rows than that allows (a vocabulary
  // projection of 128k rows x 8192 columns, say) is covered by several launches over ranges of tile rows.
  const int NT = M.N / kTileRows;
  Gemv1Plan p;
  int chunks = 1;
  while (!plan_gemv1<FMT>(M, (NT + chunks - 1) / chunks, p, IDXBITS)) {
    if (p.max_units <= debug_knobs().max_units || chunks >= NT) {
      set_kernel_error_text("gemv1", "work unit does not fit shared memory");
      return kErrTooLarge;
    }
    chunks = std::min(NT, std::max(chunks + 1, chunks * p.max_units / debug_knobs().max_units));
  }
  // the attribute is raised once per kernel instantiation and device, not on every launch
  static size_t configured_per_device[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  size_t& configured = configured_per_device[dev & 63];
  if (p.smem > configured) {
    if (cudaFuncSetAttribute(k_gemv1<FMT, G, IDXBITS, LOG_R, READER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kSmemLimit)) != cudaSuccess)
      return note_launch("cudaFuncSetAttribute(k_gemv1)");
    configured = kSmemLimit;
  }
  const int per = (NT + chunks - 1) / chunks;
  for (int tr0 = 0; tr0 < NT; tr0 += per) {
    const int ntr = std::min(per, NT - tr0);
    if (ntr != per && !plan_gemv1<FMT>(M, ntr, p, IDXBITS)) {
      set_kernel_error_text("gemv1", "work unit does not fit shared memory");
      return kErrTooLarge;
    }
    const Gemv1Args a = make_args(p, X, x_is_half, P, Y, err, tr0, ntr);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_config(cfg, attr, p.blocks, (p.helpers + p.producers) * 32, p.smem, st, a.pdl != 0);
    cudaLaunchKernelEx(&cfg, k_gemv1<FMT, G, IDXBITS, LOG_R, READER>, M, a);
    const int rc = note_launch("k_gemv1");
    if (rc) return rc;
  }
  return kOk;
}

template <int FMT, int G>
static int launch_i(const MatDev& M, const void* X, bool x_is_half, float* P, float* Y, unsigned int* err, cudaStream_t st) {
  // LW_GEMV1_LOOKUP=limit: the comparator decoder instead of the table (a measurement switch, read once)
  static const bool use_limit = [] {
    const char* e = getenv("LW_GEMV1_LOOKUP");
    return e && std::string(e) == "limit";
  }();
  if (use_limit && M.cmp_tab) return launch_t<FMT, G, 10, kGemv1LogCopies, kReaderLimit>(M, X, x_is_half, P, Y, err, st);
  if (M.index_bits == 10) return launch_t<FMT, G, 10, kGemv1LogCopies>(M, X, x_is_half, P, Y, err, st);
  return launch_t<FMT, G, 11, ring_log_copies(11)>(M, X, x_is_half, P, Y, err, st);
}

template <int FMT>
static int launch_g(const MatDev& M, const void* X, bool x_is_half, float* P, float* Y, unsigned int* err, cudaStream_t st) {
  if constexpr (is_pair_layout(FMT)) {
    if constexpr (pair_code_bits_max(FMT) == 12)
      if (M.index_bits == 12) return launch_t<FMT, 3, 12, ring_log_copies(12)>(M, X, x_is_half, P, Y, err, st);
    return launch_t<FMT, 3, 11, ring_log_copies(11)>(M, X, x_is_half, P, Y, err, st);
  } else {
    if (M.reader == 1) return launch_t<FMT, 3, 10, kGemv1LogCopies, kReaderFixed>(M, X, x_is_half, P, Y, err, st);
    switch (M.group) {
      case 3: return launch_i<FMT, 3>(M, X, x_is_half, P, Y, err, st);
      case 4: return launch_i<FMT, 4>(M, X, x_is_half, P, Y, err, st);
    }
    if constexpr (!is_paired(FMT)) {
      switch (M.group) {
        case 5: return launch_i<FMT, 5>(M, X, x_is_half, P, Y, err, st);
        case 6: return launch_i<FMT, 6>(M, X, x_is_half, P, Y, err, st);
      }
    }
    set_kernel_error_text("gemv1", "no kernel for this group size");
    return kErrArg;
  }
}

bool gemv1_usable(const MatDev& M) {
  if (is_pair_layout(M.fmt))
    return (M.index_bits == 11 || M.index_bits == pair_code_bits_max(M.fmt)) && M.pad == pair_pad_bits(M.index_bits) && M.split == default_split(M.fmt) && M.unit_slow && M.row_done &&
           M.group == 3 && M.reader == 0;
  const bool fmt_ok = M.fmt >= kFmtQ4K && M.fmt <= kFmtIQ4XS;
  const int gmax = is_paired(M.fmt) ? 4 : 6;
  return fmt_ok && (M.index_bits == 10 || M.index_bits == 11) && M.pad == kRingLogCopies + 2 && M.split == default_split(M.fmt) && M.unit_slow && M.row_done && M.group >= 3 &&
         M.group <= gmax;
}

int launch_gemv1(const MatDev& M, const void* X, bool x_is_half, float* P, float* Y, unsigned int* err, cudaStream_t st) {
  if (!err) {
    set_kernel_error_text("gemv1", "no device error word");
    return kErrCuda;
  }
  if ((reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(P)) & 15u) {
    set_kernel_error_text("gemv1", "the result and the scratch must be 16-byte aligned");
    return kErrArg;
  }
  switch (M.fmt) {
    case kFmtQ4K: return launch_g<kFmtQ4K>(M, X, x_is_half, P, Y, err, st);
    case kFmtQ5K: return launch_g<kFmtQ5K>(M, X, x_is_half, P, Y, err, st);
    case kFmtIQ4XS: return launch_g<kFmtIQ4XS>(M, X, x_is_half, P, Y, err, st);
    case kFmtQ6KP: return launch_g<kFmtQ6KP>(M, X, x_is_half, P, Y, err, st);
    case kFmtQ5KP: return launch_g<kFmtQ5KP>(M, X, x_is_half, P, Y, err, st);
    default: return launch_g<kFmtQ6K>(M, X, x_is_half, P, Y, err, st);
  }
}

}  // namespace lw

#ifdef LW_GEMV1_PROFILE
extern "C" int lw_debug_prof(unsigned long long* out, int reset) {
  cudaDeviceSynchronize();
  if (cudaMemcpyFromSymbol(out, lw::g_gemv1_prof, sizeof(unsigned long long) * 8) != cudaSuccess) return -1;
  if (reset) {
    unsigned long long z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    cudaMemcpyToSymbol(lw::g_gemv1_prof, z, sizeof z);
  }
  return 0;
}
#endif
