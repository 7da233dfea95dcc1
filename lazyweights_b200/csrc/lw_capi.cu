// The extern "C" surface (include/lwb200.h): bundle handles, per-matrix products and decodes, the host codec.
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/lwb200.h"
#include "lw_host.h"
#include "lw_gemv1.h"
#include "lw_kernels.h"
#include "lw_model.h"

namespace lw {

void set_kernel_error_text(const char* what, const char* detail) { set_error("%s: %s", what, detail); }

int cuda_fail(const char* what, cudaError_t e) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver ? kErrNoDevice : kErrCuda;
}

static int require_device(int* dev) {
  int n = 0;
  const cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    set_error("no CUDA device: this library has no CPU path for GPU entry points");
    return kErrNoDevice;
  }
  if (cudaGetDevice(dev) != cudaSuccess) return cuda_fail("cudaGetDevice", cudaGetLastError());
  return kOk;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Host-side result of validating, indexing and re-laying out one blob: everything that goes to the device.
struct HostImage {
  PairImage pair;   // fmt == kFmtNone: the matrix has no pair layout
  std::vector<uint16_t> lut;
  std::vector<uint32_t> fat, symtab, cmp, group_base, words;
  std::vector<uint8_t> unit_slow;
  int KT = 0, T = 0, split = 1, pad = 0, max_len = 0, group = 0, index_bits = 0;
  double slow_fraction = 0.0;
  uint32_t max_unit = 0, max_tile = 0;
};

static int check_side(const Matrix& mx, const uint8_t* side, size_t side_nbytes) {
  if (mx.fmt == kFmtNone) return kOk;
  const size_t want = static_cast<size_t>(mx.N) * (mx.K / 256) * side_bytes(mx.fmt);
  if (mx.K % 256 || side_nbytes != want || !side) {
    set_error("%s: side tensor of %zu bytes, expected %zu", mx.name.c_str(), side_nbytes, want);
    return kErrFormat;
  }
  return kOk;
}

// Matrices with a block format whose bundle code uses 11-bit words are re-coded at load with the same rule limited to
// 10 bits (LW_RECODE=0, read at every load: keep the bundle's own code).  The symbols are the same; the device then holds
// a code whose 1024-window table fits sixteen times where the 2048-window table fits eight times, and shared-memory
// bank conflicts are what bounds the product kernels (Q4_K 4096 x 4096: 4.5 instead of 5.1 us per product).
static bool recode_wanted() {
  const char* e = getenv("LW_RECODE");
  return !(e && e[0] == '0');
}

static int prepare_matrix(const Matrix& mx, const uint8_t* blob, size_t nbytes, const uint8_t* side, size_t side_nbytes,
                          int threads, HostImage& im, bool may_recode = true) {
  BlobView v;
  int rc = make_view(blob, nbytes, mx.N, mx.Ks, v);
  if (rc) return rc;
  if ((rc = check_side(mx, side, side_nbytes))) return rc;
  auto tab = std::make_unique<HuffTable>();
  if ((rc = table_from_lut(v.lut(), *tab))) return rc;
  if (may_recode && recode_wanted() && mx.fmt != kFmtNone && tab->max_len > 10) {
    // validate and decode the bundle's blob, encode the symbols again with the shorter limit, lay that blob out
    std::vector<uint8_t> symbols(static_cast<size_t>(mx.N) * mx.Ks), shorter;
    if ((rc = walk_blob(v, *tab, default_split(mx.fmt), threads, nullptr, nullptr, symbols.data(), nullptr))) return rc;
    rc = encode_huf8(symbols.data(), mx.N, mx.Ks, shorter, nullptr, 10, threads);
    symbols = std::vector<uint8_t>();
    if (rc == kOk) return prepare_matrix(mx, shorter.data(), shorter.size(), side, side_nbytes, threads, im, false);
    if (rc != kErrTooLarge) return rc;   // a payload at the format's 2^32-bit limit: the bundle's own code stays
  }
  const int split = default_split(mx.fmt);
  std::vector<uint32_t> chain_start, lane_end;
  im.fat.resize(kLutSize);
  fat_table(*tab, mx.fmt, im.fat.data());
  im.symtab.resize(kLutSize);
  fat_table(*tab, kFmtNone, im.symtab.data());   // length << 28 | symbol
  im.cmp.resize(kCmpTabWords);
  comparator_table(*tab, mx.fmt, im.cmp.data());
  GroupScan scan;
  scan.quad_syms = 4 * sub_syms(mx.fmt);
  const bool grouped = mx.fmt != kFmtNone && split == default_split(mx.fmt);
  // Q6_K / Q5_K rows of whole 512-weight tiles also get a pair layout for the one-row product (LW_PAIRS=0: none); it
  // is built from the decoded codes, which the same walk writes out
  static const bool pairs_wanted = [] {
    const char* e = getenv("LW_PAIRS");
    return !(e && e[0] == '0');
  }();
  const bool pairs = pairs_wanted && grouped && pair_layout_of(mx.fmt) != kFmtNone && mx.K % 512 == 0 && side;
  std::vector<uint8_t> codes;
  if (pairs) codes.resize(static_cast<size_t>(mx.N) * mx.Ks);
  if ((rc = walk_blob(v, *tab, split, threads, &chain_start, &lane_end, pairs ? codes.data() : nullptr, grouped ? &scan : nullptr)))
    return rc;
  if (pairs && (rc = build_pairs(codes.data(), mx.N, mx.K, mx.fmt, side, threads, im.pair))) return rc;
  codes = std::vector<uint8_t>();
  // The batch-1 kernel's table: 1024 windows (codes up to 10 bits; units that hold a longer code are decoded symbol
  // by symbol) or 2048, 16 copies each; and the group size: units where groups of g symbols are not exact fall back
  // to groups of two.  Estimated cost per symbol: 8.3 instructions + 10 per group; groups of two cost about 22
  // (measured: more than their instruction count); the larger table leaves a third fewer staging buffers (+ 8 %);
  // symbol by symbol costs about 30.  LW_GEMV1_G / LW_GEMV1_IDX override.
  int idx_bits = tab->max_len <= 10 ? 10 : 11, group = 0;
  if (grouped) {
    const int gmax = is_paired(mx.fmt) ? 4 : kScanMaxG;
    const char* eg = getenv("LW_GEMV1_G");
    const char* ei = getenv("LW_GEMV1_IDX");
    double best = 1e30;
    const double n = static_cast<double>(std::max<size_t>(1, scan.mask.size()));
    for (int ib = 10; ib <= 11; ++ib) {
      if (ei && atoi(ei) != ib) continue;
      for (int g = kScanMinG; g <= gmax; ++g) {
        if (eg && atoi(eg) != g) continue;
        const uint8_t gbit = static_cast<uint8_t>(1u << (g - kScanMinG));
        size_t two = 0, single = 0;
        for (uint8_t m : scan.mask) {
          if (ib == 10 && (m & 0x80u)) ++single;
          else if (m & gbit) ++two;
        }
        const double f2 = two / n, f1 = single / n;
        const double cost = ((1.0 - f2 - f1) * (8.3 + 10.0 / g) + f2 * 22.0) * (ib == 11 ? 1.08 : 1.0) + f1 * 30.0;
        if (cost < best) {
          best = cost;
          group = g;
          idx_bits = ib;
          im.slow_fraction = f1 + f2;
        }
      }
    }
    if (group) {
      const uint8_t gbit = static_cast<uint8_t>(1u << (group - kScanMinG));
      im.unit_slow.resize(scan.mask.size());
      for (size_t i = 0; i < scan.mask.size(); ++i)
        im.unit_slow[i] = (idx_bits == 10 && (scan.mask[i] & 0x80u)) ? 2 : (scan.mask[i] & gbit) ? 1 : 0;
    }
  }
  // Leading zero bits of every chain: they place the decode window on the address bits of the batch-1 kernel's
  // table of 4-byte entries, 16 copies (64 bytes) per window.
  const int pad = 6;
  if ((rc = relayout(v, split, pad, chain_start, lane_end, threads, im.group_base, im.words, &im.max_unit, &im.max_tile,
                     mx.fmt, group ? side : nullptr)))
    return rc;
  im.group = group;
  im.index_bits = idx_bits;
  im.lut.assign(v.lut(), v.lut() + kLutSize);
  im.KT = v.KT;
  im.T = v.T;
  im.split = split;
  im.pad = pad;
  im.max_len = tab->max_len;
  return kOk;
}

// The pair layout as a second device image with a descriptor of its own.
static int upload_pairs(Matrix& mx, const PairImage& p) {
  const size_t off_gb = align_up(p.tab32.size() * 4, 256);
  const size_t off_words = align_up(off_gb + p.group_base.size() * 4, 256);
  const size_t off_cls = align_up(off_words + p.words.size() * 4, 256);
  const size_t off_done = off_cls + align_up(p.unit_class.size(), 256);
  const size_t total = off_done + align_up(static_cast<size_t>(mx.N / kTileRows) * kRowDoneStride * 4, 256);
  cudaError_t e = cudaMalloc(&mx.d_pair, total);
  if (e != cudaSuccess) return cuda_fail("cudaMalloc (pair layout)", e);
  uint8_t* d = static_cast<uint8_t*>(mx.d_pair);
  if ((e = cudaMemset(d + off_cls, 0, total - off_cls)) != cudaSuccess ||
      (e = cudaMemcpy(d, p.tab32.data(), p.tab32.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_gb, p.group_base.data(), p.group_base.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_words, p.words.data(), p.words.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_cls, p.unit_class.data(), p.unit_class.size(), cudaMemcpyHostToDevice)) != cudaSuccess)
    return cuda_fail("cudaMemcpy (pair layout)", e);
  MatDev& P = mx.pair;
  P = MatDev{};
  P.tab32 = reinterpret_cast<const uint32_t*>(d);
  P.group_base = reinterpret_cast<const uint32_t*>(d + off_gb);
  P.words = reinterpret_cast<const uint32_t*>(d + off_words);
  P.unit_slow = d + off_cls;
  P.row_done = reinterpret_cast<unsigned int*>(d + off_done);
  P.index_bits = p.index_bits;
  P.group = p.group;
  P.N = mx.N;
  P.K = mx.K;
  P.Ks = mx.K / 2;
  P.KT = p.KT;
  P.T = p.T;
  P.fmt = p.fmt;
  P.split = p.split;
  P.reader = 0;
  P.pad = p.pad;
  P.max_len = p.max_len;
  P.max_tile_words = p.max_tile_words;
  P.max_unit_words = p.max_unit_words;
  mx.pair_bytes = (p.words.size() - kTailWords) * 4;
  mx.pair_epoch = 0;
  mx.device_bytes += total;
  return kOk;
}

static int upload_matrix(Matrix& mx, const HostImage& im, const uint8_t* side, size_t side_nbytes) {
  const int rc_side = check_side(mx, side, side_nbytes);
  if (rc_side) return rc_side;
  const size_t off_fat = align_up(2 * kLutSize, 256);
  const size_t off_sym = align_up(off_fat + 4 * kLutSize, 256);
  const size_t off_cmp = align_up(off_sym + 4 * kLutSize, 256);
  const size_t off_gb = align_up(off_cmp + 4 * kCmpTabWords, 256);
  const size_t off_words = align_up(off_gb + im.group_base.size() * 4, 256);
  const size_t off_side = align_up(off_words + im.words.size() * 4, 256);
  const size_t off_slow = off_side + align_up(side_nbytes, 256);
  const size_t off_done = off_slow + align_up(im.unit_slow.size(), 256);
  const size_t total = off_done + align_up(static_cast<size_t>(mx.N / kTileRows) * kRowDoneStride * 4, 256);
  cudaError_t e = cudaMalloc(&mx.d_block, total);
  if (e != cudaSuccess) return cuda_fail("cudaMalloc (matrix)", e);
  uint8_t* d = static_cast<uint8_t*>(mx.d_block);
  if ((e = cudaMemcpy(d, im.lut.data(), 2 * kLutSize, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_fat, im.fat.data(), 4 * kLutSize, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_sym, im.symtab.data(), 4 * kLutSize, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_cmp, im.cmp.data(), 4 * kCmpTabWords, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_gb, im.group_base.data(), im.group_base.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_words, im.words.data(), im.words.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (side_nbytes && (e = cudaMemcpy(d + off_side, side, side_nbytes, cudaMemcpyHostToDevice)) != cudaSuccess) ||
      (!im.unit_slow.empty() &&
       (e = cudaMemcpy(d + off_slow, im.unit_slow.data(), im.unit_slow.size(), cudaMemcpyHostToDevice)) != cudaSuccess))
    return cuda_fail("cudaMemcpy (matrix)", e);
  if ((e = cudaMemset(d + off_done, 0, total - off_done)) != cudaSuccess) return cuda_fail("cudaMemset (matrix)", e);
  mx.dev.row_done = reinterpret_cast<unsigned int*>(d + off_done);
  mx.device_bytes = total;
  mx.slow_fraction = im.slow_fraction;
  mx.dev.lut = reinterpret_cast<const uint16_t*>(d);
  mx.dev.tab32 = reinterpret_cast<const uint32_t*>(d + off_fat);
  mx.dev.symtab32 = reinterpret_cast<const uint32_t*>(d + off_sym);
  mx.dev.cmp_tab = reinterpret_cast<const uint32_t*>(d + off_cmp);
  mx.dev.reader = 0;
  mx.dev.pad = im.pad;
  mx.dev.max_len = im.max_len;
  mx.dev.group_base = reinterpret_cast<const uint32_t*>(d + off_gb);
  mx.dev.words = reinterpret_cast<const uint32_t*>(d + off_words);
  tile_output_warm();
  mx.dev.side = side_nbytes ? d + off_side : nullptr;
  mx.dev.unit_slow = im.unit_slow.empty() ? nullptr : d + off_slow;
  mx.dev.group = im.unit_slow.empty() ? 0 : im.group;
  mx.dev.index_bits = im.index_bits;
  mx.dev.N = mx.N;
  mx.dev.K = mx.K;
  mx.dev.Ks = mx.Ks;
  mx.dev.KT = im.KT;
  mx.dev.T = im.T;
  mx.dev.fmt = mx.fmt;
  mx.dev.split = im.split;
  mx.dev.max_tile_words = im.max_tile;
  mx.dev.max_unit_words = im.max_unit;
  return im.pair.fmt != kFmtNone && mx.dev.group ? upload_pairs(mx, im.pair) : kOk;
}

// Validates, indexes, re-lays out and uploads one blob.  Ks = symbols per row.
static int load_matrix(Matrix& mx, const uint8_t* blob, size_t nbytes, const uint8_t* side, size_t side_nbytes,
                       int threads) {
  HostImage im;
  const int rc = prepare_matrix(mx, blob, nbytes, side, side_nbytes, threads, im);
  return rc ? rc : upload_matrix(mx, im, side, side_nbytes);
}

static int finish_model(Model* M) {
  size_t need = 0;
  for (auto& m : M->mats) {
    if (m.fmt != kFmtNone && m.dev.group) {
      need = std::max(need, gemv_partial_floats(m.dev, 8));
      if (m.K % 512 == 0) need = std::max(need, gemm_t5_plane_floats(m.dev, 64));   // planes of the tcgen05 path
    }
    M->resident_bytes += m.device_bytes;
    M->coded_bytes += m.blob_bytes;
    M->side_bytes += m.side_bytes;
  }
  if (need) {
    const cudaError_t e = cudaMalloc(&M->d_partials, need * sizeof(float));
    if (e != cudaSuccess) return cuda_fail("cudaMalloc (partials)", e);
    M->partial_floats = need;
    // range factors of the rows of fp32 activations on the fp16 paths: here, not on first use, so that a pass that is
    // being captured into a graph never allocates
    const cudaError_t e2 = cudaMalloc(&M->d_row_scale, 4096 * sizeof(float));
    if (e2 != cudaSuccess) return cuda_fail("cudaMalloc (row factors)", e2);
    M->row_scale_floats = 4096;
  }
  return kOk;
}

static Matrix* matrix_by_id(void* h, int id) {
  Model* M = static_cast<Model*>(h);
  if (!M || id < 0 || id >= static_cast<int>(M->mats.size())) {
    set_error("no matrix with id %d", id);
    return nullptr;
  }
  return &M->mats[id];
}

// m: rows of the product (1 also stands for the row-count-free users: decode to weights, the tensor-core kernel)
static bool reads_pairs(const Matrix& mx, int m) { return m >= 1 && m <= 8 && mx.d_pair && debug_knobs().pairs; }

// Codes of one matrix, a byte each (a paired format: a byte per pair unless `expand`). An unpaired format's codes are its
// symbols, so its pair layout yields two per table lookup; a shape that layout's kernel does not take reads the bundle's code.
static int decode_codes_of(const Matrix& mx, uint8_t* out, bool expand, cudaStream_t st) {
  int rc = !mx.paired && reads_pairs(mx, 1) ? launch_decode_codes(mx.pair, out, true, st) : kErrTooLarge;
  if (rc == kErrTooLarge) rc = launch_decode_codes(mx.dev, out, expand && mx.paired, st);
  return rc;
}

const MatDev* matrix_descriptor(void* handle, int id, bool one_row) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx || check_device(static_cast<Model*>(handle))) return nullptr;
  return reads_pairs(*mx, one_row ? 1 : 0) ? &mx->pair : &mx->dev;
}

unsigned int* matrix_clean_epoch(void* handle, int id, bool one_row) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return nullptr;
  return reads_pairs(*mx, one_row ? 1 : 0) ? &mx->pair_epoch : &mx->clean_epoch;
}

int check_device(const Model* M) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return cuda_fail("cudaGetDevice", cudaGetLastError());
  if (dev != M->device) {
    set_error("the handle was opened on device %d but the current device is %d", M->device, dev);
    return kErrArg;
  }
  return kOk;
}

static int matrix_id(Model* M, const char* name) {
  if (!M || !name) return -1;
  auto it = M->by_name.find(name);
  if (it == M->by_name.end()) {
    set_error("no coded matrix named %s", name);
    return -1;
  }
  return it->second;
}

template <class T>
static int grow(T** buf, size_t* have, size_t want, const char* what) {
  if (want <= *have) return kOk;
  if (*buf) cudaFree(*buf);
  *buf = nullptr;
  *have = 0;
  const cudaError_t e = cudaMalloc(reinterpret_cast<void**>(buf), want * sizeof(T));
  if (e != cudaSuccess) return cuda_fail(what, e);
  *have = want;
  return kOk;
}

// Decode + GEMM (the reference's path for more than eight rows, kernels/llmrt.cu:1827-1841): tile rows are decoded to
// fp16 weights in chunks that fit the scratch (grown on first use, at most kDecodeScratchBytes) and multiplied on the
// tensor cores.
constexpr size_t kDecodeScratchBytes = size_t(64) << 20;

static int linear_decode_gemm(Model* M, Matrix& mx, const void* x, bool x_half, int m, float* y, int ldy,
                              cudaStream_t st) {
  int rc;
  const __half* x16 = static_cast<const __half*>(x);
  const float* unscale = nullptr;
  if (!x_half) {
    if ((rc = grow(&M->d_x16, &M->x16_halfs, static_cast<size_t>(m) * mx.K, "cudaMalloc (fp16 activations)"))) return rc;
    if ((rc = grow(&M->d_row_scale, &M->row_scale_floats, static_cast<size_t>(2) * m, "cudaMalloc (row factors)"))) return rc;
    if ((rc = launch_row_scales(static_cast<const float*>(x), m, mx.K, M->d_row_scale, st))) return rc;
    if ((rc = launch_to_half_rows(static_cast<const float*>(x), M->d_x16, m, mx.K, M->d_row_scale, st))) return rc;
    x16 = M->d_x16;
    unscale = M->d_row_scale + m;
  }
  const int NT = mx.N / kTileRows;
  const size_t row_halfs = static_cast<size_t>(kTileRows) * mx.K;
  const int fit = static_cast<int>(std::max<size_t>(1, kDecodeScratchBytes / 2 / row_halfs));
  const int chunk = std::min(NT, fit);
  if ((rc = grow(&M->d_w16, &M->w16_halfs, static_cast<size_t>(chunk) * row_halfs, "cudaMalloc (decoded weights)")))
    return rc;
  for (int tr0 = 0; tr0 < NT; tr0 += chunk) {
    const int tr1 = std::min(NT, tr0 + chunk);
    rc = reads_pairs(mx, 1) ? launch_decode_weights_rows(mx.pair, M->d_w16, tr0, tr1, st) : kErrTooLarge;   // two weights per lookup
    if (rc == kErrTooLarge) rc = launch_decode_weights_rows(mx.dev, M->d_w16, tr0, tr1, st);
    if (rc) return rc;
    if ((rc = launch_gemm_tc(x16, M->d_w16, y + static_cast<size_t>(tr0) * kTileRows, m, (tr1 - tr0) * kTileRows, mx.K,
                             ldy, M->d_partials, M->partial_floats, unscale, st)))
      return rc;
  }
  return kOk;
}

int linear_device(Model* M, Matrix& mx, const void* x, bool x_half, int m, float* y, int ldy, cudaStream_t st,
                  int path) {
  if (const int rc = check_device(M)) return rc;
  if (mx.fmt == kFmtNone) {
    set_error("%s has no side tensor: products need a block format", mx.name.c_str());
    return kErrArg;
  }
  // path 0: up to eight rows the fused decode + product kernels; 9 .. 64 rows the decode + tcgen05 GEMM (decoded weights
  // go to tensor memory, never to DRAM); more rows, or shapes that kernel does not take, decode to fp16 weights in DRAM
  // and a tensor-core GEMM over them (the decode is paid once however many rows follow).  path 3 forces the tcgen05 kernel.
  if (path == 3 || (path == 0 && m >= debug_knobs().t5_min_rows && m <= 64)) {
    if (!x_half) {   // range factors of the rows, once for whichever layout takes the product
      if (const int rc = grow(&M->d_row_scale, &M->row_scale_floats, 128, "cudaMalloc (row factors)")) return rc;
      if (const int rc = launch_row_scales(static_cast<const float*>(x), m, mx.K, M->d_row_scale, st)) return rc;
    }
    int rc = kErrTooLarge;
    if (reads_pairs(mx, 1))   // two weights per lookup; falls through where the larger units leave no room
      rc = launch_gemm_coded(mx.pair, x, x_half, m, y, ldy, M->d_partials, M->partial_floats, M->d_row_scale, st);
    if (rc == kErrTooLarge) rc = launch_gemm_coded(mx.dev, x, x_half, m, y, ldy, M->d_partials, M->partial_floats, M->d_row_scale, st);
    if (rc != kErrTooLarge || path == 3) return rc;
  }
  if (path == 2 || (path == 0 && m > 16)) return linear_decode_gemm(M, mx, x, x_half, m, y, ldy, st);
  const size_t xe = x_half ? 2 : 4;
  for (int r0 = 0; r0 < m; r0 += 8) {
    const int mm = std::min(8, m - r0);
    const bool pr = reads_pairs(mx, mm);
    const void* xr = static_cast<const uint8_t*>(x) + static_cast<size_t>(r0) * mx.K * xe;
    float* yr = y + static_cast<size_t>(r0) * ldy;
    int rc = pr ? launch_gemv(mx.pair, xr, x_half, mm, yr, ldy, M->d_partials, M->partial_floats, st, &mx.pair_epoch) : kErrTooLarge;
    if (rc == kErrTooLarge)   // no pair layout, or its larger units do not fit this kernel's shared memory
      rc = launch_gemv(mx.dev, xr, x_half, mm, yr, ldy, M->d_partials, M->partial_floats, st, &mx.clean_epoch);
    if (rc) return rc;
  }
  return kOk;
}

int linear_batch_device(Model* M, int n, const int* mat_index, const float* const* xs, float* const* ys, cudaStream_t st) {
  if (n < 1 || n > 8) return kErrArg;
  const MatDev* mats[8];
  const void* xv[8];
  float* partials[8];
  unsigned int* epochs[8];
  size_t off = 0;
  for (int j = 0; j < n; ++j) {
    Matrix& mx = M->mats[mat_index[j]];
    if (mx.fmt == kFmtNone || !gemv1_usable(mx.dev)) {
      set_error("%s has no side tensor: products need a block format", mx.name.c_str());
      return kErrArg;
    }
    const size_t need = (gemv_partial_floats(mx.dev, 1) + 63) & ~size_t(63);
    if (off + need > M->partial_floats) return kErrTooLarge;
    mats[j] = reads_pairs(mx, 1) ? &mx.pair : &mx.dev;
    xv[j] = xs[j];
    partials[j] = M->d_partials + off;
    epochs[j] = reads_pairs(mx, 1) ? &mx.pair_epoch : &mx.clean_epoch;
    off += need;
  }
  return launch_gemv_batch(n, mats, xv, false, ys, partials, st, epochs);
}

}  // namespace lw

using namespace lw;

extern "C" {

const char* lw_last_error(void) { return last_error(); }

int lw_last_status(void) { return last_status(); }

int lw_kernel_error(void) {
  unsigned int v = 0;
  if (read_kernel_error(&v, true)) return kErrCuda;
  return static_cast<int>(v);
}

long long lw_launch_count(void) { return launch_count(); }

int lw_debug_set(const char* key, long long value) {
  if (!key) return kErrArg;
  DebugKnobs& k = debug_knobs();
  const std::string s(key);
  if (s == "max_units" && value >= 2 && value <= 1024) k.max_units = static_cast<int>(value) & ~1;
  else if (s == "wait_limit" && value >= 1 && value <= (1ll << 30)) k.wait_limit = static_cast<uint32_t>(value);
  else if (s == "drop_unit" && value >= -1 && value < 1024) k.drop_unit = static_cast<int>(value);
  else if (s == "t5_min_rows" && value >= 1 && value <= 65) k.t5_min_rows = static_cast<int>(value);
  else if (s == "pairs" && (value == 0 || value == 1)) k.pairs = static_cast<int>(value);
  else if (s == "reset") k = DebugKnobs();
  else {
    set_error("lw_debug_set: unknown key or value out of range (%s)", key);
    return kErrArg;
  }
  return kOk;
}

int lw_debug_wait_probe(long long limit) {
  if (limit < 1 || limit > (1ll << 22)) return kErrArg;
  int dev = 0;
  int rc = require_device(&dev);
  if (rc) return rc;
  int gave_up = 0;
  if ((rc = launch_wait_probe(static_cast<unsigned int>(limit), &gave_up))) return rc;
  return gave_up;
}

void rt_close(void* handle) { delete static_cast<Model*>(handle); }

void* rt_open(const char* dir, int max_ctx, int max_batch, long long budget_mb, int floor_mb, int verbose) {
  (void)max_ctx; (void)max_batch; (void)budget_mb; (void)floor_mb;
  note_status(kOk);
  if (!dir) {
    set_error("rt_open: null directory");
    note_status(kErrArg);
    return nullptr;
  }
  auto M = std::make_unique<Model>();
  M->dir = dir;
  M->verbose = verbose != 0;
  if (note_status(read_manifest(M->dir, M->man))) return nullptr;
  if (M->man.cfg.count("n_layers") && note_status(validate_model(M->man))) return nullptr;
  M->fd = open((M->dir + "/weights.bin").c_str(), O_RDONLY);
  if (M->fd < 0) {
    set_error("cannot open %s/weights.bin", dir);
    note_status(kErrGeneric);
    return nullptr;
  }
  if (note_status(require_device(&M->device))) return nullptr;
  const auto t0 = std::chrono::steady_clock::now();
  const int threads = default_threads();
  std::vector<uint8_t> blob, side;
  std::map<std::tuple<long long, long long, int, long long>, HostImage> images;
  for (const TensorEntry& t : M->man.tensors) {
    if (t.enc != "huf8" && t.enc != "huf4p") continue;
    Matrix mx;
    mx.name = t.name;
    mx.N = t.N;
    mx.K = t.K;
    mx.paired = t.enc == "huf4p";
    mx.Ks = mx.paired ? t.K / 2 : t.K;
    mx.blob_bytes = t.nbytes;
    mx.file_offset = t.offset;
    if (mx.paired && t.K % 2) {
      set_error("%s: odd K for a paired matrix", t.name.c_str());
      note_status(kErrFormat);
      return nullptr;
    }
    if (note_status(read_blob(M->fd, t, blob))) return nullptr;
    const TensorEntry* s = M->man.find(t.name + ".kqs");
    size_t sbytes = 0;
    if (s) {
      mx.fmt = format_of_side_enc(s->enc);
      if (mx.fmt == kFmtNone || is_paired(mx.fmt) != mx.paired || s->N != t.N) {
        set_error("%s: side tensor %s does not fit a %s matrix", t.name.c_str(), s->enc.c_str(), t.enc.c_str());
        note_status(kErrFormat);
        return nullptr;
      }
      if (note_status(read_blob(M->fd, *s, side))) return nullptr;
      sbytes = static_cast<size_t>(s->nbytes);
      mx.side_bytes = s->nbytes;
    }
    // several tensors may share one blob in the file (synthetic models reuse a layer): prepare it once
    const auto key = std::make_tuple(t.offset, t.nbytes, mx.fmt, s ? s->offset : -1ll);
    auto hit = images.find(key);
    if (hit == images.end()) {
      HostImage im;
      if (note_status(prepare_matrix(mx, blob.data(), static_cast<size_t>(t.nbytes), s ? side.data() : nullptr, sbytes,
                                     threads, im)))
        return nullptr;
      if (images.size() >= 16) images.clear();
      hit = images.emplace(key, std::move(im)).first;
    }
    if (note_status(upload_matrix(mx, hit->second, s ? side.data() : nullptr, sbytes))) {
      if (mx.d_block) cudaFree(mx.d_block);
      return nullptr;
    }
    M->by_name[mx.name] = static_cast<int>(M->mats.size());
    M->mats.push_back(std::move(mx));
  }
  if (note_status(finish_model(M.get()))) return nullptr;
  if (verbose) {
    const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    fprintf(stderr, "[lwb200] %s: %zu coded matrices, %.1f MB coded + %.1f MB side, %.1f MB on device, load %.2f s\n",
            dir, M->mats.size(), M->coded_bytes / 1e6, M->side_bytes / 1e6, M->resident_bytes / 1e6, s);
  }
  // a bundle with model configuration also gets the decoder runtime (activations, KV cache, norms, rotary tables)
  if (M->man.cfg.count("n_layers") && note_status(runtime_init(M.get(), max_ctx, max_batch))) return nullptr;
  return M.release();
}

void* lw_matrix_create(const uint8_t* blob, long long blob_bytes, int N, int Ks, int fmt, const uint8_t* side,
                       long long side_bytes) {
  if (!blob || blob_bytes <= 0 || fmt < kFmtNone || fmt > kFmtIQ4XS) {
    set_error("lw_matrix_create: bad argument");
    note_status(kErrArg);
    return nullptr;
  }
  note_status(kOk);
  auto M = std::make_unique<Model>();
  if (note_status(require_device(&M->device))) return nullptr;
  Matrix mx;
  mx.name = "m";
  mx.N = N;
  mx.Ks = Ks;
  mx.fmt = fmt;
  mx.paired = fmt != kFmtNone && is_paired(fmt);
  mx.K = mx.paired ? 2 * Ks : Ks;
  mx.blob_bytes = blob_bytes;
  mx.side_bytes = fmt != kFmtNone ? side_bytes : 0;
  std::vector<uint8_t> copy(static_cast<size_t>(blob_bytes) + 16, 0);   // the walker reads 8 bytes at a time
  std::memcpy(copy.data(), blob, static_cast<size_t>(blob_bytes));
  if (note_status(load_matrix(mx, copy.data(), static_cast<size_t>(blob_bytes), fmt != kFmtNone ? side : nullptr,
                              fmt != kFmtNone ? static_cast<size_t>(side_bytes) : 0, default_threads()))) {
    if (mx.d_block) cudaFree(mx.d_block);
    return nullptr;
  }
  M->by_name[mx.name] = 0;
  M->mats.push_back(std::move(mx));
  if (note_status(finish_model(M.get()))) return nullptr;
  return M.release();
}

int lw_matrix_id(void* handle, const char* name) { return matrix_id(static_cast<Model*>(handle), name); }

int lw_matrix_info(void* handle, int id, int* N, int* K, int* fmt, long long* blob_bytes, long long* side_bytes,
                   long long* device_bytes) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return kErrGeneric;
  if (N) *N = mx->N;
  if (K) *K = mx->K;
  if (fmt) *fmt = mx->fmt;
  if (blob_bytes) *blob_bytes = mx->blob_bytes;
  if (side_bytes) *side_bytes = mx->side_bytes;
  if (device_bytes) *device_bytes = static_cast<long long>(mx->device_bytes);
  return kOk;
}

int lw_matrix_plan(void* handle, int id, int* group, int* index_bits, double* slow_fraction) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return kErrGeneric;
  if (group) *group = mx->dev.group;
  if (index_bits) *index_bits = mx->dev.group ? mx->dev.index_bits : 0;
  if (slow_fraction) *slow_fraction = mx->slow_fraction;
  return kOk;
}

int lw_linear(void* handle, int id, const void* x_dev, int x_is_half, int m, float* y_dev, void* stream) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return kErrGeneric;
  if (!x_dev || !y_dev || m < 1) {
    set_error("lw_linear: bad argument");
    return kErrArg;
  }
  return linear_device(static_cast<Model*>(handle), *mx, x_dev, x_is_half != 0, m, y_dev, mx->N,
                       static_cast<cudaStream_t>(stream));
}

int lw_linear_batch(int n, void* const* handles, const int* ids, const void* const* xs_dev, int x_is_half,
                    float* const* ys_dev, void* stream) {
  if (n < 1 || !handles || !ids || !xs_dev || !ys_dev) {
    set_error("lw_linear_batch: bad argument");
    return kErrArg;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  constexpr int kChunk = 8;
  for (int i0 = 0; i0 < n; i0 += kChunk) {
    const int c = std::min(kChunk, n - i0);
    const MatDev* mats[kChunk];
    float* partials[kChunk];
    unsigned int* epochs[kChunk];
    std::map<Model*, size_t> used;   // scratch already handed out per handle within this chunk
    for (int j = 0; j < c; ++j) {
      Model* M = static_cast<Model*>(handles[i0 + j]);
      Matrix* mx = matrix_by_id(M, ids[i0 + j]);
      if (!mx) return kErrGeneric;
      if (const int rc = check_device(M)) return rc;
      if (!xs_dev[i0 + j] || !ys_dev[i0 + j] || mx->fmt == kFmtNone || !gemv1_usable(mx->dev)) {
        set_error("lw_linear_batch: entry %d: null pointer or a matrix without block format", i0 + j);
        return kErrArg;
      }
      size_t& off = used[M];
      const size_t need = (gemv_partial_floats(mx->dev, 1) + 63) & ~size_t(63);
      if (off + need > M->partial_floats) {
        set_error("lw_linear_batch: the products of one handle need more scratch than the handle holds");
        return kErrTooLarge;
      }
      mats[j] = reads_pairs(*mx, 1) ? &mx->pair : &mx->dev;
      partials[j] = M->d_partials + off;
      epochs[j] = reads_pairs(*mx, 1) ? &mx->pair_epoch : &mx->clean_epoch;
      off += need;
    }
    const int rc = launch_gemv_batch(c, mats, xs_dev + i0, x_is_half != 0, ys_dev + i0, partials, st, epochs);
    if (rc) return rc;
  }
  return kOk;
}

int lw_matrix_make_twin(void* handle, int id) {
  Model* M = static_cast<Model*>(handle);
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return kErrGeneric;
  if (mx->d_twin) return kOk;
  int rc = check_device(M);
  if (rc) return rc;
  if (mx->fmt == kFmtNone || !gemv1_usable(mx->dev)) {
    set_error("%s: no block format, no twin", mx->name.c_str());
    return kErrArg;
  }
  // the symbols come from the GPU decoder (bit-exact against the host decoder by the parity tests)
  const size_t nsym = static_cast<size_t>(mx->N) * mx->Ks;
  uint8_t* d_sym = nullptr;
  cudaError_t e = cudaMalloc(&d_sym, nsym);
  if (e != cudaSuccess) return cuda_fail("cudaMalloc (twin symbols)", e);
  std::vector<uint8_t> sym(nsym), side(static_cast<size_t>(mx->side_bytes));
  rc = launch_decode_codes(mx->dev, d_sym, false, nullptr);
  if (!rc && ((e = cudaMemcpy(sym.data(), d_sym, nsym, cudaMemcpyDeviceToHost)) != cudaSuccess ||
              (e = cudaMemcpy(side.data(), mx->dev.side, side.size(), cudaMemcpyDeviceToHost)) != cudaSuccess))
    rc = cuda_fail("cudaMemcpy (twin symbols)", e);
  cudaFree(d_sym);
  if (rc) return rc;
  std::vector<uint32_t> gb, words, vals(256);
  uint32_t unit_words = 0;
  if ((rc = build_twin(sym.data(), mx->N, mx->Ks, mx->fmt, side.data(), default_threads(), gb, words, &unit_words))) return rc;
  symbol_values(mx->fmt, vals.data());
  const size_t n_units = gb.size() / 2;
  const size_t off_gb = align_up(256 * 4, 256), off_words = align_up(off_gb + gb.size() * 4, 256);
  const size_t off_cls = align_up(off_words + words.size() * 4, 256), off_done = off_cls + align_up(n_units, 256);
  const size_t total = off_done + align_up(static_cast<size_t>(mx->N / kTileRows) * kRowDoneStride * 4, 256);
  if ((e = cudaMalloc(&mx->d_twin, total)) != cudaSuccess) return cuda_fail("cudaMalloc (twin)", e);
  uint8_t* d = static_cast<uint8_t*>(mx->d_twin);
  if ((e = cudaMemset(d, 0, total)) != cudaSuccess || (e = cudaMemcpy(d, vals.data(), 1024, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_gb, gb.data(), gb.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (e = cudaMemcpy(d + off_words, words.data(), words.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess) {
    cudaFree(mx->d_twin);
    mx->d_twin = nullptr;
    return cuda_fail("cudaMemcpy (twin)", e);
  }
  mx->twin = mx->dev;
  mx->twin.reader = 1;
  mx->twin.tab32 = reinterpret_cast<const uint32_t*>(d);
  mx->twin.cmp_tab = nullptr;
  mx->twin.symtab32 = nullptr;
  mx->twin.group_base = reinterpret_cast<const uint32_t*>(d + off_gb);
  mx->twin.words = reinterpret_cast<const uint32_t*>(d + off_words);
  mx->twin.unit_slow = d + off_cls;
  mx->twin.row_done = reinterpret_cast<unsigned int*>(d + off_done);
  mx->twin.index_bits = 10;
  mx->twin.group = 3;
  mx->twin.max_unit_words = unit_words;
  mx->twin.max_tile_words = unit_words * mx->dev.split;
  mx->twin_bytes = (words.size() - kTailWords) * 4;
  mx->twin_epoch = 0;
  return kOk;
}

long long lw_matrix_twin_bytes(void* handle, int id) {
  Matrix* mx = matrix_by_id(handle, id);
  return mx && mx->d_twin ? static_cast<long long>(mx->twin_bytes) : -1;
}

int lw_matrix_drop_twin(void* handle, int id) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return kErrGeneric;
  if (mx->d_twin) {
    cudaDeviceSynchronize();
    cudaFree(mx->d_twin);
    mx->d_twin = nullptr;
    mx->twin_bytes = 0;
  }
  return kOk;
}

int lw_linear_twin(void* handle, int id, const void* x_dev, int x_is_half, float* y_dev, void* stream) {
  Model* M = static_cast<Model*>(handle);
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return kErrGeneric;
  if (!mx->d_twin || !x_dev || !y_dev) {
    set_error("lw_linear_twin: no twin (call lw_matrix_make_twin) or bad argument");
    return kErrArg;
  }
  if (const int rc = check_device(M)) return rc;
  return launch_gemv(mx->twin, x_dev, x_is_half != 0, 1, y_dev, mx->N, M->d_partials, M->partial_floats,
                     static_cast<cudaStream_t>(stream), &mx->twin_epoch);
}

int lw_decode_weights(void* handle, int id, void* w_half_dev, void* stream) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return kErrGeneric;
  if (!w_half_dev) return kErrArg;
  if (const int rc = check_device(static_cast<Model*>(handle))) return rc;
  int rc = reads_pairs(*mx, 1) ? launch_decode_weights(mx->pair, static_cast<__half*>(w_half_dev), static_cast<cudaStream_t>(stream))
                               : kErrTooLarge;
  if (rc == kErrTooLarge) rc = launch_decode_weights(mx->dev, static_cast<__half*>(w_half_dev), static_cast<cudaStream_t>(stream));
  return rc;
}

int lw_decode_codes(void* handle, int id, uint8_t* out_dev, int expand, void* stream) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return kErrGeneric;
  if (!out_dev) return kErrArg;
  if (const int rc = check_device(static_cast<Model*>(handle))) return rc;
  return decode_codes_of(*mx, out_dev, expand != 0, static_cast<cudaStream_t>(stream));
}

int rt_test_matmul(void* handle, const char* name, const float* X, int m, float* Y, int path) {
  Model* M = static_cast<Model*>(handle);
  const int id = matrix_id(M, name);
  if (id < 0) return -1;
  Matrix& mx = M->mats[id];
  if (!X || !Y || m < 1 || path < 0 || path > 3) {
    set_error("rt_test_matmul: bad argument");
    return kErrArg;
  }
  cudaError_t e;
  const size_t nx = static_cast<size_t>(m) * mx.K, ny = static_cast<size_t>(m) * mx.N;
  if (nx > M->x_floats) {
    if (M->d_x) cudaFree(M->d_x);
    M->d_x = nullptr;
    M->x_floats = 0;
    if ((e = cudaMalloc(&M->d_x, nx * 4)) != cudaSuccess) return cuda_fail("rt_test_matmul buffers", e);
    M->x_floats = nx;
  }
  if (ny > M->y_floats) {
    if (M->d_y) cudaFree(M->d_y);
    M->d_y = nullptr;
    M->y_floats = 0;
    if ((e = cudaMalloc(&M->d_y, ny * 4)) != cudaSuccess) return cuda_fail("rt_test_matmul buffers", e);
    M->y_floats = ny;
  }
  // Host buffers go through one pinned staging area with asynchronous copies on the stream of the product and a
  // single synchronisation: two blocking copies from pageable memory cost about 10 us more per call.
  if (nx + ny > M->pin_floats) {
    if (M->h_pin) cudaFreeHost(M->h_pin);
    M->h_pin = nullptr;
    M->pin_floats = 0;
    if ((e = cudaMallocHost(&M->h_pin, (nx + ny) * 4)) != cudaSuccess) return cuda_fail("rt_test_matmul pinned buffer", e);
    M->pin_floats = nx + ny;
  }
  std::memcpy(M->h_pin, X, nx * 4);
  if ((e = cudaMemcpyAsync(M->d_x, M->h_pin, nx * 4, cudaMemcpyHostToDevice, nullptr)) != cudaSuccess)
    return cuda_fail("rt_test_matmul copy in", e);
  // A small result is written by the kernels straight into the pinned buffer (it is mapped into the device's address
  // space): no copy-back to enqueue and wait for.  Large results go through device memory and one copy.
  const bool direct = ny * 4 <= (size_t(1) << 20);
  int rc = linear_device(M, mx, M->d_x, false, m, direct ? M->h_pin + nx : M->d_y, mx.N, nullptr, path);
  if (!rc && !direct && (e = cudaMemcpyAsync(M->h_pin + nx, M->d_y, ny * 4, cudaMemcpyDeviceToHost, nullptr)) != cudaSuccess)
    rc = cuda_fail("rt_test_matmul copy back", e);
  if ((e = cudaStreamSynchronize(nullptr)) != cudaSuccess && !rc) rc = cuda_fail("rt_test_matmul", e);
  if (!rc) std::memcpy(Y, M->h_pin + nx, ny * 4);
  return rc;
}

int rt_test_decode(void* handle, const char* name, uint8_t* out) {
  Model* M = static_cast<Model*>(handle);
  const int id = matrix_id(M, name);
  if (id < 0) return -1;
  Matrix& mx = M->mats[id];
  if (!out) return kErrArg;
  if (const int rc = check_device(M)) return rc;
  const size_t n = static_cast<size_t>(mx.N) * mx.K;
  uint8_t* d = nullptr;
  cudaError_t e = cudaMalloc(&d, n);
  if (e != cudaSuccess) return cuda_fail("rt_test_decode buffer", e);
  int rc = decode_codes_of(mx, d, true, nullptr);
  if (!rc && (e = cudaMemcpy(out, d, n, cudaMemcpyDeviceToHost)) != cudaSuccess) rc = cuda_fail("rt_test_decode copy", e);
  cudaFree(d);
  return rc;
}

static int cpu_decode_entry(Model* M, const Matrix& mx, int threads, uint8_t* out, double* seconds) {
  const TensorEntry* t = M->man.find(mx.name);
  if (!t) {
    set_error("%s was not loaded from a bundle directory", mx.name.c_str());
    return kErrGeneric;
  }
  std::vector<uint8_t> blob;
  int rc = read_blob(M->fd, *t, blob);
  if (rc) return rc;
  BlobView v;
  if ((rc = make_view(blob.data(), static_cast<size_t>(t->nbytes), mx.N, mx.Ks, v))) return rc;
  auto tab = std::make_unique<HuffTable>();
  if ((rc = table_from_lut(v.lut(), *tab))) return rc;
  const auto t0 = std::chrono::steady_clock::now();
  rc = walk_blob(v, *tab, 1, std::max(1, threads), nullptr, nullptr, out);
  if (seconds) *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  return rc;
}

int rt_test_cpu_decode(void* handle, const char* name, int threads, uint8_t* out) {
  Model* M = static_cast<Model*>(handle);
  const int id = matrix_id(M, name);
  if (id < 0) return -1;
  if (!out) return kErrArg;
  return cpu_decode_entry(M, M->mats[id], threads, out, nullptr);
}

double rt_cpu_decode_all(void* handle, int threads, long long* symbols) {
  Model* M = static_cast<Model*>(handle);
  if (!M) return -1;
  double total = 0;
  long long nsym = 0;
  std::vector<uint8_t> out;
  for (auto& mx : M->mats) {
    out.resize(static_cast<size_t>(mx.N) * mx.Ks);
    double s = 0;
    if (cpu_decode_entry(M, mx, threads, out.data(), &s)) return -1;
    total += s;
    nsym += static_cast<long long>(mx.N) * mx.Ks;
  }
  if (symbols) *symbols = nsym;
  return total;
}

double rt_gpu_decode_all(void* handle, int reps) {
  Model* M = static_cast<Model*>(handle);
  if (!M || reps < 1 || check_device(M)) return -1;
  size_t cap = 0;
  for (auto& mx : M->mats) cap = std::max(cap, static_cast<size_t>(mx.N) * mx.K);
  uint8_t* scratch = nullptr;
  if (cudaMalloc(&scratch, std::max<size_t>(cap, 16)) != cudaSuccess) {
    cuda_fail("rt_gpu_decode_all scratch", cudaGetLastError());
    return -1;
  }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  std::vector<double> secs;
  bool ok = true;
  for (int r = 0; r < reps && ok; ++r) {
    cudaEventRecord(e0);
    for (auto& mx : M->mats)
      if (decode_codes_of(mx, scratch, true, nullptr)) ok = false;
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) ok = false;
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    secs.push_back(ms / 1e3);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(scratch);
  if (!ok) return -1;
  std::sort(secs.begin(), secs.end());
  return secs[secs.size() / 2];
}

double rt_stat(void* handle, const char* key) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !key) return -1;
  const std::string k(key);
  if (k == "resident_bytes") return static_cast<double>(M->resident_bytes);
  if (k == "coded_bytes") return static_cast<double>(M->coded_bytes);
  if (k == "side_bytes") return static_cast<double>(M->side_bytes);
  if (k == "n_matrices") return static_cast<double>(M->mats.size());
  if (k == "graph_launches" || k == "graph_captures" || k == "collective_us" || k == "collective_calls" ||
      k == "time_collectives")
    return runtime_stat(M, k.c_str());
  if (k == "streamed_bytes" || k == "n_streamed" || k == "stream_wait_s" || k == "stream_bytes_moved") return 0;
  return -1;
}

long long lw_encode_huf8(const uint8_t* sym, int N, int Ks, uint8_t* out, long long cap, long long* nbits) {
  if (!sym) {
    set_error("lw_encode_huf8: null input");
    return kErrArg;
  }
  std::vector<uint8_t> blob;
  int64_t bits = 0;
  const int rc = encode_huf8(sym, N, Ks, blob, &bits, kMaxLen, default_threads());   // the bytes do not depend on the threads
  if (rc) return rc;
  if (nbits) *nbits = bits;
  if (out && cap >= static_cast<long long>(blob.size())) std::memcpy(out, blob.data(), blob.size());
  return static_cast<long long>(blob.size());
}

static int host_view(const uint8_t* blob, long long nbytes, int N, int Ks, std::vector<uint8_t>& copy, BlobView& v,
                     HuffTable& tab) {
  if (!blob || nbytes <= 0) {
    set_error("null or empty blob");
    return kErrArg;
  }
  copy.assign(static_cast<size_t>(nbytes) + 16, 0);
  std::memcpy(copy.data(), blob, static_cast<size_t>(nbytes));
  int rc = make_view(copy.data(), static_cast<size_t>(nbytes), N, Ks, v);
  if (rc) return rc;
  return table_from_lut(v.lut(), tab);
}

long long lw_host_layout(const uint8_t* blob, long long blob_bytes, int N, int Ks, int fmt, const uint8_t* side,
                         long long side_bytes, int* info, uint32_t* group_base, long long group_base_cap,
                         uint32_t* words, long long words_cap, uint8_t* unit_class, long long unit_class_cap) {
  if (!blob || blob_bytes <= 0 || !info || fmt < kFmtNone || fmt > kFmtIQ4XS) {
    set_error("lw_host_layout: bad argument");
    return kErrArg;
  }
  Matrix mx;
  mx.name = "m";
  mx.N = N;
  mx.Ks = Ks;
  mx.fmt = fmt;
  mx.paired = is_paired(fmt);
  mx.K = mx.paired ? 2 * Ks : Ks;
  std::vector<uint8_t> copy(static_cast<size_t>(blob_bytes) + 16, 0);   // the walk reads 8 bytes at a time
  std::memcpy(copy.data(), blob, static_cast<size_t>(blob_bytes));
  HostImage im;
  const int rc = prepare_matrix(mx, copy.data(), static_cast<size_t>(blob_bytes), side,
                                static_cast<size_t>(std::max(0ll, side_bytes)), default_threads(), im);
  if (rc) return rc;
  info[0] = im.split;
  info[1] = im.pad;
  info[2] = im.unit_slow.empty() ? 0 : im.group;
  info[3] = im.index_bits;
  info[4] = static_cast<int>(im.group_base.size());
  info[5] = static_cast<int>(im.unit_slow.size());
  info[6] = im.unit_slow.empty() ? 0 : unit_side_words(fmt);
  info[7] = static_cast<int>(im.max_unit);
  if (group_base && group_base_cap >= static_cast<long long>(im.group_base.size()))
    std::memcpy(group_base, im.group_base.data(), im.group_base.size() * 4);
  if (words && words_cap >= static_cast<long long>(im.words.size()))
    std::memcpy(words, im.words.data(), im.words.size() * 4);
  if (unit_class && unit_class_cap >= static_cast<long long>(im.unit_slow.size()) && !im.unit_slow.empty())
    std::memcpy(unit_class, im.unit_slow.data(), im.unit_slow.size());
  return static_cast<long long>(im.words.size());
}

int lw_host_layout_table(const uint8_t* blob, long long blob_bytes, int N, int Ks, int fmt, const uint8_t* side,
                         long long side_bytes, uint16_t* lut) {
  if (!blob || blob_bytes <= 0 || !lut || fmt < kFmtNone || fmt > kFmtIQ4XS) {
    set_error("lw_host_layout_table: bad argument");
    return kErrArg;
  }
  Matrix mx;
  mx.name = "m";
  mx.N = N;
  mx.Ks = Ks;
  mx.fmt = fmt;
  mx.paired = is_paired(fmt);
  mx.K = mx.paired ? 2 * Ks : Ks;
  std::vector<uint8_t> copy(static_cast<size_t>(blob_bytes) + 16, 0);   // the walk reads 8 bytes at a time
  std::memcpy(copy.data(), blob, static_cast<size_t>(blob_bytes));
  HostImage im;
  const int rc = prepare_matrix(mx, copy.data(), static_cast<size_t>(blob_bytes), side,
                                static_cast<size_t>(std::max(0ll, side_bytes)), default_threads(), im);
  if (rc) return rc;
  std::memcpy(lut, im.lut.data(), 2 * kLutSize);
  return im.max_len;
}

long long lw_host_pairs(const uint8_t* codes, int N, int K, int fmt, const uint8_t* side, long long side_bytes_n, int* info,
                        uint32_t* table, long long table_cap, uint32_t* group_base, long long group_base_cap,
                        uint32_t* words, long long words_cap) {
  if (!codes || !info || !side || side_bytes_n != static_cast<long long>(N) * (K / 256) * side_bytes(fmt)) {
    set_error("lw_host_pairs: bad argument");
    return kErrArg;
  }
  PairImage p;
  const int rc = build_pairs(codes, N, K, fmt, side, default_threads(), p);
  if (rc) return rc;
  info[0] = p.split;
  info[1] = p.pad;
  info[2] = p.group;
  info[3] = p.index_bits;
  info[4] = static_cast<int>(p.group_base.size());
  info[5] = p.max_len;
  info[6] = unit_side_words(p.fmt);
  info[7] = static_cast<int>(p.max_unit_words);
  if (table && table_cap >= static_cast<long long>(p.tab32.size())) std::memcpy(table, p.tab32.data(), p.tab32.size() * 4);
  if (group_base && group_base_cap >= static_cast<long long>(p.group_base.size()))
    std::memcpy(group_base, p.group_base.data(), p.group_base.size() * 4);
  if (words && words_cap >= static_cast<long long>(p.words.size())) std::memcpy(words, p.words.data(), p.words.size() * 4);
  return static_cast<long long>(p.words.size());
}

long long lw_matrix_pair_bytes(void* handle, int id) {
  Matrix* mx = matrix_by_id(handle, id);
  if (!mx) return -1;
  return mx->d_pair ? static_cast<long long>(mx->pair_bytes) : 0;
}

int lw_validate_bundle(const char* dir) {
  if (!dir) return kErrArg;
  Manifest man;
  int rc = read_manifest(dir, man);
  if (rc) return rc;
  const int fd = open((std::string(dir) + "/weights.bin").c_str(), O_RDONLY);
  if (fd < 0) {
    set_error("cannot open %s/weights.bin", dir);
    return kErrGeneric;
  }
  const off_t size = lseek(fd, 0, SEEK_END);
  close(fd);
  for (const TensorEntry& t : man.tensors)
    if (t.offset + t.nbytes > size) {
      set_error("tensor %s reaches past the end of weights.bin", t.name.c_str());
      return kErrFormat;
    }
  return man.cfg.count("n_layers") ? validate_model(man) : kOk;
}

int lw_validate_blob(const uint8_t* blob, long long blob_bytes, int N, int Ks) {
  std::vector<uint8_t> copy;
  BlobView v;
  auto tab = std::make_unique<HuffTable>();
  int rc = host_view(blob, blob_bytes, N, Ks, copy, v, *tab);
  if (rc) return rc;
  return walk_blob(v, *tab, 1, default_threads(), nullptr, nullptr, nullptr);
}

int lw_cpu_decode(const uint8_t* blob, long long blob_bytes, int N, int Ks, int threads, uint8_t* out) {
  if (!out) return kErrArg;
  std::vector<uint8_t> copy;
  BlobView v;
  auto tab = std::make_unique<HuffTable>();
  int rc = host_view(blob, blob_bytes, N, Ks, copy, v, *tab);
  if (rc) return rc;
  return walk_blob(v, *tab, 1, std::max(1, threads), nullptr, nullptr, out);
}

}  // extern "C"
