// CUDA kernels (sm_100a) of the coded-weight path and their launchers.
//
//   k_decode_codes    chain groups -> uint8 codes [N, K]           (role of k_decode_hufi, kernels/llmrt.cu:767-806)
//   k_decode_weights  chain groups + side bytes -> fp16 [N, K]     (decode fused with the block dequantisation)
//   k_sum_partials    ordered sum over tile columns                (role of k_sum_kt, kernels/llmrt.cu:1173-1180)
//
// The fused decode + product kernels live in lw_gemv1.cu (one row) and lw_gemvm.cu (2..8 rows); this file dispatches
// to them (launch_gemv, the role of matmul(), kernels/llmrt.cu:1794-1826).
//
// Common shape of the two decode kernels here: one warp owns one 64 x 256-symbol tile.  Lane l decodes tile rows l and l + 32 as two independent
// chains.  The tile's interleaved words are staged into shared memory by one bulk copy (cp.async.bulk, completion
// on an mbarrier) issued by lane 0; the lanes then read their next words from shared memory, bank = lane.
#include "lw_kernels.h"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include <cuda.h>
#include <cudaTypedefs.h>

#include "lw_ring.cuh"
#include "lw_gemv1.h"

namespace lw {

// Error word set by kernels that give up on a wait instead of spinning for ever (bit 0: bulk-copy wait timed out).
__device__ unsigned int g_kernel_error;

constexpr int kWarpsPerBlock = 8;
constexpr int kSlackWords = 96;   // read-ahead of the last chains of a tile lands here

__host__ __device__ constexpr uint32_t tile_buf_words(uint32_t max_tile_words) {
  return (max_tile_words + kSlackWords + 31u) & ~31u;
}

// Stages tile t into `buf` and returns false if the copy did not land in time.
__device__ __forceinline__ bool stage_tile(const MatDev& M, int t, uint32_t* buf, uint64_t* bar, int lane,
                                           uint32_t* tile_base) {
  const int G = 2 * M.split;
  const uint32_t b0 = __ldg(M.group_base + static_cast<size_t>(t) * G);
  const uint32_t b1 = __ldg(M.group_base + static_cast<size_t>(t + 1) * G);
  *tile_base = b0;
  const uint32_t bar_a = smem_addr(bar);
  if (lane == 0) {
    mbar_init(bar_a, 1);
    bulk_load(smem_addr(buf), M.words + b0, (b1 - b0) * 4u, bar_a);
  }
  __syncwarp();
  return mbar_wait(bar_a, 0, &g_kernel_error);
}

// ------------------------------------------------------------------------------------------------ decode to codes

template <bool EXPAND>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) k_decode_codes(MatDev M, uint8_t* __restrict__ out) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint16_t* lut = reinterpret_cast<uint16_t*>(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * kLutSize);
  uint32_t* bufs = reinterpret_cast<uint32_t*>(smem + 2 * kLutSize + 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kLutSize / 2; i += blockDim.x)
    reinterpret_cast<uint32_t*>(lut)[i] = __ldg(reinterpret_cast<const uint32_t*>(M.lut) + i);
  __syncthreads();
  const int t = blockIdx.x * kWarpsPerBlock + warp;
  if (t >= M.T) return;
  uint32_t* buf = bufs + static_cast<size_t>(warp) * tile_buf_words(M.max_tile_words);
  uint32_t base;
  if (!stage_tile(M, t, buf, bars + warp, lane, &base)) return;
  const int tr = t / M.KT, tc = t - tr * M.KT;
  const int row_bytes = EXPAND ? 2 * M.Ks : M.Ks;
  const int tile_bytes = EXPAND ? 2 * kTileSyms : kTileSyms;
#pragma unroll 1
  // A lane owns a row, so every store instruction touches 32 different lines: 32-byte pieces (a whole sector each).
  const int G = 2 * M.split, per_seg = tile_bytes / 32 / M.split;
  for (int half = 0; half < 2; ++half) {
    Chain ch;
    uint8_t* dst = out + static_cast<size_t>(tr * kTileRows + half * 32 + lane) * row_bytes +
                   static_cast<size_t>(tc) * tile_bytes;
#pragma unroll 1
    for (int c = 0; c < tile_bytes / 32; ++c) {
      if (c % per_seg == 0)   // next column segment: its own chain
        ch.init(buf + (__ldg(M.group_base + static_cast<size_t>(t) * G + 2 * (c / per_seg) + half) - base) + lane, M.pad);
      uint32_t v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (EXPAND) {
          const uint32_t e0 = ch.next(lut), e1 = ch.next(lut);
          v[j] = (e0 & 15u) | ((e0 & 0xF0u) << 4) | ((e1 & 15u) << 16) | ((e1 & 0xF0u) << 20);
        } else {
          v[j] = ch.next(lut) & 255u;
          v[j] |= (ch.next(lut) & 255u) << 8;
          v[j] |= (ch.next(lut) & 255u) << 16;
          v[j] |= (ch.next(lut) & 255u) << 24;
        }
      }
      asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 32 * c), "r"(v[0]), "r"(v[1]),
                   "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                   : "memory");
    }
  }
}

// ---------------------------------------------------------------------------------------------- decode to weights

template <int FMT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    k_decode_weights(MatDev M, __half* __restrict__ out, int tr0, int tr1) {
  constexpr bool PAIR = is_paired(FMT);
  constexpr int TW = PAIR ? 2 * kTileSyms : kTileSyms;   // weights per tile row
  constexpr int GW = sub_width(FMT), SB = side_bytes(FMT);
  extern __shared__ __align__(128) uint8_t smem[];
  uint16_t* lut = reinterpret_cast<uint16_t*>(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * kLutSize);
  float* iq4 = reinterpret_cast<float*>(smem + 2 * kLutSize + 64);
  uint32_t* bufs = reinterpret_cast<uint32_t*>(smem + 2 * kLutSize + 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kLutSize / 2; i += blockDim.x)
    reinterpret_cast<uint32_t*>(lut)[i] = __ldg(reinterpret_cast<const uint32_t*>(M.lut) + i);
  if (threadIdx.x < 16) iq4[threadIdx.x] = c_iq4_grid[threadIdx.x];
  __syncthreads();
  const int t = tr0 * M.KT + blockIdx.x * kWarpsPerBlock + warp;   // tiles of tile rows tr0 .. tr1 - 1
  if (t >= tr1 * M.KT) return;
  uint32_t* buf = bufs + static_cast<size_t>(warp) * tile_buf_words(M.max_tile_words);
  uint32_t base;
  if (!stage_tile(M, t, buf, bars + warp, lane, &base)) return;
  const int tr = t / M.KT, tc = t - tr * M.KT;
  out -= static_cast<size_t>(tr0) * kTileRows * M.K;               // `out` holds rows from tile row tr0 on
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const int n = tr * kTileRows + half * 32 + lane;
    Chain ch;
    const int G = 2 * M.split, sub_per_seg = (TW / GW) / M.split;
    const uint8_t* srow = M.side + (static_cast<size_t>(n) * (M.K / 256) + static_cast<size_t>(tc) * (TW / 256)) * SB;
    __half* orow = out + static_cast<size_t>(n) * M.K + static_cast<size_t>(tc) * TW;
#pragma unroll 1
    for (int sb = 0; sb < TW / 256; ++sb) {
      SideRegs<FMT> sr;
      sr.load(srow + sb * SB);
#pragma unroll
      for (int jj = 0; jj < 256 / GW; ++jj) {
        float s, o;
        sr.sub(jj, s, o);
        const int g = sb * (256 / GW) + jj;
        if (g % sub_per_seg == 0)   // next column segment: its own chain
          ch.init(buf + (__ldg(M.group_base + static_cast<size_t>(t) * G + 2 * (g / sub_per_seg) + half) - base) + lane,
                  M.pad);
#pragma unroll
        for (int c = 0; c < GW / 8; ++c) {   // 8 weights -> one 16-byte store
          __half h[8];
          if (PAIR) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t e = ch.next(lut);
              h[2 * i] = __float2half_rn(__fsub_rn(__fmul_rn(s, grid_value<FMT>(e & 15u, iq4)), o));
              h[2 * i + 1] = __float2half_rn(__fsub_rn(__fmul_rn(s, grid_value<FMT>((e >> 4) & 15u, iq4)), o));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              h[i] = __float2half_rn(__fsub_rn(__fmul_rn(s, grid_value<FMT>(ch.next(lut) & 255u, iq4)), o));
          }
          *reinterpret_cast<uint4*>(orow + sb * 256 + jj * GW + c * 8) = *reinterpret_cast<const uint4*>(h);
        }
      }
    }
  }
}

}  // namespace lw
#include "lw_gemm_tc.cuh"
namespace lw {

// Y[j, n] = sum over the `terms` partial rows of P[term, j, n], added in term order (no atomics: results do not
// depend on scheduling).  One thread per four consecutive outputs: 16-byte loads, eight terms in flight.
// unscale (may be null): factor per output row j, applied to the finished sum.
__global__ void k_sum_partials(const float* __restrict__ P, float* __restrict__ Y, int m, int N, int ldy, int terms,
                               const float* __restrict__ unscale = nullptr) {
  pdl_trigger();   // launched as a programmatic dependent of the kernel that writes P (see lw_device.cuh)
  pdl_wait();
  const int quads = N / 4, i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m * quads) return;
  const int j = i / quads, n = (i - j * quads) * 4;
  const float4* p = reinterpret_cast<const float4*>(P + static_cast<size_t>(j) * N + n);
  const size_t stride = static_cast<size_t>(m) * quads;   // one term further, in float4
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int t0 = 0; t0 < terms; t0 += 8) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = t0 + u < terms ? __ldg(p + (t0 + u) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      acc.x += v[u].x;
      acc.y += v[u].y;
      acc.z += v[u].z;
      acc.w += v[u].w;
    }
  }
  if (unscale) {
    const float f = unscale[j];
    acc.x *= f;
    acc.y *= f;
    acc.z *= f;
    acc.w *= f;
  }
  float* y = Y + static_cast<size_t>(j) * ldy + n;
  y[0] = acc.x;
  y[1] = acc.y;
  y[2] = acc.z;
  y[3] = acc.w;
}

// ------------------------------------------------------------------------------------------------------ launchers

static DebugKnobs g_debug_knobs;
DebugKnobs& debug_knobs() { return g_debug_knobs; }

static std::atomic<long long> g_launches{0};
long long launch_count() { return g_launches.load(); }

static int check_cuda(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_kernel_error_text(what, cudaGetErrorString(e));
    return kErrCuda;
  }
  return kOk;
}

static int check_launch(const char* what) {
  g_launches.fetch_add(1);
  return check_cuda(what);
}

int note_launch(const char* what) { return check_launch(what); }

bool tile_output_enabled() {
  static const bool on = !(getenv("LW_TILE_OUT") && atoi(getenv("LW_TILE_OUT")) == 0);
  return on;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point table (no link against the driver library); null where
// the driver does not offer it.
static PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
  static const PFN_cuTensorMapEncodeTiled encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess || found != cudaDriverEntryPointSuccess)
      fn = nullptr;
    (void)cudaGetLastError();
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
  }();
  return encode;
}

void tile_output_warm() { (void)tensor_map_encoder(); }

bool make_row_tile_map(void* tensor_map, void* base, size_t row_bytes, size_t rows) {
  const PFN_cuTensorMapEncodeTiled encode = tensor_map_encoder();
  if (!encode || (reinterpret_cast<uintptr_t>(base) & 15u) || row_bytes % 32 || rows % kTileRows) return false;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {32, kTileRows};
  const cuuint32_t estr[2] = {1, 1};
  return encode(static_cast<CUtensorMap*>(tensor_map), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// SMs of the current device (cached per device: a process may hold handles on several).
int sm_count() {
  static std::atomic<int> per_device[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  int v = per_device[dev].load();
  if (v > 0) return v;
  cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
  v = v > 0 ? v : 1;
  per_device[dev].store(v);
  return v;
}

// Device address of the error word, for kernels of other translation units.
static unsigned int* error_word() {
  static std::mutex mu;
  static unsigned int* per_device[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!per_device[dev] && cudaGetSymbolAddress(reinterpret_cast<void**>(&per_device[dev]), g_kernel_error) != cudaSuccess) {
    cudaGetLastError();
    per_device[dev] = nullptr;
  }
  return per_device[dev];
}

static size_t stage_bytes(const MatDev& M) { return static_cast<size_t>(tile_buf_words(M.max_tile_words)) * 4; }

template <class K>
static int prepare(K kernel, size_t smem) {
  if (smem > 227 * 1024) {
    set_kernel_error_text("launch", "tile staging does not fit shared memory");
    return kErrTooLarge;
  }
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
      cudaSuccess)
    return check_cuda("cudaFuncSetAttribute");
  return kOk;
}

int launch_decode_codes(const MatDev& M, uint8_t* out, bool expand_pairs, cudaStream_t st) {
  if (reinterpret_cast<uintptr_t>(out) & 31u) {
    set_kernel_error_text("decode_codes", "the output must be 32-byte aligned");
    return kErrArg;
  }
  if (is_pair_layout(M.fmt))   // only the ring kernel reads a pair layout: kErrTooLarge sends the caller to the bundle's code
    return gemv1_usable(M) ? launch_decode_codes_ring(M, out, true, error_word(), st) : kErrTooLarge;
  if (gemv1_usable(M) && M.symtab32) {   // the shared decoder, where the layout allows
    const int rc = launch_decode_codes_ring(M, out, expand_pairs, error_word(), st);
    if (rc != kErrTooLarge) return rc;
  }
  const size_t smem = 2 * kLutSize + 128 + kWarpsPerBlock * stage_bytes(M);
  const int blocks = (M.T + kWarpsPerBlock - 1) / kWarpsPerBlock;
  int rc;
  if (expand_pairs) {
    if ((rc = prepare(k_decode_codes<true>, smem))) return rc;
    k_decode_codes<true><<<blocks, kWarpsPerBlock * 32, smem, st>>>(M, out);
  } else {
    if ((rc = prepare(k_decode_codes<false>, smem))) return rc;
    k_decode_codes<false><<<blocks, kWarpsPerBlock * 32, smem, st>>>(M, out);
  }
  return check_launch("k_decode_codes");
}

int launch_decode_weights_rows(const MatDev& M, __half* out, int tr0, int tr1, cudaStream_t st) {
  if (is_pair_layout(M.fmt))   // only the ring kernel reads a pair layout: kErrTooLarge sends the caller to the bundle's code
    return gemv1_usable(M) ? launch_decw(M, out, tr0, tr1, error_word(), st) : kErrTooLarge;
  if (gemv1_usable(M)) {   // the decoder of the batch-1 kernel, where the layout allows
    const int rc = launch_decw(M, out, tr0, tr1, error_word(), st);
    if (rc != kErrTooLarge) return rc;
  }
  const size_t smem = 2 * kLutSize + 128 + kWarpsPerBlock * stage_bytes(M);
  const int tiles = (tr1 - tr0) * M.KT;
  const int blocks = (tiles + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (tr0 < 0 || tr1 > M.N / kTileRows || tiles <= 0) {
    set_kernel_error_text("decode_weights", "bad tile-row range");
    return kErrArg;
  }
  int rc = kErrArg;
#define LW_CASE(F)                                                                      \
  case F:                                                                               \
    if ((rc = prepare(k_decode_weights<F>, smem))) return rc;                           \
    k_decode_weights<F><<<blocks, kWarpsPerBlock * 32, smem, st>>>(M, out, tr0, tr1);   \
    break;
  switch (M.fmt) {
    LW_CASE(kFmtQ4K)
    LW_CASE(kFmtQ5K)
    LW_CASE(kFmtQ6K)
    LW_CASE(kFmtIQ4XS)
    default:
      set_kernel_error_text("decode_weights", "matrix has no block format");
      return kErrArg;
  }
#undef LW_CASE
  return check_launch("k_decode_weights");
}

int launch_decode_weights(const MatDev& M, __half* out, cudaStream_t st) {
  return launch_decode_weights_rows(M, out, 0, M.N / kTileRows, st);
}

// Scratch of one product: one 64-row partial product per tile for one row (added by the same kernel), one per work
// unit and row for 2..8 rows (added by k_sum_partials).
size_t gemv_partial_floats(const MatDev& M, int m) {
  return m <= 1 ? static_cast<size_t>(M.KT) * M.N : gemvm_partial_floats(M, m);
}

// Set by read_kernel_error when a kernel reported that a wait gave up: such a kernel may have left tile-row counters
// of the batch-1 product non-zero, so every matrix zeroes its counters again before its next product.
static std::atomic<unsigned int> g_error_epoch{1};

int launch_gemv(const MatDev& M, const void* X, bool x_is_half, int m, float* Y, int ldy, float* partials,
                size_t partial_capacity, cudaStream_t st, unsigned int* clean_epoch) {
  if (m < 1 || m > 8) {
    set_kernel_error_text("gemv", "m must be 1..8");
    return kErrArg;
  }
  if (!gemv1_usable(M)) {
    set_kernel_error_text("gemv", "matrix has no block format or was not laid out for the fused kernels");
    return kErrArg;
  }
  if (partial_capacity < gemv_partial_floats(M, m)) {
    set_kernel_error_text("gemv", "scratch too small for this product");
    return kErrTooLarge;
  }
  if (m == 1) {
    const unsigned int epoch = g_error_epoch.load();
    if (clean_epoch && *clean_epoch != epoch) {
      if (cudaMemsetAsync(M.row_done, 0, static_cast<size_t>(M.N / kTileRows) * kRowDoneStride * sizeof(unsigned int), st) !=
          cudaSuccess)
        return check_cuda("cudaMemsetAsync(row counters)");
      *clean_epoch = epoch;
    }
    return launch_gemv1(M, X, x_is_half, partials, Y, error_word(), st);   // adds its partial products itself
  }
  const int rc = launch_gemvm(M, X, x_is_half, m, partials, error_word(), st);
  if (rc) return rc;
  const int terms = M.KT * M.split;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((m * (M.N / 4) + 127) / 128);
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // measured: waiting early pays for small products (Q4_K 4096 x 4096, 8 rows: 26 -> 20 us) and costs on large ones
    // (Q6_K 14336 x 4096, 8 rows: 78 -> 88 us), so only up to 16 MB of partial products
    cfg.numAttrs = static_cast<size_t>(terms) * m * M.N * 4 <= (size_t(16) << 20) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, k_sum_partials, static_cast<const float*>(partials), Y, m, M.N, ldy, terms,
                       static_cast<const float*>(nullptr));
  }
  return check_launch("k_sum_partials");
}

// Y[m, N] = X . W^T for up to 64 rows on the tcgen05 path: planes of partial products, then their ordered sum.
// row_scale: the per-row range factors of fp32 activations and their inverses, 2 m floats filled by launch_row_scales
// before this call; unused and may be null when X is fp16.
int launch_gemm_coded(const MatDev& M, const void* X, bool x_is_half, int m, float* Y, int ldy, float* scratch,
                      size_t scratch_floats, float* row_scale, cudaStream_t st) {
  if (!gemv1_usable(M) || M.K % 512 || scratch_floats < gemm_t5_plane_floats(M, m)) {
    set_kernel_error_text("gemm (tcgen05)", "matrix not laid out for it, K not a multiple of 512, or scratch too small");
    return kErrTooLarge;
  }
  if (!x_is_half && !row_scale) {
    set_kernel_error_text("gemm (tcgen05)", "fp32 activations need scratch for their per-row factors");
    return kErrArg;
  }
  int terms = 0;
  const int rc = launch_gemm_t5(M, X, x_is_half, x_is_half ? nullptr : row_scale, m, scratch, error_word(), st, &terms);
  if (rc) return rc;
  k_sum_partials<<<(m * (M.N / 4) + 127) / 128, 128, 0, st>>>(scratch, Y, m, M.N, ldy, terms,
                                                             x_is_half ? nullptr : row_scale + m);
  return check_launch("k_sum_partials");
}

int launch_gemv_batch(int n, const MatDev* const* mats, const void* const* xs, bool x_is_half, float* const* ys,
                      float* const* partials, cudaStream_t st, unsigned int* const* clean_epochs) {
  const unsigned int epoch = g_error_epoch.load();
  for (int j = 0; j < n; ++j) {
    if (clean_epochs && clean_epochs[j] && *clean_epochs[j] != epoch) {
      const MatDev& M = *mats[j];
      if (cudaMemsetAsync(M.row_done, 0, static_cast<size_t>(M.N / kTileRows) * kRowDoneStride * sizeof(unsigned int), st) !=
          cudaSuccess)
        return check_cuda("cudaMemsetAsync(row counters)");
      *clean_epochs[j] = epoch;
    }
  }
  // products whose matrices share format and decode plan go out together, the others one by one
  bool done[8] = {false, false, false, false, false, false, false, false};
  for (int j = 0; j < n; ++j) {
    if (done[j]) continue;
    int idx[8], c = 0;
    for (int i = j; i < n; ++i)
      if (!done[i] && mats[i]->fmt == mats[j]->fmt && mats[i]->group == mats[j]->group &&
          mats[i]->index_bits == mats[j]->index_bits && mats[i]->reader == mats[j]->reader)
        idx[c++] = i;
    const MatDev* gm[8];
    const void* gx[8];
    float* gp[8];
    float* gy[8];
    for (int i = 0; i < c; ++i) {
      gm[i] = mats[idx[i]];
      gx[i] = xs[idx[i]];
      gp[i] = partials[idx[i]];
      gy[i] = ys[idx[i]];
      done[idx[i]] = true;
    }
    int rc = c > 1 ? launch_gemv1_batch(c, gm, gx, x_is_half, gp, gy, error_word(), st) : kErrTooLarge;
    if (rc == kErrTooLarge)
      for (int i = 0; i < c && (rc == kErrTooLarge || rc == kOk); ++i)
        rc = launch_gemv1(*gm[i], gx[i], x_is_half, gp[i], gy[i], error_word(), st);
    if (rc) return rc;
  }
  return kOk;
}

// ---------------------------------------------------------------------------------- product without any allocation
//
// Scratch for the split-K partial sums of lw_linear_static, built into the library image: every GPU that loads the
// library holds these 16 MiB until the process exits.  In host code `g_static_partials` is only a handle for the
// runtime; the device address is looked up once per device with cudaGetSymbolAddress and passed to the kernels.
constexpr size_t kStaticPartialFloats = size_t(4) << 20;
static __device__ __align__(256) float g_static_partials[kStaticPartialFloats];

static int static_partials(float** out) {
  static std::mutex mu;
  static float* per_device[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return check_cuda("cudaGetDevice");
  if (dev < 0 || dev >= 64) {
    set_kernel_error_text("lw_linear_static", "device index out of range");
    return kErrArg;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!per_device[dev]) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_partials);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      set_kernel_error_text("cudaGetSymbolAddress(static scratch)", cudaGetErrorString(e));
      return kErrCuda;
    }
    per_device[dev] = p;
  }
  *out = per_device[dev];
  return kOk;
}

}  // namespace lw

// Declared in include/lwb200.h.  Lives in this file because the scratch array, the look-up of its device address and
// the kernels that receive that address must share one translation unit.
extern "C" int lw_linear_static(void* handle, int id, const void* x_dev, int x_is_half, int m, float* y_dev,
                                void* stream) {
  using namespace lw;
  const MatDev* M = matrix_descriptor(handle, id, m == 1);
  if (!M) return kErrGeneric;
  if (!x_dev || !y_dev || m < 1 || m > 8) {
    set_kernel_error_text("lw_linear_static", "bad argument (m must be 1..8)");
    return kErrArg;
  }
  if (M->fmt == kFmtNone) {
    set_kernel_error_text("lw_linear_static", "matrix has no block format");
    return kErrArg;
  }
  if (gemv_partial_floats(*M, m) > kStaticPartialFloats) {
    set_kernel_error_text("lw_linear_static",
                          "this product needs more partial sums than the built-in scratch holds (tile columns x N for "
                          "one row, tile columns x column segments x m x N for more, must be <= 4194304); use lw_linear");
    return kErrTooLarge;
  }
  float* scratch = nullptr;
  const int rc = static_partials(&scratch);
  if (rc) return rc;
  return launch_gemv(*M, x_dev, x_is_half != 0, m, y_dev, M->N, scratch, kStaticPartialFloats,
                     static_cast<cudaStream_t>(stream), matrix_clean_epoch(handle, id, m == 1));
}

namespace lw {

int launch_row_scales(const float* X, int m, int K, float* scales, cudaStream_t st) {
  k_row_scales<<<m, 256, 0, st>>>(X, K, m, scales);
  return check_launch("k_row_scales");
}

// dst = fp16 of src [m, K] with row r multiplied by scales[r] (launch_row_scales)
int launch_to_half_rows(const float* src, __half* dst, int m, int K, const float* scales, cudaStream_t st) {
  k_to_half_rows<<<dim3((K + 255) / 256, m), 256, 0, st>>>(src, dst, K, scales);
  return check_launch("k_to_half_rows");
}

// Y[m, rows] (row stride ldy, starting at column col0) = X[m, K] . W[rows, K]^T on the tensor cores
// unscale (may be null): per-token factor applied to the finished products (inverse of the activations' range factors)
int launch_gemm_tc(const __half* X, const __half* W, float* Y, int m, int rows, int K, int ldy, float* partials,
                   size_t partial_capacity, const float* unscale, cudaStream_t st) {
  if (m < 1 || rows % kGemmRows || K % kGemmK) {
    set_kernel_error_text("gemm_tc", "shape must be a multiple of 64 rows x 64 columns");
    return kErrArg;
  }
  // split K while the partial planes fit the scratch: one block per 64 rows streaming all of K leaves the SMs idle
  int ks = 8;
  while (ks > 1 && (K % (ks * kGemmK) || static_cast<size_t>(ks) * m * rows > partial_capacity || !partials)) ks /= 2;
  dim3 grid(rows / kGemmRows, (m + kGemmTokens - 1) / kGemmTokens, ks);
  if (ks == 1) {
    k_gemm_tc<<<grid, 128, 0, st>>>(X, W, Y, m, K, ldy, K, 0, unscale);
    return check_launch("k_gemm_tc");
  }
  k_gemm_tc<<<grid, 128, 0, st>>>(X, W, partials, m, K, rows, K / ks, static_cast<size_t>(m) * rows, nullptr);
  int rc = check_launch("k_gemm_tc");
  if (rc) return rc;
  k_sum_partials<<<(m * (rows / 4) + 127) / 128, 128, 0, st>>>(partials, Y, m, rows, ldy, ks, unscale);
  return check_launch("k_sum_partials");
}

// A wait that nothing ends: one warp waits on a barrier no copy will complete and on a release counter nothing
// advances, each for `limit` polls; both must give up, set the error word and return.  Used by lw_debug_wait_probe
// to show that a lost copy cannot hang a kernel.
__global__ void k_wait_probe(unsigned int* err, uint32_t limit, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ uint32_t released;
  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&bar), 1);
    released = 0u;
  }
  __syncthreads();
  const bool a = mbar_wait(smem_addr(&bar), 0, err, limit);
  const bool b = wait_released(&released, 1u, err, limit);
  if (threadIdx.x == 0) *gave_up = (a ? 0 : 1) + (b ? 0 : 2);
}

int launch_wait_probe(unsigned int limit, int* gave_up_host) {
  int* d = nullptr;
  if (cudaMalloc(&d, sizeof(int)) != cudaSuccess) return check_cuda("cudaMalloc(wait probe)");
  cudaMemset(d, 0, sizeof(int));
  k_wait_probe<<<1, 32>>>(error_word(), limit, d);
  int rc = check_launch("k_wait_probe");
  if (!rc && cudaMemcpy(gave_up_host, d, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) rc = check_cuda("wait probe");
  cudaFree(d);
  return rc;
}

int read_kernel_error(unsigned int* value, bool clear) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_kernel_error, sizeof v) != cudaSuccess) return check_cuda("read error word");
  if (v) g_error_epoch.fetch_add(1);   // a kernel gave up: tile-row counters may be stale (see launch_gemv)
  if (clear && v) {
    const unsigned int z = 0;
    cudaMemcpyToSymbol(g_kernel_error, &z, sizeof z);
  }
  *value = v;
  return kOk;
}

}  // namespace lw
