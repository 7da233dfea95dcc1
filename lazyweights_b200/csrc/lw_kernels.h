// Launchers of the CUDA kernels (implemented in lw_kernels.cu).  All take device pointers and a stream; none
// allocates.  They return lw::Status codes and leave a message for lw_last_error() on failure.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "lw_core.h"

namespace lw {

constexpr int kRowDoneStride = 32;

// One coded matrix on the device (all pointers are device pointers; passed to kernels by value).
struct MatDev {
  const uint16_t* lut;          // [2048] symbol | length << 8
  const uint32_t* tab32;        // [2048] length << 28 | grid value(s) as int8 (see lw::fat_table); for a fixed-width
                                // twin: [256] grid values of a paired symbol (unused for unpaired formats)
  const uint32_t* symtab32;     // [2048] length << 28 | symbol: the decode-to-codes kernel's table (or null)
  const uint32_t* cmp_tab;      // comparator form of the code (lw::comparator_table): [0..11] limit per length,
                                // [12..23] index offset per length, [24..279] grid values in canonical order; or null
  const uint32_t* group_base;   // [T * groups + 1] word offset of every chain group
  const uint32_t* words;        // interleaved chain words (+ zero tail)
  const uint8_t* side;          // [N, K / 256 * side_bytes] or null (symbols only)
  const uint8_t* unit_slow;     // [T * split] how the batch-1 kernel decodes the unit: 0 = groups of `group` symbols,
                                // 1 = groups of two, 2 = symbol by symbol (or null: kernel not usable)
  unsigned int* row_done;       // [N / 64][kRowDoneStride] tiles of a tile row finished by the running batch-1 product
                                // (zero between launches; one counter per 128-byte line: neighbours would contend)
  int index_bits;               // windows of the batch-1 kernel's table = 1 << index_bits; its copies = 1 << (pad - 2)
  int group;                    // symbols per group of the batch-1 kernel's grouped decoder (0 = kernel not usable)
  int N, K, Ks, KT, T;
  int fmt, split;
  int reader;                   // 0: Huffman-coded chains; 1: fixed-width twin (lw::build_twin)
  int pad;                      // zero bits at the start of every chain
  int max_len;                  // longest code of the table
  uint32_t max_tile_words;      // largest tile, in words
  uint32_t max_unit_words;      // largest column segment of a tile (both row halves), in words
};

// uint8 [N, K] (expand_pairs: each paired symbol becomes two bytes, low nibble first) or symbols [N, Ks].
int launch_decode_codes(const MatDev& M, uint8_t* out, bool expand_pairs, cudaStream_t st);
// fp16 [N, K], bit-exact float32 block arithmetic rounded once to fp16.
int launch_decode_weights(const MatDev& M, __half* out, cudaStream_t st);
// Only tile rows tr0 .. tr1 - 1 (64 matrix rows each); `out` receives those rows, [ (tr1 - tr0) * 64, K ].
int launch_decode_weights_rows(const MatDev& M, __half* out, int tr0, int tr1, cudaStream_t st);
// fp32 -> fp16 copy, and Y[m, rows] = X[m, K] . W[rows, K]^T (fp16 in, fp32 out, tensor cores) for the decode + GEMM path.
// fp32 activations on their way to fp16: scales[r] = a power of two that brings row r inside fp16's range (1 unless the
// row holds values above 2^15), scales[m + r] = its inverse, to be applied to row r of the product.
int launch_row_scales(const float* X, int m, int K, float* scales, cudaStream_t st);
int launch_to_half_rows(const float* src, __half* dst, int m, int K, const float* scales, cudaStream_t st);
int launch_gemm_tc(const __half* X, const __half* W, float* Y, int m, int rows, int K, int ldy, float* partials,
                   size_t partial_capacity, const float* unscale, cudaStream_t st);
// Y[j, n] (row stride ldy) = sum_k X[j, k] W[n, k] for m <= 8 rows of X (fp16 or fp32, row-major [m, K]).
// `partials` (partial_capacity floats) must hold gemv_partial_floats(M, m) floats.  `clean_epoch` (may be null) is the
// caller's per-matrix note of when the matrix's tile-row counters were last known to be zero: after a kernel reported
// a wait that gave up, the next one-row product of every matrix zeroes them again.
size_t gemv_partial_floats(const MatDev& M, int m);
int launch_gemv(const MatDev& M, const void* X, bool x_is_half, int m, float* Y, int ldy, float* partials,
                size_t partial_capacity, cudaStream_t st, unsigned int* clean_epoch = nullptr);
// Y[m, N] = X[m, K] . W^T for 1 <= m <= 64 with the decode + tcgen05 kernel (lw_gemm_t5.cuh): the decoded weights go
// from registers to tensor memory, never to DRAM.  `scratch` holds the K / 512 planes of partial products.  Returns
// kErrTooLarge, with nothing launched, where that kernel cannot take the product.  row_scale (fp32 activations only):
// 2 m floats already filled by launch_row_scales.
int launch_gemm_coded(const MatDev& M, const void* X, bool x_is_half, int m, float* Y, int ldy, float* scratch,
                      size_t scratch_floats, float* row_scale, cudaStream_t st);

// n one-row products y_j = W_j x_j (each with its own scratch of gemv_partial_floats(M_j, 1) floats); in one launch
// where the matrices share a format and decode plan, one by one otherwise.
int launch_gemv_batch(int n, const MatDev* const* mats, const void* const* xs, bool x_is_half, float* const* ys,
                      float* const* partials, cudaStream_t st, unsigned int* const* clean_epochs);

// Reads (and optionally clears) the device error word that kernels set when a bounded wait gives up.
int read_kernel_error(unsigned int* value, bool clear);

// Test entry: a kernel whose waits nothing ends, with `limit` polls each; *gave_up = 1 (barrier) + 2 (counter).
int launch_wait_probe(unsigned int limit, int* gave_up);

void set_kernel_error_text(const char* what, const char* detail);
// Device descriptor of matrix `id` of a handle (implemented next to the handle type), or null; and that matrix's
// clean-epoch note (see launch_gemv).
// one_row: the descriptor (and its counter epoch) a product of ONE activation row reads - the matrix's pair layout
// where it has one
const MatDev* matrix_descriptor(void* handle, int id, bool one_row = false);
unsigned int* matrix_clean_epoch(void* handle, int id, bool one_row = false);
// Kernels launched by this library since it was loaded.
long long launch_count();

}  // namespace lw
