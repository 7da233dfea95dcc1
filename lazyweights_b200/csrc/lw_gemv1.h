// Launcher of the batch-1 kernel (lw_gemv1.cuh; instantiated in lw_gemv1.cu) and helpers it shares with lw_kernels.cu.
#pragma once
#include "lw_kernels.h"

namespace lw {

// True if the matrix was laid out for the batch-1 kernel (default column split, pad 6 or 7, unit flags present).
bool gemv1_usable(const MatDev& M);
// y[N] = W x for one activation row; partials[KT * split][N] is scratch for the per-segment partial products (added
// in a fixed order by the same kernel); `err` = device error word.
int launch_gemv1(const MatDev& M, const void* X, bool x_is_half, float* partials, float* y, unsigned int* err,
                 cudaStream_t st);

// n <= 8 one-row products y_j = W_j x_j in ONE launch (matrices of one format and decode plan); kErrTooLarge, with
// nothing launched, where the products cannot share a launch.
int launch_gemv1_batch(int n, const MatDev* const* mats, const void* const* xs, bool x_is_half, float* const* partials,
                       float* const* ys, unsigned int* err, cudaStream_t st);

// 2 <= m <= 8 rows (lw_gemvm.cuh): partials[KT * split][m][N] = one partial product per work unit and row, to be added
// by the caller over KT * split terms; gemvm_partial_floats = the floats that takes.
size_t gemvm_partial_floats(const MatDev& M, int m);
int launch_gemvm(const MatDev& M, const void* X, bool x_is_half, int m, float* partials, unsigned int* err,
                 cudaStream_t st);

// Symbols [N, Ks] (or, for paired formats with `expand`, codes [N, K]) on the batch-1 kernel's decoder (lw_decc.cuh);
// kErrTooLarge (nothing launched) where it cannot take the matrix.
int launch_decode_codes_ring(const MatDev& M, uint8_t* out, bool expand, unsigned int* err, cudaStream_t st);

// Decode + tcgen05 GEMM for up to 64 rows (lw_gemm_t5.cuh): planes[K / 512][m][N] of partial products, *terms = K / 512,
// to be added by the caller; kErrTooLarge (nothing launched) where this kernel cannot take the product.  row_scale (may
// be null): factor per row of X applied before the conversion to fp16; the caller multiplies the sums by the inverse.
size_t gemm_t5_plane_floats(const MatDev& M, int m);
int launch_gemm_t5(const MatDev& M, const void* X, bool x_is_half, const float* row_scale, int m, float* planes,
                   unsigned int* err, cudaStream_t st, int* terms);

// fp16 weights of tile rows tr0 .. tr1 - 1 on the batch-1 kernel's decoder (lw_decw.cuh); kErrTooLarge (nothing
// launched) where it cannot take the matrix.
int launch_decw(const MatDev& M, __half* out, int tr0, int tr1, unsigned int* err, cudaStream_t st);

// Test switches (set through lw_debug_set; defaults are the production values).
struct DebugKnobs {
  int max_units = 1024;            // cap on the units a block is dealt per launch (smaller: more launches per product)
  uint32_t wait_limit = 1u << 22;  // polls after which a device-side wait gives up
  int drop_unit = -1;              // the producers of block 0 skip the copy of this unit (its consumer's wait runs out)
  int t5_min_rows = 9;             // products of at least this many rows (and at most 64) take the tcgen05 kernel (eight
                                   // rows: the fused kernel, 46-49 against 54 us on 14336 x 4096 in all four formats)
  int pairs = 1;                   // one-row products read a matrix's pair layout where it has one (0: the bundle's code)
};
DebugKnobs& debug_knobs();

// Tensor map (a CUtensorMap, 128 bytes, 64-byte aligned) over an output buffer seen as bytes [rows][row_bytes] with boxes of
// 64 rows x 32 bytes and the 32-byte swizzle; false where the driver does not offer the encoder or refuses the shape.
bool make_row_tile_map(void* tensor_map, void* base, size_t row_bytes, size_t rows);
// False with LW_TILE_OUT=0 in the environment (read once): the decode kernels then keep their 32-byte stores.
bool tile_output_enabled();
// Looks the tensor-map encoder up now (done when a matrix is loaded, so that a first decode inside a stream capture makes
// no such call).
void tile_output_warm();
int note_launch(const char* what);   // counts a launch and returns the status of cudaGetLastError
int sm_count();

}  // namespace lw
