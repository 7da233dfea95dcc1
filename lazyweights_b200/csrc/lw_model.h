// The handle type behind the C ABI: a bundle's coded matrices on one GPU and, when the bundle carries a model
// configuration, the decoder runtime state (lw_runtime.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "lw_host.h"
#include "lw_kernels.h"

namespace lw {

struct Matrix {
  std::string name;
  int N = 0, K = 0, Ks = 0, fmt = kFmtNone;
  bool paired = false;
  long long blob_bytes = 0, side_bytes = 0, file_offset = -1;
  size_t device_bytes = 0;
  double slow_fraction = 0.0;   // share of work units the batch-1 kernel decodes symbol by symbol
  void* d_block = nullptr;   // one allocation: table, group bases, words, side bytes
  MatDev dev{};
  unsigned int clean_epoch = 0;   // when the tile-row counters were last known to be zero (see launch_gemv)
  // fixed-width twin (lw_matrix_make_twin): a second device image of the same matrix, read by the same kernel
  void* d_twin = nullptr;
  MatDev twin{};
  size_t twin_bytes = 0;          // chain words + unit scales: what one product of the twin reads
  unsigned int twin_epoch = 0;
  // pair layout (lw::build_pairs; Q6_K / Q5_K with K a multiple of 512): what the one-row product and the decode to
  // fp16 weights read instead of `dev` - the other kernels keep reading the bundle's own code
  void* d_pair = nullptr;
  MatDev pair{};
  size_t pair_bytes = 0;
  unsigned int pair_epoch = 0;
};

struct Runtime;   // decoder state, defined in lw_runtime.cu
struct Model;
void runtime_free(Model* M);

struct Model {
  std::string dir;
  Manifest man;
  int fd = -1;
  int device = 0;
  bool verbose = false;
  std::vector<Matrix> mats;
  std::map<std::string, int> by_name;
  float* d_partials = nullptr;   // split-K partial sums, sized for the largest matrix at m = 8
  size_t partial_floats = 0;
  float *d_x = nullptr, *d_y = nullptr;   // staging of rt_test_matmul's host buffers (grown on demand, kept)
  size_t x_floats = 0, y_floats = 0;
  float* h_pin = nullptr;                 // pinned host staging for the same call (x, then y)
  size_t pin_floats = 0;
  __half *d_w16 = nullptr, *d_x16 = nullptr;   // decode + GEMM path: decoded weights of a chunk of tile rows, fp16 x
  size_t w16_halfs = 0, x16_halfs = 0;
  float* d_row_scale = nullptr;   // per-row range factors of fp32 activations headed for fp16 (2 floats per row)
  size_t row_scale_floats = 0;
  size_t resident_bytes = 0;
  long long coded_bytes = 0, side_bytes = 0;
  Runtime* rt = nullptr;
  ~Model() {
    runtime_free(this);   // the decoder state, if any (also after a failed rt_open)
    for (auto& m : mats) {
      if (m.d_block) cudaFree(m.d_block);
      if (m.d_twin) cudaFree(m.d_twin);
      if (m.d_pair) cudaFree(m.d_pair);
    }
    if (d_partials) cudaFree(d_partials);
    if (d_x) cudaFree(d_x);
    if (d_y) cudaFree(d_y);
    if (h_pin) cudaFreeHost(h_pin);
    if (d_w16) cudaFree(d_w16);
    if (d_x16) cudaFree(d_x16);
    if (d_row_scale) cudaFree(d_row_scale);
    if (fd >= 0) close(fd);
  }
};

int cuda_fail(const char* what, cudaError_t e);
// path 0: fused decode + product in chunks of eight rows up to 16 rows, decode + tensor-core GEMM above; 1: always
// fused; 2: always decode + GEMM.
int linear_device(Model* M, Matrix& mx, const void* x, bool x_half, int m, float* y, int ldy, cudaStream_t st,
                  int path = 0);
// n one-row products of matrices of this handle (indices into M->mats) against fp32 activations, in one launch where
// they share format and decode plan (see launch_gemv_batch).
int linear_batch_device(Model* M, int n, const int* mat_index, const float* const* xs, float* const* ys, cudaStream_t st);
int runtime_init(Model* M, int max_ctx, int max_batch);
// True if the calling thread's current device is the one the handle was opened on (kernels and scratch belong to it).
int check_device(const Model* M);
double runtime_stat(const Model* M, const char* key);

}  // namespace lw
