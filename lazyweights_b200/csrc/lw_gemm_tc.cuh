// Tensor-core GEMM for the decode + GEMM path (more than eight activation rows, or path 2 of rt_test_matmul):
// Y[m, n] = sum_k X[m, k] W[n, k], fp16 operands, fp32 accumulation.  The role of the reference's k_gemm_raw8 /
// k_gemm2_raw8 (kernels/llmrt.cu:211-343), which run SIMT float FMAs on decoded codes; here the decoded, dequantised
// fp16 weights (k_decode_weights) feed mma.sync.m16n8k16.  A block owns 64 weight rows x up to 32 tokens; four warps
// take 16 rows each; K advances in slabs of 64 staged in shared memory (rows padded by 8 halfs so that fragment
// loads are conflict-free).  Small M keeps this path bound by the decode and by reading the fp16 weights once.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace lw {

constexpr int kGemmRows = 64, kGemmTokens = 32, kGemmK = 64, kGemmPad = 8;

// fp32 activations enter the tensor cores as fp16, whose largest finite value is 65504: a row with larger entries
// (the input of a down projection can be the product of two unnormalised projections) would turn into infinities and
// the product into NaN.  Each row therefore gets a power-of-two factor that brings its largest |x| to at most 2^15 -
// exactly 1 for every row that already fits, so ordinary inputs are converted bit for bit as before - and the
// product's rows are multiplied by the inverse afterwards (exact: both are powers of two).
// scales[r] = factor of row r, scales[m + r] = its inverse.  One block per row.
__global__ void __launch_bounds__(256) k_row_scales(const float* __restrict__ X, int K, int m, float* __restrict__ scales) {
  __shared__ float part[8];
  const int r = blockIdx.x;
  const float* x = X + static_cast<size_t>(r) * K;
  float amax = 0.f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(x[k]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, part[w]);
    int e = 0;
    if (amax > 32768.f && amax <= 3.0e38f) {   // frexp: amax = f 2^e with f in [0.5, 1)
      frexpf(amax, &e);
      e -= 15;
    }
    scales[r] = ldexpf(1.f, -e);
    scales[m + r] = ldexpf(1.f, e);
  }
}

// dst[r][k] = half(src[r][k] * scales[r]); grid (ceil(K / 256), m)
__global__ void k_to_half_rows(const float* __restrict__ src, __half* __restrict__ dst, int K,
                               const float* __restrict__ scales) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
  if (k < K) dst[static_cast<size_t>(r) * K + k] = __float2half_rn(src[static_cast<size_t>(r) * K + k] * scales[r]);
}

__global__ void __launch_bounds__(128)
    k_gemm_tc(const __half* __restrict__ X, const __half* __restrict__ W, float* __restrict__ Y, int m, int K, int ldy,
              int kspan, size_t zstride, const float* __restrict__ unscale) {
  __shared__ __align__(16) __half ws[kGemmRows][kGemmK + kGemmPad];
  __shared__ __align__(16) __half xs[kGemmTokens][kGemmK + kGemmPad];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * kGemmRows, m0 = blockIdx.y * kGemmTokens;
  const int mt = min(kGemmTokens, m - m0);
  float acc[4][4];   // [token block of 8][fragment]
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  // blockIdx.z takes the K range [z * kspan, (z + 1) * kspan) and writes its own output plane (split K: more blocks
  // and more loads in flight than one block per 64 rows streaming all of K)
  Y += blockIdx.z * zstride;
  for (int k0 = blockIdx.z * kspan; k0 < (blockIdx.z + 1) * kspan; k0 += kGemmK) {
    // stage 64 x 64 weights and up to 32 x 64 activations (16-byte chunks)
    for (int c = threadIdx.x; c < kGemmRows * (kGemmK / 8); c += blockDim.x) {
      const int r = c / (kGemmK / 8), q = c % (kGemmK / 8);
      *reinterpret_cast<uint4*>(&ws[r][q * 8]) =
          *reinterpret_cast<const uint4*>(W + static_cast<size_t>(n0 + r) * K + k0 + q * 8);
    }
    for (int c = threadIdx.x; c < kGemmTokens * (kGemmK / 8); c += blockDim.x) {
      const int r = c / (kGemmK / 8), q = c % (kGemmK / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < mt) v = *reinterpret_cast<const uint4*>(X + static_cast<size_t>(m0 + r) * K + k0 + q * 8);
      *reinterpret_cast<uint4*>(&xs[r][q * 8]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGemmK; kk += 16) {
      // A fragment (weights, row-major 16 x 16): rows g, g + 8 of this warp's 16 rows
      const __half* wr = &ws[warp * 16 + g][kk + 2 * t];
      const uint32_t a0 = *reinterpret_cast<const uint32_t*>(wr);
      const uint32_t a1 = *reinterpret_cast<const uint32_t*>(wr + 8 * (kGemmK + kGemmPad));
      const uint32_t a2 = *reinterpret_cast<const uint32_t*>(wr + 8);
      const uint32_t a3 = *reinterpret_cast<const uint32_t*>(wr + 8 * (kGemmK + kGemmPad) + 8);
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        // B fragment (activations as a 16 x 8 column-major tile): token nb * 8 + g, k = kk + 2 t (+ 8)
        const __half* xr = &xs[nb * 8 + g][kk + 2 * t];
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xr);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xr + 8);
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(acc[nb][0]), "+f"(acc[nb][1]), "+f"(acc[nb][2]), "+f"(acc[nb][3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
      }
    }
    __syncthreads();
  }
  // C fragment: rows g, g + 8 (weight rows = output columns), columns 2 t, 2 t + 1 (tokens)
#pragma unroll
  for (int nb = 0; nb < 4; ++nb)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tok = m0 + nb * 8 + 2 * t + (j & 1), row = n0 + warp * 16 + g + (j >> 1) * 8;
      if (tok < m) Y[static_cast<size_t>(tok) * ldy + row] = unscale ? acc[nb][j] * unscale[tok] : acc[nb][j];
    }
}

}  // namespace lw
