// Device-side building blocks shared by the kernels: the matrix descriptor, bulk-copy staging of a tile's words
// into shared memory (cp.async.bulk + mbarrier), the per-chain bit reader and the block dequantisation arithmetic.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "lw_core.h"
#include "lw_kernels.h"

namespace lw {

// ------------------------------------------------------------------------------------------- shared memory + TMA

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Starts one bulk copy global -> shared that signals `bar` with its byte count.  dst, src and bytes are multiples
// of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// Waits for phase `parity` of the barrier.  The wait is bounded: after kWaitLimit polls it records the failure in
// the device error word `err` (bit 0) and returns false, so a copy that never lands cannot hang the device.
// `limit` is an argument so that a test can make a wait run out quickly.
constexpr uint32_t kWaitLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int* err,
                                          uint32_t limit = kWaitLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  atomicOr(err, 1u);
  return false;
}

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may start while its
// predecessor in the stream is still running (as soon as every block of the predecessor has called pdl_trigger or
// left), and must call pdl_wait before it touches anything the predecessor writes: the wait returns when the
// predecessor has completed and its writes are visible.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ chain reader

// Reads one chain (a re-based bit stream whose word i sits at base + 32 i + lane) out of shared memory.  Three words
// are held: the 64-bit window (w0, w1) and the next word, fetched one refill ahead so that the shared-memory load is
// off the symbol-to-symbol dependency.
struct Chain {
  const uint32_t* p;
  uint32_t w0, w1, w2, bp;
  __device__ __forceinline__ void init(const uint32_t* chain_words, int pad) {
    w0 = chain_words[0];
    w1 = chain_words[32];
    w2 = chain_words[64];
    p = chain_words + 96;
    bp = pad;
  }
  __device__ __forceinline__ uint32_t next(const uint16_t* lut) {
    const uint32_t e = lut[__funnelshift_r(w0, w1, bp) & (kLutSize - 1)];
    bp += e >> 8;
    if (bp >= 32) {
      bp -= 32;
      w0 = w1;
      w1 = w2;
      w2 = *p;
      p += 32;
    }
    return e;
  }
};

// ------------------------------------------------------------------------------------------------- block formats

__device__ __forceinline__ float half_bits_to_float(uint32_t v) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(v)));
}

// Side bytes of one 256-weight super-block held as little-endian 32-bit words.
template <int FMT>
struct SideRegs {
  static constexpr int kWords = (side_bytes(FMT) + 3) / 4;
  uint32_t w[kWords];
  __device__ __forceinline__ uint32_t byte(int i) const { return (w[i >> 2] >> (8 * (i & 3))) & 255u; }
  __device__ __forceinline__ void load(const uint8_t* p) {
    if (FMT == kFmtQ6K) {   // 18-byte records: only 2-byte aligned
      const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
#pragma unroll
      for (int i = 0; i < kWords; ++i)
        w[i] = __ldg(h + 2 * i) | (2 * i + 1 < 9 ? static_cast<uint32_t>(__ldg(h + 2 * i + 1)) << 16 : 0u);
    } else {
      const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
#pragma unroll
      for (int i = 0; i < kWords; ++i) w[i] = __ldg(q + i);
    }
  }
  // (scale, offset) of sub-block j: weight = scale * f(code) - offset, all in float32, every operation rounded
  // separately (llama.cpp's block formulas; reference: scripts/a2_kq_bundle.py:50-68, kernels/llmrt.cu:126-149).
  __device__ __forceinline__ void sub(int j, float& s, float& o) const {
    if (FMT == kFmtQ4K || FMT == kFmtQ5K) {
      uint32_t sc, mn;
      if (j < 4) {
        sc = byte(4 + j) & 63u;
        mn = byte(8 + j) & 63u;
      } else {
        sc = (byte(8 + j) & 15u) | ((byte(j) >> 6) << 4);
        mn = (byte(8 + j) >> 4) | ((byte(4 + j) >> 6) << 4);
      }
      s = __fmul_rn(half_bits_to_float(w[0]), static_cast<float>(sc));
      o = __fmul_rn(half_bits_to_float(w[0] >> 16), static_cast<float>(mn));
    } else if (FMT == kFmtQ6K) {
      s = __fmul_rn(half_bits_to_float(w[4]), static_cast<float>(static_cast<int8_t>(byte(j))));
      o = 0.f;
    } else {
      const uint32_t ls = ((byte(4 + j / 2) >> (4 * (j & 1))) & 15u) | (((w[0] >> (16 + 2 * j)) & 3u) << 4);
      s = __fmul_rn(half_bits_to_float(w[0]), static_cast<float>(static_cast<int>(ls) - 32));
      o = 0.f;
    }
  }
};

__constant__ float c_iq4_grid[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// f(code): the format's grid value.  2^23 + q has q in its low mantissa bits, so the subtraction is exact.
template <int FMT>
__device__ __forceinline__ float grid_value(uint32_t q, const float* iq4) {
  if (FMT == kFmtIQ4XS) return iq4[q];
  return __uint_as_float(0x4B000000u | q) - (FMT == kFmtQ6K ? 8388640.f : 8388608.f);
}

}  // namespace lw
