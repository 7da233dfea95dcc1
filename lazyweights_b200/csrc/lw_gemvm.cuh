// Fused decode + dequant + product for 2..8 activation rows: the batch-1 kernel's decoder (lw_gemv1.cuh: replicated
// 32-bit table, grouped refills chosen from the data, unit scales staged with the chains, producer warps feeding a ring
// of staging buffers, units drawn from a shared counter) with MR dot products per decoded symbol instead of one.
// Included by lw_gemvm.cu.
//
// What differs from the batch-1 kernel:
//  * activations: MR rows, quantised to 16-bit fixed point per sub-block as there, stored symbol-major
//    (xq[column][symbol][row]) so that one 16-byte shared-memory load brings four rows' operands of one symbol;
//  * registers: 2 x MR integer sums and 2 x MR float totals per lane, so the block is smaller (768 threads for four
//    rows, 640 for eight) and holds fewer tile columns of activations;
//  * output: one partial product per work unit and row, P[unit term][row][N], added by k_sum_partials (a second
//    launch; the in-kernel sum of the batch-1 kernel would need MR times its shared-memory ring).
#pragma once
#include "lw_gemv1.cuh"

namespace lw {

// One sub-block of both chains against MR activation rows.  xs points at the sub-block's operands, [symbol][MR] words.
template <int G, int SPG, uint32_t MASK, int MR, class CH>
__device__ __forceinline__ void sub_block_m(CH& ca, CH& cb, const uint8_t* tab, uint32_t lane_off,
                                            const uint32_t* xs, const int first, const bool last, int (&acc_a)[MR],
                                            int (&acc_b)[MR]) {
#pragma unroll
  for (int c = 0; c < SPG; ++c) {
    const int f = first + c;
    if (f % G == 0) {
      ca.begin();
      cb.begin();
    }
    const uint32_t ea = ca.template sym<MASK>(tab, lane_off), eb = cb.template sym<MASK>(tab, lane_off);
#pragma unroll
    for (int r4 = 0; r4 < MR / 4; ++r4) {
      const uint4 x = *reinterpret_cast<const uint4*>(xs + c * MR + 4 * r4);
      acc_a[4 * r4 + 0] = __dp2a_lo(static_cast<int>(x.x), static_cast<int>(ea), acc_a[4 * r4 + 0]);
      acc_a[4 * r4 + 1] = __dp2a_lo(static_cast<int>(x.y), static_cast<int>(ea), acc_a[4 * r4 + 1]);
      acc_a[4 * r4 + 2] = __dp2a_lo(static_cast<int>(x.z), static_cast<int>(ea), acc_a[4 * r4 + 2]);
      acc_a[4 * r4 + 3] = __dp2a_lo(static_cast<int>(x.w), static_cast<int>(ea), acc_a[4 * r4 + 3]);
      acc_b[4 * r4 + 0] = __dp2a_lo(static_cast<int>(x.x), static_cast<int>(eb), acc_b[4 * r4 + 0]);
      acc_b[4 * r4 + 1] = __dp2a_lo(static_cast<int>(x.y), static_cast<int>(eb), acc_b[4 * r4 + 1]);
      acc_b[4 * r4 + 2] = __dp2a_lo(static_cast<int>(x.z), static_cast<int>(eb), acc_b[4 * r4 + 2]);
      acc_b[4 * r4 + 3] = __dp2a_lo(static_cast<int>(x.w), static_cast<int>(eb), acc_b[4 * r4 + 3]);
    }
    if (f % G == G - 1 || (last && c == SPG - 1)) {
      ca.end();
      cb.end();
    }
  }
}

template <int SPG, int MR, class CH>
__device__ __forceinline__ void sub_block_slow_m(CH& ca, CH& cb, const uint32_t* tab32, uint32_t pad,
                                                 const uint32_t* xs, int (&acc_a)[MR], int (&acc_b)[MR]) {
#pragma unroll 1
  for (int c = 0; c < SPG; ++c) {
    const uint32_t ea = ca.slow_sym(tab32, pad), eb = cb.slow_sym(tab32, pad);
#pragma unroll
    for (int r = 0; r < MR; ++r) {
      const uint32_t xw = xs[c * MR + r];
      acc_a[r] = __dp2a_lo(static_cast<int>(xw), static_cast<int>(ea), acc_a[r]);
      acc_b[r] = __dp2a_lo(static_cast<int>(xw), static_cast<int>(eb), acc_b[r]);
    }
  }
}

constexpr int gemvm_threads(int mr) { return mr <= 4 ? 768 : 640; }

struct GemvmArgs {
  RingArgs r;
  const void* x;     // activations [m][K], fp16 or fp32
  float* partials;   // P[KT * SPLIT][m][N]
  int x_is_half;
  int pdl;           // launched as a programmatic dependent: the activations may only be read after pdl_wait
  int m;             // rows in use (<= MR; the others are computed as zeros and not written)
};

template <int FMT, int G, int IDXBITS, int LOG_R, int MR>
__global__ void __launch_bounds__(gemvm_threads(MR), 1) k_gemvm(MatDev M, GemvmArgs A) {
  const RingArgs& RA = A.r;
  constexpr bool PAIR = is_paired(FMT);
  constexpr int SPLIT = default_split(FMT);
  constexpr int TW = PAIR ? 2 * kTileSyms : kTileSyms;
  constexpr int GW = sub_width(FMT), SPG = sub_syms(FMT), SIDEW = unit_side_words(FMT);
  constexpr int NSB = TW / GW;                                    // sub-blocks per tile row
  constexpr int USYM = kTileSyms / SPLIT;
  constexpr int NSU = NSB / SPLIT;                                // sub-blocks per unit
  static_assert(NSU == 4 || NSU == 8, "a unit is four sub-blocks (eight of the 16-weight sub-blocks of a Q6_K pair layout)");
  static_assert(MR == 4 || MR == 8, "four or eight rows");
  constexpr bool PAIR_LAYOUT = is_pair_layout(FMT);
  constexpr bool HAS_OFFSET = FMT == kFmtQ4K || FMT == kFmtQ5K || FMT == kFmtQ5KP;
  constexpr int NIDX = 1 << IDXBITS, R = 1 << LOG_R;
  constexpr bool SINGLE = NIDX <= kLutSize;
  constexpr uint32_t MASK = static_cast<uint32_t>(NIDX - 1) << (LOG_R + 2);
  constexpr int kReplicatedTableBytes = NIDX * R * 4;
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t* tab = reinterpret_cast<uint32_t*>(smem);
  uint32_t* tab1 = reinterpret_cast<uint32_t*>(smem + kReplicatedTableBytes);
  uint32_t* xq = tab1 + kLutSize;                                                   // [cols][kTileSyms][MR] words
  float* xscale = reinterpret_cast<float*>(xq + static_cast<size_t>(RA.cols_per_set) * kTileSyms * MR);   // [cols][NSB][MR]
  float* xg = xscale + static_cast<size_t>(RA.cols_per_set) * NSB * MR;              // [cols][NSB][MR] (offset formats)
  RingMem RM;
  RM.carve(xg + (HAS_OFFSET ? RA.cols_per_set * NSB * MR : 0), RA);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TableLoad<IDXBITS, LOG_R, SINGLE> table;   // the matrix is not written by the kernel before: no need to wait for it
  table.issue(M.tab32, warp, lane, RA.warps);
  BlockShare S;
  S.init(M, RA, SPLIT, blockIdx.x, gridDim.x);
  const int set = S.set, ncol = S.ncol, nmine = S.nmine;
  pdl_trigger();   // see lw_gemv1.cuh: set-up overlaps the previous kernel's tail, pdl_wait before the activations
  const bool consumer = warp < RA.warps;
  const int nthr = RA.warps * 32, m = A.m;

  // 1. the block's list (whole tiles, symbol-by-symbol tiles first) and the ring's barriers
  ring_reset(RM);
  __syncthreads();
  ring_build_list<SPLIT>(M, RA, S, RM);
  __syncthreads();

  if (!consumer) {
    ring_produce(M, RA, RM, nmine, warp - RA.warps, lane);   // 2a. producers
    return;
  }

  // 2b. consumers: tables, then the activations of the block's tile columns for all rows
  table.finish(M.tab32, tab, tab1, warp, lane, RA.warps);
  if (A.pdl) pdl_wait();
  constexpr int XB = 8;
  const int per_row = ncol * TW, total = per_row * MR;   // rows >= m are stored as zeros
  for (int base = 0; base < total; base += XB * nthr) {
    float xv[XB];
#pragma unroll
    for (int u = 0; u < XB; ++u) {
      const int i = base + u * nthr + threadIdx.x;
      xv[u] = 0.f;
      if (i < total) {
        const int r = i / per_row, w = i - r * per_row, j = w / TW, k = w - j * TW;
        if (r < m) {
          const size_t src = static_cast<size_t>(r) * M.K + static_cast<size_t>(set + RA.nsets * j) * TW + k;
          xv[u] = A.x_is_half ? __half2float(static_cast<const __half*>(A.x)[src]) : static_cast<const float*>(A.x)[src];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < XB; ++u) {
      const int i = base + u * nthr + threadIdx.x;
      if (i < total) {   // whole warps take this branch together: sizes are multiples of 32
        const int r = i / per_row, w = i - r * per_row;
        float amax = fabsf(xv[u]), sum = xv[u];
#pragma unroll
        for (int o = 1; o < GW; o <<= 1) {
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          if (HAS_OFFSET) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        const int q = __float2int_rn(xv[u] * (amax > 0.f ? 32767.f / amax : 0.f));
        if (PAIR) {
          const int qn = __shfl_down_sync(0xffffffffu, q, 1);
          if ((lane & 1) == 0) xq[static_cast<size_t>(w >> 1) * MR + r] = (static_cast<uint32_t>(q) & 0xFFFFu) | (static_cast<uint32_t>(qn) << 16);
        } else {
          xq[static_cast<size_t>(w) * MR + r] = static_cast<uint32_t>(q) & 0xFFFFu;
        }
        if ((lane & (GW - 1)) == 0) {
          xscale[static_cast<size_t>(w / GW) * MR + r] = amax * (1.f / 32767.f);
          if (HAS_OFFSET) xg[static_cast<size_t>(w / GW) * MR + r] = sum;
        }
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
  const uint32_t lane_off = (lane & (R - 1)) << 2;
#pragma unroll 1
  for (;;) {
    Unit u;
    const int got = ring_draw(RA, RM, nmine, lane, u);
    if (got == 0) break;
    if (got < 0) return;
    const uint32_t j = u.j, seg = u.seg, tr = u.tr, cls = u.cls, lines = u.lines, second = u.second;
    const int tc = set + RA.nsets * static_cast<int>(j);
    const int na = static_cast<int>(tr) * kTileRows + lane, nb = na + 32;
    const uint32_t* xt = xq + (static_cast<size_t>(j) * kTileSyms + seg * USYM) * MR;
    const float* xst = xscale + (static_cast<size_t>(j) * NSB + seg * NSU) * MR;
    const float* xgt = xg + (static_cast<size_t>(j) * NSB + seg * NSU) * MR;
    const uint32_t* buf = u.buf;
    UnitSide<FMT> side_a, side_b;
    side_a.load(buf + lines * 32u - SIDEW, lane);
    side_b.load(buf + lines * 32u - SIDEW, lane + 32);
    typename ChainOf<PAIR_LAYOUT, IDXBITS>::type ca, cb;
    ca.init(buf + lane, kRingLogCopies - LOG_R);
    cb.init(buf + second * 32u + lane, kRingLogCopies - LOG_R);
    float tot_a[MR], tot_b[MR];
#pragma unroll
    for (int r = 0; r < MR; ++r) tot_a[r] = tot_b[r] = 0.f;
    auto finish_sub = [&](const int jj, const int (&acc_a)[MR], const int (&acc_b)[MR]) {
      float s_a, o_a, s_b, o_b;
      side_a.sub(jj, s_a, o_a);
      side_b.sub(jj, s_b, o_b);
#pragma unroll
      for (int r = 0; r < MR; ++r) {
        const float xsc = xst[jj * MR + r];
        const float fa = static_cast<float>(acc_a[r]) * xsc, fb = static_cast<float>(acc_b[r]) * xsc;
        if (HAS_OFFSET) {
          const float gx = xgt[jj * MR + r];
          tot_a[r] += s_a * fa - o_a * gx;
          tot_b[r] += s_b * fb - o_b * gx;
        } else {
          tot_a[r] = fmaf(s_a, fa, tot_a[r]);
          tot_b[r] = fmaf(s_b, fb, tot_b[r]);
        }
      }
    };
    if (PAIR_LAYOUT || cls == 0) {   // a pair layout has no other class
#pragma unroll
      for (int jj = 0; jj < NSU; ++jj) {
        int acc_a[MR], acc_b[MR];
#pragma unroll
        for (int r = 0; r < MR; ++r) acc_a[r] = acc_b[r] = 0;
        sub_block_m<G, SPG, MASK, MR>(ca, cb, smem, lane_off, xt + jj * SPG * MR, jj * SPG, jj == NSU - 1, acc_a, acc_b);
        finish_sub(jj, acc_a, acc_b);
      }
    } else if constexpr (!PAIR_LAYOUT) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        int acc_a[MR], acc_b[MR];
#pragma unroll
        for (int r = 0; r < MR; ++r) acc_a[r] = acc_b[r] = 0;
        if (cls == 1)
          sub_block_m<2, SPG, MASK, MR>(ca, cb, smem, lane_off, xt + jj * SPG * MR, jj * SPG, jj == 3, acc_a, acc_b);
        else
          sub_block_slow_m<SPG, MR>(ca, cb, tab1, LOG_R + 2, xt + jj * SPG * MR, acc_a, acc_b);
        finish_sub(jj, acc_a, acc_b);
      }
    }
    ring_release(RM, u, lane);
    float* prow = A.partials + static_cast<size_t>(tc * SPLIT + static_cast<int>(seg)) * m * M.N;
#pragma unroll
    for (int r = 0; r < MR; ++r)
      if (r < m) {
        prow[static_cast<size_t>(r) * M.N + na] = tot_a[r];
        prow[static_cast<size_t>(r) * M.N + nb] = tot_b[r];
      }
  }
}

}  // namespace lw
