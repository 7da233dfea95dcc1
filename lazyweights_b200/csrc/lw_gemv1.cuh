// Fused decode + dequant + matrix-vector product for ONE activation row (batch 1).  Included by lw_gemv1.cu.
//
// The decoder (replicated 32-bit table, grouped refills, staging ring fed by producer warps, unit lists) is shared with
// the other persistent kernels: lw_ring.cuh.  What is specific to this kernel, each point backed by a measured counter
// of an earlier variant (Q6_K 14336 x 4096, ncu on B200):
//  * The grid values in a table entry are signed bytes that feed a dp2a instruction directly: no mask, no int-to-float
//    conversion, and one instruction per symbol (both weights of a paired symbol; an unpaired symbol meets an
//    activation word whose upper half is zero).  The activations are re-quantised once per launch to 16-bit fixed
//    point with one scale per sub-block (error at most 2^-16 of the sub-block's largest |x|; the reference's default
//    kernel uses 8 bits per 32, kernels/llmrt.cu:1037-1055); products accumulate exactly in int32 inside a sub-block
//    and in float32 across sub-blocks.
//  * The chain words are staged in shared memory by bulk copies (cp.async.bulk + mbarrier), one per work unit, issued
//    by a few lanes of dedicated producer warps.  Reading them from global memory instead cannot be hidden: a register
//    that is still being loaded cannot be shifted along the window without waiting for it, and per-lane cp.async rings
//    cost 6 more instructions per symbol in divergent refill code.
//  * A work unit is one column segment of a tile (default_split segments per tile row): lane l decodes rows l and
//    l + 32 over that segment as two independent chains that share their activations.  One persistent block per SM;
//    units are dealt round-robin over all warps of the grid, so that every SM gets the same share.
#pragma once
#include "lw_ring.cuh"

namespace lw {

// Multiply-accumulate of one decoded table entry with its activation word.  Paired formats: dp2a (two int16
// activations x the entry's two signed bytes).  Unpaired formats: one 32-bit multiply-add (the FMA pipe, which this
// kernel leaves mostly idle, instead of the half-rate integer pipe that bounds it): the entry carries its grid value
// sign-extended over bits 0-27 and the code length above, the activation is a sign-extended int16, so the low 28 bits of
// the running sum are exact (|sum| < 2^26 over a sub-block) whatever the length bits add on top; mac_result drops them.
template <bool PAIR>
__device__ __forceinline__ int mac(uint32_t xw, uint32_t e, int acc) {
  if (PAIR) return __dp2a_lo(static_cast<int>(xw), static_cast<int>(e), acc);
  return static_cast<int>(xw) * static_cast<int>(e) + acc;
}
template <bool PAIR>
__device__ __forceinline__ int mac_result(int acc) {
  return PAIR ? acc : static_cast<int>(static_cast<uint32_t>(acc) << 4) >> 4;
}

// One sub-block (SPG symbols) of both chains: acc_a / acc_b += sum x16 * v (exact, int32).  xq points at the
// sub-block's activation words (one per symbol: the int16 pair of a paired symbol's two weights, or one int16 in the
// low half).  `first` = index of the sub-block's first symbol within its quad (fixes the phase of the groups); `last`:
// the quad ends with this sub-block.
template <int G, int SPG, uint32_t MASK, bool PAIR, class CH>
__device__ __forceinline__ void sub_block(CH& ca, CH& cb, const uint8_t* tab, uint32_t lane_off,
                                          const uint32_t* xq, const int first, const bool last, int& acc_a,
                                          int& acc_b) {
  uint4 x = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int c = 0; c < SPG; ++c) {
    const int f = first + c;
    if (f % G == 0) {
      ca.begin();
      cb.begin();
    }
    const uint32_t ea = ca.template sym<MASK>(tab, lane_off), eb = cb.template sym<MASK>(tab, lane_off);
    if (c % 4 == 0) x = *reinterpret_cast<const uint4*>(xq + c);
    const uint32_t xw = c % 4 == 0 ? x.x : c % 4 == 1 ? x.y : c % 4 == 2 ? x.z : x.w;
    acc_a = mac<PAIR>(xw, ea, acc_a);
    acc_b = mac<PAIR>(xw, eb, acc_b);
    if (f % G == G - 1 || (last && c == SPG - 1)) {
      ca.end();
      cb.end();
    }
  }
}

template <int SPG, bool PAIR, class CH>
__device__ __forceinline__ void sub_block_slow(CH& ca, CH& cb, const uint32_t* tab32, uint32_t pad,
                                               const uint32_t* xq, int& acc_a, int& acc_b) {
#pragma unroll 2
  for (int c = 0; c < SPG; ++c) {
    const uint32_t ea = ca.slow_sym(tab32, pad), eb = cb.slow_sym(tab32, pad);
    const uint32_t xw = xq[c];
    acc_a = mac<PAIR>(xw, ea, acc_a);
    acc_b = mac<PAIR>(xw, eb, acc_b);
  }
}

// ------------------------------------------------------------------------------------------ alternative readers
//
// kReaderTable   the shipping decoder: replicated 32-bit table, one lookup per symbol (above)
// kReaderFixed   the fixed-width twin (lw::build_twin): codes at static bit positions, no table for the length and no
//                data-dependent shift - the same kernel without Huffman decoding, i.e. the upper bound of this design
//                (the reference's packed twins LaneR / LaneQ, kernels/llmrt.cu:543-630, play the same role)
// kReaderLimit   the comparator decoder of the reference's hardware unit (hw/huff/huff_engine.h:54-77,
//                hw/huff/rtl/huff_lane.sv:72-95): the window is bit-reversed, the code length comes from compares
//                against per-length limit registers, the symbol from a table indexed in canonical order, off the
//                length's dependency chain.  Built to be measured against the table form.
constexpr int kReaderTable = 0, kReaderFixed = 1, kReaderLimit = 2;

// Length of the code in window value v (11 bits, MSB first): 1 + the number of limits it reaches.
__device__ __forceinline__ uint32_t limit_length(uint32_t v, const uint32_t (&lim)[10]) {
  uint32_t len = 1;
#pragma unroll
  for (int l = 0; l < 10; ++l) len += v >= lim[l] ? 1u : 0u;
  return len;
}

// One symbol of a chain with the comparator decoder.  ctab: shared memory, [256][32] grid values in canonical order
// (copy = lane, no bank conflicts) followed by [12][32] index offsets per length; lane4 = lane * 4.
template <int PAD>
__device__ __forceinline__ uint32_t sym_limit(GroupChain& ch, const uint8_t* ctab, uint32_t lane4,
                                              const uint32_t (&lim)[10]) {
  const uint32_t t = __funnelshift_r(ch.a, ch.b, ch.off);
  const uint32_t v = (__brev(t) >> (21 - PAD)) & (kLutSize - 1);   // the window's 11 bits, first stream bit on top
  const uint32_t len = limit_length(v, lim);
  ch.off += len;
  const int adj = *reinterpret_cast<const int*>(ctab + 256 * 128 + ((len << 7) | lane4));
  const uint32_t idx = (v >> (kMaxLen - len)) + static_cast<uint32_t>(adj);
  return *reinterpret_cast<const uint32_t*>(ctab + (((idx & 255u) << 7) | lane4));
}

template <int G, int SPG, int PAD, bool PAIR>
__device__ __forceinline__ void sub_block_limit(GroupChain& ca, GroupChain& cb, const uint8_t* ctab, uint32_t lane4,
                                                const uint32_t (&lim)[10], const uint32_t* xq, const int first,
                                                const bool last, int& acc_a, int& acc_b) {
  uint4 x = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int c = 0; c < SPG; ++c) {
    const int f = first + c;
    if (f % G == 0) {
      ca.begin();
      cb.begin();
    }
    const uint32_t ea = sym_limit<PAD>(ca, ctab, lane4, lim), eb = sym_limit<PAD>(cb, ctab, lane4, lim);
    if (c % 4 == 0) x = *reinterpret_cast<const uint4*>(xq + c);
    const uint32_t xw = c % 4 == 0 ? x.x : c % 4 == 1 ? x.y : c % 4 == 2 ? x.z : x.w;
    acc_a = mac<PAIR>(xw, ea, acc_a);
    acc_b = mac<PAIR>(xw, eb, acc_b);
    if (f % G == G - 1 || (last && c == SPG - 1)) {
      ca.end();
      cb.end();
    }
  }
}

// One sub-block of both chains of a fixed-width twin.  wa / wb: the chains' words of this sub-block (word i at
// [32 i]); B bits per symbol; SPG * B is a whole number of words.  Paired symbols go through vtab ([256][32] grid
// value bytes, copy = lane); 6-bit codes are stored centred and sign-extended; 5-bit codes are their own grid value.
template <int FMT, int SPG>
__device__ __forceinline__ void sub_block_fixed(const uint32_t* wa, const uint32_t* wb, const uint8_t* vtab,
                                                uint32_t lane4, const uint32_t* xq, int& acc_a, int& acc_b) {
  constexpr int B = FMT == kFmtQ5K ? 5 : FMT == kFmtQ6K ? 6 : 8, NW = SPG * B / 32;
  static_assert(SPG * B % 32 == 0, "a sub-block is a whole number of words");
  uint32_t a[NW + 1], b[NW + 1];
#pragma unroll
  for (int i = 0; i < NW; ++i) {
    a[i] = wa[32 * i];
    b[i] = wb[32 * i];
  }
  a[NW] = b[NW] = 0u;
  uint4 x = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int c = 0; c < SPG; ++c) {
    constexpr uint32_t mask = (1u << B) - 1u;
    constexpr bool PAIR = is_paired(FMT);
    const int i = c * B / 32, s = c * B % 32;
    uint32_t va = s + B <= 32 ? a[i] >> s : __funnelshift_r(a[i], a[i + 1], s);
    uint32_t vb = s + B <= 32 ? b[i] >> s : __funnelshift_r(b[i], b[i + 1], s);
    uint32_t ea, eb;
    if (is_paired(FMT)) {
      ea = *reinterpret_cast<const uint32_t*>(vtab + (((va & mask) << 7) | lane4));
      eb = *reinterpret_cast<const uint32_t*>(vtab + (((vb & mask) << 7) | lane4));
    } else if (FMT == kFmtQ6K) {
      ea = static_cast<uint32_t>(static_cast<int>(va << (32 - B)) >> (32 - B));
      eb = static_cast<uint32_t>(static_cast<int>(vb << (32 - B)) >> (32 - B));
    } else {
      ea = va & mask;
      eb = vb & mask;
    }
    if (c % 4 == 0) x = *reinterpret_cast<const uint4*>(xq + c);
    const uint32_t xw = c % 4 == 0 ? x.x : c % 4 == 1 ? x.y : c % 4 == 2 ? x.z : x.w;
    acc_a = mac<PAIR>(xw, ea, acc_a);
    acc_b = mac<PAIR>(xw, eb, acc_b);
  }
}

constexpr int kGemv1LogCopies = kRingLogCopies;
constexpr int kGemv1MaxWarps = kRingMaxWarps;
constexpr int kGemv1MaxSlots = kRingMaxSlots;
constexpr int kGemv1MaxUnits = kRingMaxUnits;

struct Gemv1Args {
  RingArgs r;
  const void* x;          // activations [K], fp16 or fp32
  float* partials;        // [N / 64][KT][64]: per tile row, one 64-row partial product per tile
  float* y;               // [N] result
  int x_is_half;
  int helpers;            // warps that share the prologue (table, activations): the consumers and then some
  int pdl;                // launched as a programmatic dependent: the activations may only be read after pdl_wait
  int tile_ring_log2;     // the ring in which the segments of a tile meet holds 1 << tile_ring_log2 tiles
};

// A block's list is made of whole tiles: the SPLIT units of a tile are consecutive entries, decoded by different warps
// at about the same time.  Their totals meet in shared memory (a ring of 8 or 16 tiles); the warp that brings
// the last one adds them in segment order and writes ONE partial product per tile.  The warp that completes the last
// tile of a tile row (counted in M.row_done, which it resets) adds the row's partial products in a fixed order and
// writes the result: no second kernel, and the row sum is a single round trip to L2 for up to 16 tile columns.

// y[64 rows of one tile row] = sum over `terms` partial products, p[term][64].  Lane l adds rows 4 (l % 16) .. + 3 of
// the terms of its parity (l / 16) in ascending order, then the two parities are added: a fixed order.  Kept out of
// line so that it gets registers of its own: inlined into the decoder (64 registers, all in use) the loads were issued
// one at a time, one round trip to L2 (about 2000 cycles under load) each.
static __device__ __noinline__ void row_sum(const float* p, unsigned int terms, float* y, int lane) {
  const float4* q = reinterpret_cast<const float4*>(p) + lane;   // float4 i of the block: term i / 16, rows 4 (i % 16)
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const unsigned int steps = (terms + 1) / 2, parity = lane >> 4;   // two terms per step of 32 float4
  for (unsigned int s0 = 0; s0 < steps; s0 += 8) {
    float4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      v[i] = 2 * (s0 + i) + parity < terms ? __ldcg(q + static_cast<size_t>(s0 + i) * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc.x += v[i].x;
      acc.y += v[i].y;
      acc.z += v[i].z;
      acc.w += v[i].w;
    }
  }
  acc.x += __shfl_xor_sync(0xffffffffu, acc.x, 16);
  acc.y += __shfl_xor_sync(0xffffffffu, acc.y, 16);
  acc.z += __shfl_xor_sync(0xffffffffu, acc.z, 16);
  acc.w += __shfl_xor_sync(0xffffffffu, acc.w, 16);
  if (lane < 16) reinterpret_cast<float4*>(y)[lane] = acc;
}

#ifdef LW_GEMV1_PROFILE
// Built with -DLW_GEMV1_PROFILE, every consumer warp adds up the clock cycles it spends in the phases of its loop; the
// sums over all warps land here: [0] prologue, [1] drawing a unit and waiting for its copy, [2] decoding, [3] handing
// the buffer back and meeting the tile's other segments, [4] units, [5] final row sums, [6] whole loop, [7] warps.
// Read with lw_debug_prof (same build only).  Off by default: the clock reads cost a few instructions per unit.
__device__ unsigned long long g_gemv1_prof[8];
#endif
constexpr int kGemv1MaxTileRing = 16;   // tiles whose segments a block may be combining at one time (8 or 16)

// The work of one block: block `bidx` of the `nblocks` blocks that share matrix M.
template <int FMT, int G, int IDXBITS, int LOG_R, int READER>
__device__ __forceinline__ void gemv1_block(const MatDev& M, const Gemv1Args& A, const int bidx, const int nblocks) {
  constexpr bool PAIR = is_paired(FMT);
  constexpr int SPLIT = default_split(FMT);
  constexpr int TW = PAIR ? 2 * kTileSyms : kTileSyms;            // weights per tile row
  constexpr int GW = sub_width(FMT), SPG = sub_syms(FMT), SIDEW = unit_side_words(FMT);
  constexpr int NSU = TW / GW / SPLIT;                            // sub-blocks per unit
  constexpr int USYM = kTileSyms / SPLIT;                         // symbols (= activation words) per chain
  static_assert(NSU == 4 || NSU == 8, "a unit is four sub-blocks (eight of the 16-weight sub-blocks of a Q6_K pair layout)");
  constexpr bool PAIR_LAYOUT = is_pair_layout(FMT);
  static_assert(!PAIR_LAYOUT || READER == kReaderTable, "pair layouts are read through their table");
  constexpr bool HAS_OFFSET = FMT == kFmtQ4K || FMT == kFmtQ5K || FMT == kFmtQ5KP;
  constexpr int NIDX = 1 << IDXBITS, R = 1 << LOG_R;              // windows, copies of the table
  constexpr bool SINGLE = NIDX <= kLutSize;                       // a single-copy table of all 2048 windows beside it
  constexpr uint32_t MASK = static_cast<uint32_t>(NIDX - 1) << (LOG_R + 2);
  // the table area: the replicated Huffman table; or, for the other readers, [256][32] grid values (+ [12][32] offsets)
  constexpr int kReplicatedTableBytes = READER == kReaderTable ? NIDX * R * 4 : NIDX * R * 4 >= 34 * 1024 ? NIDX * R * 4 : 34 * 1024;
  extern __shared__ __align__(128) uint8_t smem[];
  const RingArgs& RA = A.r;
  uint32_t* tab = reinterpret_cast<uint32_t*>(smem);
  uint32_t* tab1 = reinterpret_cast<uint32_t*>(smem + kReplicatedTableBytes);  // [2048] single copy
  uint32_t* xq = tab1 + kLutSize;                                             // [cols_per_set][kTileSyms] words
  float* xscale = reinterpret_cast<float*>(xq + static_cast<size_t>(RA.cols_per_set) * kTileSyms);  // [cols][TW / GW]
  float* xg = xscale + static_cast<size_t>(RA.cols_per_set) * (TW / GW);      // [cols][TW / GW] sums (offset formats)
  const int ring = 1 << A.tile_ring_log2;
  uint32_t* tile_cnt = reinterpret_cast<uint32_t*>(xg + (HAS_OFFSET ? RA.cols_per_set * (TW / GW) : 0));   // [ring] segments finished, cumulative
  uint32_t* tile_free = tile_cnt + ring;                                     // [ring] generations handed back
  float* tile_acc = reinterpret_cast<float*>(tile_free + ring);              // [ring][SPLIT][64] unit totals
  RingMem RM;
  RM.carve(tile_acc + ring * SPLIT * kTileRows, RA);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  BlockShare S;
  S.init(M, RA, SPLIT, bidx, nblocks);
  const int set = S.set, ncol = S.ncol, nmine = S.nmine;
  pdl_trigger();   // the next kernel of the stream may be set up while this one runs (it waits before it reads)
#ifdef LW_GEMV1_PROFILE
  const long long prof_t0 = clock64();
  long long prof_wait = 0, prof_dec = 0, prof_tail = 0, prof_units = 0;
#endif
  const bool consumer = warp < A.helpers;   // takes part in the prologue; warps >= RA.warps leave after it
  const int nthr = A.helpers * 32;

  // 1. everything the prologue needs from global memory is requested at once: table entries and the first activations
  // (consumers), then where the block's units live (all threads)
  // The registers stay exactly as loaded until after the barriers below: converting or moving one earlier would make
  // the warp wait for its load right here.
  constexpr int TAB_PRE = 3, T1_PRE = 2, XB = 6;
  uint32_t tab_pre[TAB_PRE], t1_pre[T1_PRE], xraw[XB];
  auto load_x = [&](int base) {
#pragma unroll
    for (int u = 0; u < XB; ++u) {
      const int i = base + u * nthr + threadIdx.x;
      xraw[u] = 0u;
      if (i < ncol * TW) {
        const int j = i / TW, k = i - j * TW;
        const size_t src = static_cast<size_t>(set + RA.nsets * j) * TW + k;
        if (A.x_is_half)
          xraw[u] = static_cast<const unsigned short*>(A.x)[src];
        else
          xraw[u] = static_cast<const uint32_t*>(A.x)[src];
      }
    }
  };
  auto x_value = [&](uint32_t raw) {
    return A.x_is_half ? __half2float(__ushort_as_half(static_cast<unsigned short>(raw))) : __uint_as_float(raw);
  };
  if (consumer) {
    if (READER == kReaderTable) {
#pragma unroll
      for (int i = 0; i < TAB_PRE; ++i) {
        const int idx = (i * A.helpers + warp) * 32 + lane;
        tab_pre[i] = idx < NIDX ? __ldg(M.tab32 + idx) : 0u;
      }
#pragma unroll
      for (int i = 0; i < T1_PRE; ++i) {   // windows beyond the replicated table (single-copy table only)
        const int idx = NIDX + i * nthr + static_cast<int>(threadIdx.x);
        t1_pre[i] = idx < kLutSize ? __ldg(M.tab32 + idx) : 0u;
      }
    }
    if (!A.pdl) load_x(0);
  }
  if (threadIdx.x < ring) {
    tile_cnt[threadIdx.x] = 0u;
    tile_free[threadIdx.x] = 0u;
  }
  ring_reset(RM);
  __syncthreads();
  ring_build_list<SPLIT>(M, RA, S, RM);
  __syncthreads();

  if (!consumer) {
    ring_produce(M, RA, RM, nmine, warp - A.helpers, lane);   // 2a. producers
    return;
  }

  // 2b. consumers: table and activations (the first copies are already on their way).
  uint32_t lim[10] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
  if (READER == kReaderTable) {
#pragma unroll
    for (int i = 0; i < TAB_PRE; ++i) {
      const int i0 = (i * A.helpers + warp) * 32;
      if (i0 < NIDX) table_spread<LOG_R, SINGLE>(tab, tab1, i0, tab_pre[i], lane);
    }
    for (int i0 = (TAB_PRE * A.helpers + warp) * 32; i0 < NIDX; i0 += A.helpers * 32)
      table_spread<LOG_R, SINGLE>(tab, tab1, i0, __ldg(M.tab32 + i0 + lane), lane);
#pragma unroll
    for (int i = 0; i < T1_PRE; ++i) {
      const int idx = NIDX + i * nthr + static_cast<int>(threadIdx.x);
      if (idx < kLutSize) tab1[idx] = t1_pre[i];
    }
    for (int idx = NIDX + T1_PRE * nthr + static_cast<int>(threadIdx.x); idx < kLutSize; idx += nthr)
      tab1[idx] = __ldg(M.tab32 + idx);
  } else {
    // [256][32] grid values (entry i of the source in every lane's own bank) and, for the comparator decoder, the
    // [12][32] offsets behind them and the ten limits in registers
    const uint32_t* src = READER == kReaderLimit ? M.cmp_tab + 24 : M.tab32;
    const bool need_values = READER == kReaderLimit || PAIR;
    for (int i = warp; need_values && i < 256; i += A.helpers) tab[i * 32 + lane] = __ldg(src + i);
    if (READER == kReaderLimit) {
      for (int i = warp; i < 12; i += A.helpers) tab[(256 + i) * 32 + lane] = __ldg(M.cmp_tab + 12 + i);
#pragma unroll
      for (int l = 0; l < 10; ++l) lim[l] = __ldg(M.cmp_tab + 1 + l);
    }
  }
  // Everything up to here read only the matrix (tables, list, and the producers' copies of chain words): with a
  // programmatic launch it overlaps the tail of the previous kernel in the stream, which may still be writing x.
  if (A.pdl) pdl_wait();
  // activations -> 16-bit fixed point with one scale per sub-block (GW consecutive weights sit in GW consecutive
  // lanes).  Loads go out XB at a time so that their global-memory latencies overlap.
  for (int base = 0; base < ncol * TW; base += XB * nthr) {
    if (base > 0 || A.pdl) load_x(base);
#pragma unroll
    for (int u = 0; u < XB; ++u) {
      const int i = base + u * nthr + threadIdx.x;
      if (i < ncol * TW) {   // whole warps take this branch together: sizes are multiples of 32
        const float xvu = x_value(xraw[u]);
        float amax = fabsf(xvu), sum = xvu;
#pragma unroll
        for (int o = 1; o < GW; o <<= 1) {
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          if (HAS_OFFSET) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        const int q = __float2int_rn(xvu * (amax > 0.f ? 32767.f / amax : 0.f));
        if (PAIR) {
          const int qn = __shfl_down_sync(0xffffffffu, q, 1);
          if ((lane & 1) == 0) xq[i >> 1] = (static_cast<uint32_t>(q) & 0xFFFFu) | (static_cast<uint32_t>(qn) << 16);
        } else {
          xq[i] = static_cast<uint32_t>(q);   // sign-extended: the operand of a 32-bit multiply-add
        }
        if ((lane & (GW - 1)) == 0) {
          xscale[i / GW] = amax * (1.f / 32767.f);
          if (HAS_OFFSET) xg[i / GW] = sum;
        }
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
  if (warp >= RA.warps) return;
  const uint32_t lane_off = (lane & (R - 1)) << 2;
  const unsigned int terms = static_cast<unsigned int>(M.KT);   // partial products per tile row: one per tile
  // The warp that finishes the last unit of a tile row adds the row's partial products.  Counting a unit needs its
  // partial products to be visible first, and the count takes a round trip to L2 (about 2000 cycles each under load).
  // Both hide inside the decoding of the warp's next unit: the unit is counted (cnt_tr) after that one's first
  // sub-block, when its stores have long landed, and the answer (pend_tr, pend_done) is looked at after the third.
  constexpr unsigned int kNone = 0xFFFFFFFFu;
  unsigned int cnt_tr = kNone, pend_tr = 0, pend_done = kNone;
  auto resolve = [&]() {
    const unsigned int done = __shfl_sync(0xffffffffu, pend_done, 0);
    if (done == terms - 1u) {
      __syncwarp();   // orders the loads below after lane 0's acquire; they bypass L1 (ld.cg)
      row_sum(A.partials + static_cast<size_t>(pend_tr) * terms * kTileRows, terms, A.y + pend_tr * kTileRows, lane);
      if (lane == 0) M.row_done[pend_tr * kRowDoneStride] = 0u;
    }
    pend_done = kNone;
  };
  // lane 0 releases (at GPU scope) the stores that the warp barrier ordered before it, and counts the unit
  auto count = [&]() {
    resolve();
    if (cnt_tr != kNone) {
      __syncwarp();
      pend_tr = cnt_tr;
      if (lane == 0)
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(pend_done) : "l"(M.row_done + cnt_tr * kRowDoneStride) : "memory");
      cnt_tr = kNone;
    }
  };
#ifdef LW_GEMV1_PROFILE
  const long long prof_t1 = clock64();
#endif
#pragma unroll 1
  for (;;) {
    Unit u;
#ifdef LW_GEMV1_PROFILE
    const long long pfa = clock64();
#endif
    const int got = ring_draw(RA, RM, nmine, lane, u);
    if (got == 0) break;
    if (got < 0) return;
#ifdef LW_GEMV1_PROFILE
    const long long pfb = clock64();
    prof_wait += pfb - pfa;
    ++prof_units;
#endif
    const uint32_t j = u.j, seg = u.seg, tr = u.tr, cls = u.cls;
    const int tc = set + RA.nsets * static_cast<int>(j);
    const uint32_t* xt = xq + static_cast<size_t>(j) * kTileSyms + seg * USYM;
    const float* xst = xscale + static_cast<size_t>(j) * (TW / GW) + seg * NSU;
    const float* xgt = xg + static_cast<size_t>(j) * (TW / GW) + seg * NSU;
    const uint32_t* buf = u.buf;
    UnitSide<FMT> side_a, side_b;
    side_a.load(buf + u.lines * 32u - SIDEW, lane);
    side_b.load(buf + u.lines * 32u - SIDEW, lane + 32);
    typename ChainOf<PAIR_LAYOUT, IDXBITS>::type ca, cb;
    ca.init(buf + lane, kRingLogCopies - LOG_R);
    cb.init(buf + u.second * 32u + lane, kRingLogCopies - LOG_R);
    float tot_a = 0.f, tot_b = 0.f;
    // scales of sub-block jj applied to its exact integer sums; the previous unit is counted on the way (see above)
    auto finish_sub = [&](const int jj, int acc_a, int acc_b) {
      float s_a, o_a, s_b, o_b;
      side_a.sub(jj, s_a, o_a);
      side_b.sub(jj, s_b, o_b);
      if (jj == 0) count();
      if (jj == 2) resolve();
      const float xsc = xst[jj];
      const float fa = static_cast<float>(mac_result<PAIR>(acc_a)) * xsc, fb = static_cast<float>(mac_result<PAIR>(acc_b)) * xsc;
      if (HAS_OFFSET) {
        const float gx = xgt[jj];
        tot_a += s_a * fa - o_a * gx;
        tot_b += s_b * fb - o_b * gx;
      } else {
        tot_a = fmaf(s_a, fa, tot_a);
        tot_b = fmaf(s_b, fb, tot_b);
      }
    };
    // The common class has its four sub-blocks to itself, so that its code is contiguous: 28 warps at different
    // program counters share the instruction cache (`no_instruction` stalls were 0.9 per issued instruction with the
    // fallback bodies interleaved).
    if constexpr (READER == kReaderFixed) {
      constexpr int NW = SPG * (FMT == kFmtQ5K ? 5 : FMT == kFmtQ6K ? 6 : 8) / 32;   // words per sub-block and chain
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        int acc_a = 0, acc_b = 0;
        sub_block_fixed<FMT, SPG>(buf + lane + jj * NW * 32, buf + u.second * 32u + lane + jj * NW * 32, smem,
                                  static_cast<uint32_t>(lane) << 2, xt + jj * SPG, acc_a, acc_b);
        finish_sub(jj, acc_a, acc_b);
      }
    } else if constexpr (READER == kReaderLimit) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        int acc_a = 0, acc_b = 0;
        if (cls == 0)
          sub_block_limit<G, SPG, LOG_R + 2, PAIR>(ca, cb, smem, static_cast<uint32_t>(lane) << 2, lim, xt + jj * SPG,
                                             jj * SPG, jj == 3, acc_a, acc_b);
        else   // units where groups of G symbols are not exact: groups of two, exact for any data
          sub_block_limit<2, SPG, LOG_R + 2, PAIR>(ca, cb, smem, static_cast<uint32_t>(lane) << 2, lim, xt + jj * SPG,
                                             jj * SPG, jj == 3, acc_a, acc_b);
        finish_sub(jj, acc_a, acc_b);
      }
    } else if (PAIR_LAYOUT || cls == 0) {   // a pair layout has no other class
#pragma unroll
      for (int jj = 0; jj < NSU; ++jj) {
        int acc_a = 0, acc_b = 0;
        sub_block<G, SPG, MASK, PAIR>(ca, cb, smem, lane_off, xt + jj * SPG, jj * SPG, jj == NSU - 1, acc_a, acc_b);
        finish_sub(jj, acc_a, acc_b);
      }
    } else if constexpr (!PAIR_LAYOUT) {
#pragma unroll
      for (int jj = 0; jj < NSU; ++jj) {
        int acc_a = 0, acc_b = 0;
        if (cls == 1)
          sub_block<2, SPG, MASK, PAIR>(ca, cb, smem, lane_off, xt + jj * SPG, jj * SPG, jj == NSU - 1, acc_a, acc_b);
        else
          sub_block_slow<SPG, PAIR>(ca, cb, tab1, LOG_R + 2, xt + jj * SPG, acc_a, acc_b);
        finish_sub(jj, acc_a, acc_b);
      }
    }
#ifdef LW_GEMV1_PROFILE
    const long long pfc = clock64();
    prof_dec += pfc - pfb;
#endif
    ring_release(RM, u, lane);
    // the unit's totals meet those of the tile's other segments in shared memory
    constexpr int LOG_SPLIT = SPLIT == 8 ? 3 : SPLIT == 4 ? 2 : SPLIT == 2 ? 1 : 0;
    static_assert((1 << LOG_SPLIT) == SPLIT, "power of two");
    const uint32_t tl = static_cast<uint32_t>(u.k) >> LOG_SPLIT, ts = tl & (ring - 1), tgen = tl >> A.tile_ring_log2;
    if (!wait_released(tile_free + ts, tgen, RA.err, RA.wait_limit)) return;   // the ring slot's previous tile has been handed back
    float* ta = tile_acc + (ts * SPLIT + seg) * kTileRows;
    ta[lane] = tot_a;
    ta[lane + 32] = tot_b;
    __syncwarp();
    uint32_t arrived = 0;
    if (lane == 0)
      asm volatile("atom.add.acq_rel.cta.shared::cta.u32 %0, [%1], 1;" : "=r"(arrived) : "r"(smem_addr(tile_cnt + ts)) : "memory");
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (arrived == tgen * SPLIT + (SPLIT - 1)) {   // last segment of the tile: add them in segment order
      __syncwarp();
      float pa = 0.f, pb = 0.f;
#pragma unroll
      for (int sg = 0; sg < SPLIT; ++sg) {
        pa += tile_acc[(ts * SPLIT + sg) * kTileRows + lane];
        pb += tile_acc[(ts * SPLIT + sg) * kTileRows + lane + 32];
      }
      __syncwarp();
      if (lane == 0)
        asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_addr(tile_free + ts)), "r"(tgen + 1u) : "memory");
      float* prow = A.partials + (static_cast<size_t>(tr) * terms + tc) * kTileRows;
      prow[lane] = pa;
      prow[lane + 32] = pb;
      cnt_tr = tr;
    }
#ifdef LW_GEMV1_PROFILE
    prof_tail += clock64() - pfc;
#endif
  }
#ifdef LW_GEMV1_PROFILE
  const long long prof_t2 = clock64();
#endif
  count();
  resolve();
#ifdef LW_GEMV1_PROFILE
  if (lane == 0) {
    atomicAdd(&g_gemv1_prof[0], static_cast<unsigned long long>(prof_t1 - prof_t0));
    atomicAdd(&g_gemv1_prof[1], static_cast<unsigned long long>(prof_wait));
    atomicAdd(&g_gemv1_prof[2], static_cast<unsigned long long>(prof_dec));
    atomicAdd(&g_gemv1_prof[3], static_cast<unsigned long long>(prof_tail));
    atomicAdd(&g_gemv1_prof[4], static_cast<unsigned long long>(prof_units));
    atomicAdd(&g_gemv1_prof[5], static_cast<unsigned long long>(clock64() - prof_t2));
    atomicAdd(&g_gemv1_prof[6], static_cast<unsigned long long>(prof_t2 - prof_t1));
    atomicAdd(&g_gemv1_prof[7], 1ull);
  }
#endif
}

template <int FMT, int G, int IDXBITS, int LOG_R, int READER = kReaderTable>
__global__ void __launch_bounds__(1024, 1) k_gemv1(const __grid_constant__ MatDev M, const __grid_constant__ Gemv1Args A) {
  gemv1_block<FMT, G, IDXBITS, LOG_R, READER>(M, A, blockIdx.x, gridDim.x);
}

// Several products in ONE launch: matrix j (its own activations, scratch and result) is worked on by blocks
// first[j] .. first[j + 1] - 1 of the grid.  Every block still serves a single matrix - one decode table, one unit list -
// but a block's list is several times longer than when the whole grid shares one matrix: the set-up and the tail of a
// launch are paid once for all the products, and warps that run out of units are a smaller share of the launch
// (one matrix on 148 blocks of 28 warps gives a warp 3.5 units; eight matrices in one launch give it 28).
// All matrices of a launch share the kernel's template parameters (format, group size, table width).
constexpr int kGemv1MaxBatch = 8;
struct Gemv1Batch {
  MatDev mat[kGemv1MaxBatch];
  Gemv1Args arg[kGemv1MaxBatch];
  int first[kGemv1MaxBatch + 1];
  int count;
};

template <int FMT, int G, int IDXBITS, int LOG_R>
__global__ void __launch_bounds__(1024, 1) k_gemv1_batch(const __grid_constant__ Gemv1Batch B) {
  int j = 0;
#pragma unroll 1
  while (j + 1 < B.count && static_cast<int>(blockIdx.x) >= B.first[j + 1]) ++j;
  gemv1_block<FMT, G, IDXBITS, LOG_R, kReaderTable>(B.mat[j], B.arg[j], blockIdx.x - B.first[j], B.first[j + 1] - B.first[j]);
}

}  // namespace lw
