// Fused decode + dequant + matrix-vector product for ONE activation row (batch 1).  Included by lw_gemv1.cu.
//
// Design, each point backed by a measured counter of an earlier variant (Q6_K 14336 x 4096, ncu on B200):
//  * 32-bit decode-table entries (lw::fat_table): the code length sits in the top four bits, so the bit position
//    advances with one multiply-high-and-add (FMA pipe, not the half-rate integer pipe), and the grid values of the
//    symbol are signed bytes that feed a dp2a instruction directly: no mask, no int-to-float conversion, and one
//    instruction per symbol (both weights of a paired symbol; an unpaired symbol meets an activation word whose upper
//    half is zero).  The activations are re-quantised once per launch to 16-bit fixed point with one scale per
//    sub-block (error at most 2^-16 of the sub-block's largest |x|; the reference's default kernel uses 8 bits per 32,
//    kernels/llmrt.cu:1037-1055); products accumulate exactly in int32 inside a sub-block and in float32 across
//    sub-blocks.
//  * The table is replicated so that lanes read their own banks: with one copy, 32 lanes looking up 32 pseudo-random
//    windows collide about 3.4 ways and the shared-memory pipe (one 128-byte wavefront per clock per SM) is the bound.
//    R = 2^LOG_R copies of a table of 2^IDXBITS windows (10 bits if few work units hold an 11-bit code, else 11):
//    entry address = (window << (LOG_R + 2)) | (lane % R) << 2.  With 32 copies no two lanes share a bank; with 16
//    (8) copies two (four) lanes share a copy and collide when their windows agree modulo 32 / R (about 1.5 and 2.1
//    wavefronts per lookup), in exchange for 64 KB more staging buffers, i.e. more warps in flight.
//    Every chain starts with M.pad = LOG_R + 2 zero bits, which puts the window on exactly those address bits of the
//    funnel-shifted word: the entry address is one three-input logic operation (mask, then OR the lane's offset).
//  * Refills are checked once per group of G symbols: the 64-bit window is normalised to the chain's bit position when
//    a group starts (two funnel shifts), the G symbols only add their lengths to a local offset, one predicated word
//    shift follows.  That is exact only while every symbol of a group starts within 31 bits of the group and one word
//    per group keeps up; the loader (lw::walk_blob) checks both for every chain of the matrix, picks the largest G that
//    leaves few exceptions, and flags the work units that hold one: those run with groups of two symbols, which is
//    exact for any data.  With the 10-bit table, a unit that holds an 11-bit code is decoded symbol by symbol through
//    a single-copy table of all 2048 windows (8 KB of shared memory).
//  * The chain words are staged in shared memory by bulk copies (cp.async.bulk + mbarrier), one per work unit, issued
//    by a few lanes of dedicated producer warps.  Reading them from global memory instead cannot be hidden: a register
//    that is still being loaded cannot be shifted along the window without waiting for it, and per-lane cp.async rings
//    cost 6 more instructions per symbol in divergent refill code.
//  * A work unit is one column segment of a tile (default_split segments per tile row): lane l decodes rows l and
//    l + 32 over that segment as two independent chains that share their activations.  One persistent block per SM;
//    units are dealt round-robin over all warps of the grid, so that every SM gets the same share.
#pragma once
#include "lw_device.cuh"

namespace lw {

struct GroupChain {
  const uint32_t* p;
  uint32_t w0, w1, w2, bp;   // three stream words; bp = bits consumed so far (its low five bits place the window)
  uint32_t a, b, off;        // window normalised to bp, offset inside the group
  __device__ __forceinline__ void init(const uint32_t* chain_words) {
    w0 = chain_words[0];
    w1 = chain_words[32];
    w2 = chain_words[64];
    p = chain_words + 96;
    bp = 0;
  }
  __device__ __forceinline__ void begin() {
    a = __funnelshift_r(w0, w1, bp);
    b = __funnelshift_r(w1, w2, bp);
    off = 0;
  }
  // next table entry; tab = replicated table (start of shared memory), lane_off = this lane's byte offset inside the
  // copies of one window, MASK selects the window's address bits
  template <uint32_t MASK>
  __device__ __forceinline__ uint32_t sym(const uint8_t* tab, uint32_t lane_off) {
    const uint32_t t = __funnelshift_r(a, b, off);
    const uint32_t e = *reinterpret_cast<const uint32_t*>(tab + ((t & MASK) | lane_off));
    off = __umulhi(e, 16u) + off;   // e >> 28 = code length
    return e;
  }
  __device__ __forceinline__ void refill() {
    w0 = w1;
    w1 = w2;
    w2 = *p;
    p += 32;
  }
  // bp is a running bit count: the funnel shifts only look at its low five bits, and a word was used up exactly when
  // bit 5 changed (the loader guarantees at most one word per group)
  __device__ __forceinline__ void end() {
    const uint32_t nb = bp + off;
    if ((nb ^ bp) & 32u) refill();
    bp = nb;
  }
  // symbol by symbol, any data: tab32 = the single-copy table (shared memory)
  __device__ __forceinline__ uint32_t slow_sym(const uint32_t* tab32, uint32_t pad) {
    const uint32_t e = tab32[(__funnelshift_r(w0, w1, bp) >> pad) & (kLutSize - 1)];
    const uint32_t nb = bp + (e >> 28);
    if ((nb ^ bp) & 32u) refill();
    bp = nb;
    return e;
  }
};

// One sub-block (SPG symbols) of both chains: acc_a / acc_b += sum x16 * v (exact, int32).  xq points at the
// sub-block's activation words (one per symbol: the int16 pair of a paired symbol's two weights, or one int16 in the
// low half).  `first` = index of the sub-block's first symbol within its quad (fixes the phase of the groups); `last`:
// the quad ends with this sub-block.
template <int G, int SPG, uint32_t MASK>
__device__ __forceinline__ void sub_block(GroupChain& ca, GroupChain& cb, const uint8_t* tab, uint32_t lane_off,
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
    acc_a = __dp2a_lo(static_cast<int>(xw), static_cast<int>(ea), acc_a);
    acc_b = __dp2a_lo(static_cast<int>(xw), static_cast<int>(eb), acc_b);
    if (f % G == G - 1 || (last && c == SPG - 1)) {
      ca.end();
      cb.end();
    }
  }
}

template <int SPG>
__device__ __forceinline__ void sub_block_slow(GroupChain& ca, GroupChain& cb, const uint32_t* tab32, uint32_t pad,
                                               const uint32_t* xq, int& acc_a, int& acc_b) {
#pragma unroll 2
  for (int c = 0; c < SPG; ++c) {
    const uint32_t ea = ca.slow_sym(tab32, pad), eb = cb.slow_sym(tab32, pad);
    const uint32_t xw = xq[c];
    acc_a = __dp2a_lo(static_cast<int>(xw), static_cast<int>(ea), acc_a);
    acc_b = __dp2a_lo(static_cast<int>(xw), static_cast<int>(eb), acc_b);
  }
}

// Scales of the unit's two rows (row `lane` and row `lane + 32`), read from the block that follows the unit's chain
// words in its staging buffer (layout: lw::unit_side_words).  sub(j) = (scale, offset) of sub-block j (a constant
// after unrolling): weight = scale * f(code) - offset, every operation rounded separately in float32 (llama.cpp's
// block formulas; reference: scripts/a2_kq_bundle.py:50-68, kernels/llmrt.cu:126-149).
template <int FMT>
struct UnitSide {
  uint32_t sc, mn, dd;
  __device__ __forceinline__ void load(const uint32_t* sb, int row) {
    if (FMT == kFmtQ4K || FMT == kFmtQ5K) {
      dd = sb[row];
      sc = sb[64 + row];
      mn = sb[128 + row];
    } else {
      sc = sb[row];
      dd = reinterpret_cast<const uint16_t*>(sb)[128 + row];
      mn = 0;
    }
  }
  __device__ __forceinline__ void sub(int j, float& s, float& o) const {
    const uint32_t q = (sc >> (8 * j)) & 255u;
    if (FMT == kFmtQ6K) {
      s = __fmul_rn(half_bits_to_float(dd), static_cast<float>(static_cast<int8_t>(q)));
      o = 0.f;
    } else if (FMT == kFmtIQ4XS) {
      s = __fmul_rn(half_bits_to_float(dd), static_cast<float>(static_cast<int>(q) - 32));
      o = 0.f;
    } else {
      s = __fmul_rn(half_bits_to_float(dd), static_cast<float>(q));
      o = __fmul_rn(half_bits_to_float(dd >> 16), static_cast<float>((mn >> (8 * j)) & 255u));
    }
  }
};

constexpr int kGemv1LogCopies = 4;         // 16 copies of the table: 64 KB (1024 windows) or 128 KB (2048)
constexpr int kGemv1MaxWarps = 28;         // consumer warps; up to four more warps produce
constexpr int kGemv1MaxSlots = 64;         // staging buffers in the ring
constexpr int kGemv1MaxUnits = 1024;       // work units one block can be dealt

struct Gemv1Args {
  const void* x;          // activations [K], fp16 or fp32
  float* partials;        // [N / 64][KT][64]: per tile row, one 64-row partial product per tile
  float* y;               // [N] result
  unsigned int* err;      // device error word (bit 0: a bounded wait gave up)
  int x_is_half;
  int warps;              // consumer warps per block
  int helpers;            // warps that share the prologue (table, activations): the consumers and then some
  int producers;          // producer warps per block
  int producer_lanes;     // lanes of a producer warp that issue copies
  int slots;              // staging buffers in the ring (>= warps)
  uint32_t buf_words;     // one staging buffer, in words
  int nsets;              // tile columns are dealt to `nsets` sets of blocks (bounds the staged activations)
  int cols_per_set;       // ceil(KT / nsets)
  int max_units;          // capacity of the block's unit list (>= units of any block, multiple of 2)
  int pdl;                // launched as a programmatic dependent: the activations may only be read after pdl_wait
  int tile_ring_log2;     // the ring in which the segments of a tile meet holds 1 << tile_ring_log2 tiles
};

struct UnitMeta {          // 16 bytes: one shared-memory load per unit
  uint32_t src;           // word offset of the unit's first group
  uint16_t lines;         // size of both groups in 128-byte lines (a group is a whole number of lines)
  uint16_t second;        // offset of the second group inside the unit, in lines; bits 14-15: unit class (0 = groups
                          // of G symbols, 1 = groups of two, 2 = symbol by symbol)
  uint16_t tr;            // tile row
  uint16_t round;         // use of its staging buffer: unit index / slots
  uint8_t j, seg, slot;   // tile column within the block's set, column segment, staging buffer: unit index % slots
  uint8_t unused;
};
static_assert(sizeof(UnitMeta) == 16, "UnitMeta is read as one 16-byte word");

// Block = `warps` consumer warps + `producers` producer warps.  Unit k of the block's list goes through staging
// buffer k % slots ("round" k / slots of that buffer).  Producer lanes each own a subset of the buffers and, round
// after round, wait until a buffer is free and start the bulk copy of its next unit; a consumer warp draws the next
// unit of the list from a shared counter, waits for the buffer to fill, decodes, and frees it.  With more buffers
// than consumers the copies run ahead of the decoding, so no warp waits for DRAM in steady state.
// Everything a unit needs (coordinates, buffer, round) is worked out once, in parallel, when the block starts: the
// per-unit path has no integer division.
// A block's list is made of whole tiles: the SPLIT units of a tile are consecutive entries, decoded by different warps
// at about the same time.  Their totals meet in shared memory (a ring of 8 or 16 tiles); the warp that brings
// the last one adds them in segment order and writes ONE partial product per tile.  The warp that completes the last
// tile of a tile row (counted in M.row_done, which it resets) adds the row's partial products in a fixed order and
// writes the result: no second kernel, and the row sum is a single round trip to L2 for up to 16 tile columns.
// A parity wait on an mbarrier is only exact for a waiter that is at most one phase away, and here the waiters of
// consecutive rounds of a buffer are different threads.  So every buffer also has a plain counter of the rounds that
// were released: both sides first wait until it reaches their round (exact at any distance), after which the
// barrier is known to be in the phase the parity wait assumes.
// Every wait is bounded: a warp that gives up sets the device error word and leaves.
__device__ __forceinline__ bool wait_released(const uint32_t* released, uint32_t round, unsigned int* err) {
  const uint32_t addr = smem_addr(released);
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    if (v >= round) return true;
    __nanosleep(100);   // do not take issue slots from the warps this one is waiting for
  }
  atomicOr(err, 1u);
  return false;
}

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

constexpr int kGemv1MaxTileRing = 16;   // tiles whose segments a block may be combining at one time (8 or 16)

template <int FMT, int G, int IDXBITS, int LOG_R>
__global__ void __launch_bounds__(1024, 1) k_gemv1(MatDev M, Gemv1Args A) {
  constexpr bool PAIR = is_paired(FMT);
  constexpr int SPLIT = default_split(FMT);
  constexpr int TW = PAIR ? 2 * kTileSyms : kTileSyms;            // weights per tile row
  constexpr int GW = sub_width(FMT), SPG = sub_syms(FMT), SIDEW = unit_side_words(FMT);
  constexpr int NSU = TW / GW / SPLIT;                            // sub-blocks per unit
  constexpr int USYM = kTileSyms / SPLIT;                         // symbols (= activation words) per chain
  static_assert(NSU == 4, "a unit is one quad of sub-blocks");
  constexpr bool HAS_OFFSET = FMT == kFmtQ4K || FMT == kFmtQ5K;
  constexpr int NIDX = 1 << IDXBITS, R = 1 << LOG_R;              // windows, copies of the table
  constexpr uint32_t MASK = static_cast<uint32_t>(NIDX - 1) << (LOG_R + 2);
  constexpr int kReplicatedTableBytes = NIDX * R * 4;
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t* tab = reinterpret_cast<uint32_t*>(smem);
  uint32_t* tab1 = reinterpret_cast<uint32_t*>(smem + kReplicatedTableBytes);  // [2048] single copy
  uint32_t* xq = tab1 + kLutSize;                                             // [cols_per_set][kTileSyms] words
  float* xscale = reinterpret_cast<float*>(xq + static_cast<size_t>(A.cols_per_set) * kTileSyms);  // [cols][TW / GW]
  float* xg = xscale + static_cast<size_t>(A.cols_per_set) * (TW / GW);      // [cols][TW / GW] sums (offset formats)
  uint64_t* full = reinterpret_cast<uint64_t*>(xg + (HAS_OFFSET ? A.cols_per_set * (TW / GW) : 0));
  uint64_t* empty = full + kGemv1MaxSlots;
  uint32_t* released = reinterpret_cast<uint32_t*>(empty + kGemv1MaxSlots);  // [slots] rounds released so far
  int* next_unit = reinterpret_cast<int*>(released + kGemv1MaxSlots);        // the list's shared counter
  int* list_count = next_unit + 1;                                           // [2] slow / other tiles placed so far
  uint32_t* tile_cnt = reinterpret_cast<uint32_t*>(next_unit + 4);           // [ring] segments finished, cumulative
  const int ring = 1 << A.tile_ring_log2;
  uint32_t* tile_free = tile_cnt + ring;                                     // [ring] generations handed back
  float* tile_acc = reinterpret_cast<float*>(tile_free + ring);              // [ring][SPLIT][64] unit totals
  UnitMeta* meta = reinterpret_cast<UnitMeta*>(tile_acc + ring * SPLIT * kTileRows);   // [max_units]
  uint32_t* bufs = reinterpret_cast<uint32_t*>(meta + A.max_units);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int set = blockIdx.x % A.nsets, bi = blockIdx.x / A.nsets;
  const int nb_set = (gridDim.x - set + A.nsets - 1) / A.nsets;              // blocks of this set
  const int ncol = (M.KT - set + A.nsets - 1) / A.nsets;                     // tile columns of this set
  const int ntiles = (M.N / kTileRows) * ncol;                               // tiles of this set
  const int tmine = bi < ntiles ? (ntiles - bi + nb_set - 1) / nb_set : 0;   // tiles of this block: bi + k nb_set
  const int nmine = tmine * SPLIT;                                           // its units
  pdl_trigger();   // the next kernel of the stream may be set up while this one runs (it waits before it reads)
  const bool consumer = warp < A.helpers;   // takes part in the prologue; warps >= A.warps leave after it
  const int nthr = A.helpers * 32;

  // tile of the set -> (tile row, column index in the set)
  auto coords = [&](int v, int& tr, int& j) {
    j = v % ncol;
    tr = v / ncol;
  };

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
        const size_t src = static_cast<size_t>(set + A.nsets * j) * TW + k;
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
    if (!A.pdl) load_x(0);
  }
  // The block's list: tiles bi, bi + nb_set, ... of the set, their SPLIT units in segment order, with the tiles
  // that hold a symbol-by-symbol unit moved to the front (such a unit takes several times longer: started last, it
  // would keep the whole block waiting).  The order within the two classes is whatever the counters hand out; results
  // do not depend on it.
  if (threadIdx.x < ring) {
    tile_cnt[threadIdx.x] = 0u;
    tile_free[threadIdx.x] = 0u;
  }
  if (threadIdx.x == 0) {
    list_count[0] = 0;
    list_count[1] = 0;
    *next_unit = 0;
  }
  __syncthreads();
  for (int k0 = warp * 32; k0 < nmine; k0 += (blockDim.x >> 5) * 32) {
    const int k = k0 + lane, seg = lane % SPLIT;
    const bool valid = k < nmine, leader = seg == 0;
    int tr = 0, j = 0;
    uint32_t g0 = 0, g1 = 0, g2 = 0, cls = 0;
    bool slow = false;
    if (valid) {
      coords(bi + (k / SPLIT) * nb_set, tr, j);
      const int t = tr * M.KT + set + A.nsets * j;
      const uint32_t* gb = M.group_base + static_cast<size_t>(t) * (2 * SPLIT) + 2 * seg;
      g0 = __ldg(gb);
      g1 = __ldg(gb + 1);
      g2 = __ldg(gb + 2);
      const uint8_t* uc = M.unit_slow + static_cast<size_t>(t) * SPLIT;
      cls = __ldg(uc + seg);
#pragma unroll
      for (int i = 0; i < SPLIT; ++i) slow |= __ldg(uc + i) == 2;
    }
    const uint32_t bs = __ballot_sync(0xffffffffu, valid && leader && slow);
    const uint32_t bf = __ballot_sync(0xffffffffu, valid && leader && !slow);
    int base_s = 0, base_f = 0;
    if (lane == 0) {
      base_s = atomicAdd(list_count, __popc(bs));
      base_f = atomicAdd(list_count + 1, __popc(bf));
    }
    base_s = __shfl_sync(0xffffffffu, base_s, 0);
    base_f = __shfl_sync(0xffffffffu, base_f, 0);
    const uint32_t below = (1u << lane) - 1u;
    int tpos = slow ? base_s + __popc(bs & below) : tmine - 1 - (base_f + __popc(bf & below));
    tpos = __shfl_sync(0xffffffffu, tpos, lane - seg);   // the tile's position, from its leader
    if (valid) {
      const int pos = tpos * SPLIT + seg;
      meta[pos] = UnitMeta{g0,
                           static_cast<uint16_t>((g2 - g0) >> 5),
                           static_cast<uint16_t>(((g1 - g0) >> 5) | (cls << 14)),
                           static_cast<uint16_t>(tr),
                           static_cast<uint16_t>(pos / A.slots),
                           static_cast<uint8_t>(j),
                           static_cast<uint8_t>(seg),
                           static_cast<uint8_t>(pos % A.slots),
                           0};
    }
  }
  if (threadIdx.x < A.slots) {
    mbar_init(smem_addr(full + threadIdx.x), 1);
    mbar_init(smem_addr(empty + threadIdx.x), 1);
    released[threadIdx.x] = 0u;
  }
  __syncthreads();

  if (!consumer) {
    // 2a. producers: issuer s = (producer warp) * producer_lanes + lane owns buffers s, s + S, ... (S issuers) and
    // feeds them round by round, i.e. in the order of the block's list.  Issuing a bulk copy takes a few hundred
    // cycles, so several issuers keep more copies in flight.
    if (lane < A.producer_lanes) {
      const int issuers = A.producers * A.producer_lanes;
      for (int round = 0; round * A.slots < nmine; ++round)
        for (int slot = (warp - A.helpers) * A.producer_lanes + lane; slot < A.slots; slot += issuers) {
          const int k = round * A.slots + slot;
          if (k >= nmine) break;
          if (round > 0) {
            if (!wait_released(released + slot, round, A.err)) return;
            if (!mbar_wait(smem_addr(empty + slot), (round - 1) & 1, A.err)) return;
          }
          const UnitMeta um = meta[k];
          bulk_load(smem_addr(bufs + static_cast<size_t>(slot) * A.buf_words), M.words + um.src, um.lines * 128u,
                    smem_addr(full + slot));
        }
    }
    return;
  }

  // 2b. consumers: table and activations (the first copies are already on their way).
  // Replicate the table: a warp holds 32 entries, broadcasts them one by one and every lane stores its own copy
  // (bank = lane, no conflicts).  With 16 copies two entries go out per store.
  {
    constexpr int PER = 32 / R;   // entries per store: lane l writes copy l % R of entry i0 + j + l / R
    auto spread = [&](int i0, uint32_t mine) {
#pragma unroll 8
      for (int j = 0; j < 32; j += PER) {
        const uint32_t v = __shfl_sync(0xffffffffu, mine, j + (lane >> LOG_R));
        tab[(i0 + j) * R + lane] = v;
      }
      tab1[i0 + lane] = mine;
    };
#pragma unroll
    for (int i = 0; i < TAB_PRE; ++i) {
      const int i0 = (i * A.helpers + warp) * 32;
      if (i0 < NIDX) spread(i0, tab_pre[i]);
    }
    for (int i0 = (TAB_PRE * A.helpers + warp) * 32; i0 < NIDX; i0 += A.helpers * 32) spread(i0, __ldg(M.tab32 + i0 + lane));
  }
#pragma unroll
  for (int i = 0; i < T1_PRE; ++i) {
    const int idx = NIDX + i * nthr + static_cast<int>(threadIdx.x);
    if (idx < kLutSize) tab1[idx] = t1_pre[i];
  }
  for (int idx = NIDX + T1_PRE * nthr + static_cast<int>(threadIdx.x); idx < kLutSize; idx += nthr)
    tab1[idx] = __ldg(M.tab32 + idx);
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
          xq[i] = static_cast<uint32_t>(q) & 0xFFFFu;
        }
        if ((lane & (GW - 1)) == 0) {
          xscale[i / GW] = amax * (1.f / 32767.f);
          if (HAS_OFFSET) xg[i / GW] = sum;
        }
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
  if (warp >= A.warps) return;
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
#pragma unroll 1
  for (;;) {
    int k = 0;
    if (lane == 0) k = atomicAdd(next_unit, 1);
    k = __shfl_sync(0xffffffffu, k, 0);
    if (k >= nmine) break;
    const uint4 raw = *reinterpret_cast<const uint4*>(meta + k);
    const uint32_t lines = raw.y & 0xFFFFu, second = raw.y >> 16, tr = raw.z & 0xFFFFu, round = raw.z >> 16;
    const uint32_t j = raw.w & 255u, seg = (raw.w >> 8) & 255u, slot = (raw.w >> 16) & 255u;
    const uint32_t cls = second >> 14;
    const int tc = set + A.nsets * static_cast<int>(j);
    const uint32_t* xt = xq + static_cast<size_t>(j) * kTileSyms + seg * USYM;
    const float* xst = xscale + static_cast<size_t>(j) * (TW / GW) + seg * NSU;
    const float* xgt = xg + static_cast<size_t>(j) * (TW / GW) + seg * NSU;
    const uint32_t* buf = bufs + static_cast<size_t>(slot) * A.buf_words;
    if (round > 0 && !wait_released(released + slot, round, A.err)) return;
    if (!mbar_wait(smem_addr(full + slot), round & 1, A.err)) return;
    UnitSide<FMT> side_a, side_b;
    side_a.load(buf + lines * 32u - SIDEW, lane);
    side_b.load(buf + lines * 32u - SIDEW, lane + 32);
    GroupChain ca, cb;
    ca.init(buf + lane);
    cb.init(buf + (second & 0x3FFFu) * 32u + lane);
    float tot_a = 0.f, tot_b = 0.f;
    // scales of sub-block jj applied to its exact integer sums; the previous unit is counted on the way (see above)
    auto finish_sub = [&](const int jj, int acc_a, int acc_b) {
      float s_a, o_a, s_b, o_b;
      side_a.sub(jj, s_a, o_a);
      side_b.sub(jj, s_b, o_b);
      if (jj == 0) count();
      if (jj == 2) resolve();
      const float xsc = xst[jj];
      const float fa = static_cast<float>(acc_a) * xsc, fb = static_cast<float>(acc_b) * xsc;
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
    if (cls == 0) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        int acc_a = 0, acc_b = 0;
        sub_block<G, SPG, MASK>(ca, cb, smem, lane_off, xt + jj * SPG, jj * SPG, jj == 3, acc_a, acc_b);
        finish_sub(jj, acc_a, acc_b);
      }
    } else {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        int acc_a = 0, acc_b = 0;
        if (cls == 1)
          sub_block<2, SPG, MASK>(ca, cb, smem, lane_off, xt + jj * SPG, jj * SPG, jj == 3, acc_a, acc_b);
        else
          sub_block_slow<SPG>(ca, cb, tab1, static_cast<uint32_t>(M.pad), xt + jj * SPG, acc_a, acc_b);
        finish_sub(jj, acc_a, acc_b);
      }
    }
    // every lane has read its last word: hand the buffer back to the producer
    __syncwarp();
    if (lane == 0) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(empty + slot)) : "memory");
      asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_addr(released + slot)), "r"(round + 1u) : "memory");
    }
    // the unit's totals meet those of the tile's other segments in shared memory
    constexpr int LOG_SPLIT = SPLIT == 4 ? 2 : SPLIT == 2 ? 1 : 0;
    static_assert((1 << LOG_SPLIT) == SPLIT, "power of two");
    const uint32_t tl = static_cast<uint32_t>(k) >> LOG_SPLIT, ts = tl & (ring - 1), tgen = tl >> A.tile_ring_log2;
    if (!wait_released(tile_free + ts, tgen, A.err)) return;   // the ring slot's previous tile has been handed back
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
  }
  count();
  resolve();
}

}  // namespace lw
