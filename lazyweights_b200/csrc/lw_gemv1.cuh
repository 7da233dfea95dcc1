// Fused decode + dequant + matrix-vector product for ONE activation row (batch 1).  Included by lw_kernels.cu.
//
// Design, each point backed by a measured counter of an earlier variant (Q6_K 14336 x 4096, ncu on B200):
//  * 32-bit decode-table entries (lw::fat_table): the code length sits in the top four bits, so the bit position
//    advances with one multiply-high-and-add (FMA pipe, not the half-rate integer pipe), and the grid values of the
//    symbol are signed bytes that feed a dp2a instruction directly: no mask, no int-to-float conversion, and one
//    instruction for the two weights of a paired symbol (or for two consecutive symbols of an unpaired format).
//    The activations are re-quantised once per launch to 16-bit fixed point with one scale per sub-block (error at
//    most 2^-16 of the sub-block's largest |x|; the reference's default kernel uses 8 bits per 32, kernels/llmrt.cu:
//    1037-1055); products accumulate exactly in int32 inside a sub-block and in float32 across sub-blocks.
//    Together with the points below this took the loop from 19 to about 9 instructions per symbol.
//  * The table is replicated so that every lane reads its own bank: with one copy, 32 lanes looking up 32 pseudo-random
//    windows collide about 3.4 ways and the shared-memory pipe (one 128-byte wavefront per clock per SM) is the bound
//    (4.3 wavefronts per warp-symbol; 1.4 with the replicated table).
//      longest code <= 10 bits: 1024 windows x 32 lanes x 4 bytes = 128 KB, entry = (window << 7) | lane << 2
//      longest code == 11 bits: 2048 windows x 16 lanes x 4 bytes = 128 KB (lanes l and l + 16 share a bank pair)
//    Every chain starts with M.pad = 7 (or 6) zero bits, which puts the window on exactly those address bits of the
//    funnel-shifted word: the entry address is one AND.
//  * Refills are checked once per group of G symbols: the 64-bit window is normalised to the chain's bit position when
//    a group starts (two funnel shifts), the G symbols only add their lengths to a local offset, one predicated word
//    shift follows.  G x longest code <= 32 keeps that to one word per group.
//  * The chain words are staged in shared memory by bulk copies (cp.async.bulk + mbarrier), one per work unit, issued
//    by lane 0.  Reading them from global memory instead cannot be hidden: a register that is still being loaded
//    cannot be shifted along the window without waiting for it, and per-lane cp.async rings cost 6 more instructions
//    per symbol in divergent refill code.
//  * A work unit is one column segment of a tile (M.split segments per tile row): lane l decodes rows l and l + 32
//    over that segment as two independent chains that share their activations.  One persistent block per SM; units
//    are dealt round-robin over all warps of the grid, so that every SM gets the same share.
#pragma once
#include "lw_device.cuh"

namespace lw {

struct GroupChain {
  const uint32_t* p;
  uint32_t w0, w1, w2, bp;   // three stream words; bp < 32 between groups
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
  // next table entry; tab_lane = table base + this lane's bank offset; MASK selects the window's address bits
  template <uint32_t MASK>
  __device__ __forceinline__ uint32_t sym(const uint8_t* tab_lane) {
    const uint32_t t = __funnelshift_r(a, b, off);
    const uint32_t e = *reinterpret_cast<const uint32_t*>(tab_lane + (t & MASK));
    off = __umulhi(e, 16u) + off;   // e >> 28 = code length
    return e;
  }
  __device__ __forceinline__ void end() {
    bp += off;
    if (bp >= 32) {
      bp -= 32;
      w0 = w1;
      w1 = w2;
      w2 = *p;
      p += 32;
    }
  }
};

// One sub-block (SPG symbols) of both chains: acc_a / acc_b += sum x16 * v (exact, int32).  xq points at the
// sub-block's activations, packed as pairs of int16 (weight 2i in the low half of word i).
template <int FMT, int G, int SPG, uint32_t MASK>
__device__ __forceinline__ void sub_block(GroupChain& ca, GroupChain& cb, const uint8_t* tab_lane, const uint32_t* xq,
                                          int& acc_a, int& acc_b) {
  constexpr bool PAIR = is_paired(FMT);
  uint4 x = make_uint4(0u, 0u, 0u, 0u);
  uint32_t pa = 0, pb = 0;
#pragma unroll
  for (int c = 0; c < SPG; ++c) {
    if (c % G == 0) {
      ca.begin();
      cb.begin();
    }
    const uint32_t ea = ca.template sym<MASK>(tab_lane), eb = cb.template sym<MASK>(tab_lane);
    if (PAIR) {   // one symbol = weights 2c, 2c + 1 = word c of xq
      if (c % 4 == 0) x = *reinterpret_cast<const uint4*>(xq + c);
      const uint32_t xw = c % 4 == 0 ? x.x : c % 4 == 1 ? x.y : c % 4 == 2 ? x.z : x.w;
      acc_a = __dp2a_lo(static_cast<int>(xw), static_cast<int>(ea), acc_a);
      acc_b = __dp2a_lo(static_cast<int>(xw), static_cast<int>(eb), acc_b);
    } else if (c % 2 == 0) {
      pa = ea;
      pb = eb;
    } else {      // symbols c - 1, c = word (c - 1) / 2 of xq
      if ((c / 2) % 4 == 0) x = *reinterpret_cast<const uint4*>(xq + c / 2);
      const uint32_t xw = (c / 2) % 4 == 0 ? x.x : (c / 2) % 4 == 1 ? x.y : (c / 2) % 4 == 2 ? x.z : x.w;
      acc_a = __dp2a_lo(static_cast<int>(xw), static_cast<int>(__byte_perm(pa, ea, 0x0040)), acc_a);
      acc_b = __dp2a_lo(static_cast<int>(xw), static_cast<int>(__byte_perm(pb, eb, 0x0040)), acc_b);
    }
    if (c % G == G - 1 || c == SPG - 1) {
      ca.end();
      cb.end();
    }
  }
}

__device__ __forceinline__ uint32_t ldg_u32_2byte_aligned(const uint8_t* p) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
  return __ldg(h) | (static_cast<uint32_t>(__ldg(h + 1)) << 16);
}

// Side bytes of the NQ "quads" (four sub-blocks each) that one work unit of one row covers, loaded in one go when the
// unit starts.  Quads are consumed in order; next() rotates the raw words so that no register is indexed at run time.
// Q6_K: a quad = four int8 scales (one word); Q4_K / Q5_K: a super-block = two quads of 6-bit scales and mins
// (llama.cpp's get_scale_min_k4 packing), kept as its 16 raw bytes.
template <int FMT, int NQ>
struct UnitSide {
  static constexpr int kBlocks = NQ >= 2 ? NQ / 2 : 1;
  float d;
  uint32_t sc[NQ];
  uint4 w[kBlocks];   // IQ4_XS: x, y = the 8 side bytes of a super-block (fp16 d, scales_h; scales_l)
  // sp: side bytes of the row's first super-block in this tile; quad0: first quad of the unit within the tile row
  __device__ __forceinline__ void load(const uint8_t* sp, int quad0) {
    if (FMT == kFmtQ6K) {
      const uint8_t* blk = sp + (quad0 >> 2) * 18;
      d = half_bits_to_float(__ldg(reinterpret_cast<const uint16_t*>(blk + 16)));
#pragma unroll
      for (int q = 0; q < NQ; ++q) sc[q] = ldg_u32_2byte_aligned(blk + 4 * ((quad0 & 3) + q));
    } else if (FMT == kFmtIQ4XS) {
#pragma unroll
      for (int i = 0; i < kBlocks; ++i) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(sp) + (quad0 >> 1) + i);
        w[i] = make_uint4(v.x, v.y, 0u, 0u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kBlocks; ++i) w[i] = __ldg(reinterpret_cast<const uint4*>(sp) + (quad0 >> 1) + i);
    }
  }
  // (scale, offset) of sub-block j (0..3, a constant after unrolling) of the current quad; hi: second quad of its
  // super-block (Q4_K / Q5_K)
  __device__ __forceinline__ void sub(bool hi, int j, float& s, float& o) const {
    if (FMT == kFmtQ6K) {
      s = __fmul_rn(d, static_cast<float>(static_cast<int8_t>((sc[0] >> (8 * j)) & 255u)));
      o = 0.f;
    } else if (FMT == kFmtIQ4XS) {   // sub-block 4 hi + j of the super-block: 4-bit low part, 2-bit high part
      const uint4 v = w[0];
      const uint32_t lo = hi ? v.y >> 16 : v.y, h2 = hi ? v.x >> 24 : v.x >> 16;
      const uint32_t ls = ((lo >> (4 * j)) & 15u) | (((h2 >> (2 * j)) & 3u) << 4);
      s = __fmul_rn(half_bits_to_float(v.x), static_cast<float>(static_cast<int>(ls) - 32));
      o = 0.f;
    } else {
      const uint4 v = w[0];
      const uint32_t sc_lo = (v.y >> (8 * j)) & 63u, mn_lo = (v.z >> (8 * j)) & 63u;
      const uint32_t sc_hi = ((v.w >> (8 * j)) & 15u) | (((v.y >> (8 * j + 6)) & 3u) << 4);
      const uint32_t mn_hi = ((v.w >> (8 * j + 4)) & 15u) | (((v.z >> (8 * j + 6)) & 3u) << 4);
      s = __fmul_rn(half_bits_to_float(v.x), static_cast<float>(hi ? sc_hi : sc_lo));
      o = __fmul_rn(half_bits_to_float(v.x >> 16), static_cast<float>(hi ? mn_hi : mn_lo));
    }
  }
  __device__ __forceinline__ void next(bool hi) {
    if (FMT == kFmtQ6K) {
#pragma unroll
      for (int q = 0; q + 1 < NQ; ++q) sc[q] = sc[q + 1];
    } else if (hi) {
#pragma unroll
      for (int i = 0; i + 1 < kBlocks; ++i) w[i] = w[i + 1];
    }
  }
};

constexpr int kReplicatedTableBytes = 128 * 1024;
constexpr int kGemv1MaxWarps = 28;         // consumer warps; up to four more warps produce
constexpr int kGemv1MaxSlots = 64;         // staging buffers in the ring
constexpr int kGemv1MaxUnits = 512;        // work units one block can be dealt

struct Gemv1Args {
  const void* x;          // activations [K], fp16 or fp32
  float* partials;        // [KT * SPLIT][N]
  int x_is_half;
  int warps;              // consumer warps per block
  int producers;          // producer warps per block
  int prefetch;           // units pulled into L2 ahead of their copy (0 = none)
  int slots;              // staging buffers in the ring (>= warps)
  uint32_t buf_words;     // one staging buffer, in words
  int nsets;              // tile columns are dealt to `nsets` sets of blocks (bounds the staged activations)
  int cols_per_set;       // ceil(KT / nsets)
};

struct UnitMeta {
  uint32_t src;           // word offset of the unit's first group
  uint16_t lines;         // size of both groups in 128-byte lines (a group is a whole number of lines)
  uint16_t second;        // offset of the second group inside the unit, in lines
};

// Block = `warps` consumer warps + one producer warp.  The producer (one lane) walks the block's list of work units
// and, for each, waits until a staging buffer of the ring is free and starts the bulk copy of the unit's words into
// it; consumer warp c takes units c, c + warps, ... of the list, waits for the buffer to fill, decodes, and frees it.
// With more buffers than consumers the copies run ahead of the decoding, so no warp waits for DRAM in steady state.
// Every wait is bounded (mbar_wait): a warp that gives up sets the device error word and leaves.
template <int FMT, int G, int IDXBITS, int SPLIT>
__global__ void __launch_bounds__(1024, 1) k_gemv1(MatDev M, Gemv1Args A) {
  constexpr bool PAIR = is_paired(FMT);
  constexpr int TW = PAIR ? 2 * kTileSyms : kTileSyms;            // weights per tile row
  constexpr int GW = sub_width(FMT), SPG = PAIR ? GW / 2 : GW, SB = side_bytes(FMT);
  constexpr int NSU = TW / GW / SPLIT;                            // sub-blocks per unit
  constexpr int NQ = NSU / 4;                                     // quads per unit
  static_assert(NQ >= 1 && NSU % 4 == 0, "a unit must hold whole quads of sub-blocks");
  constexpr bool HAS_OFFSET = FMT == kFmtQ4K || FMT == kFmtQ5K;
  constexpr int LOG_R = IDXBITS == 10 ? 5 : 4;                    // copies of the table = 1 << LOG_R
  constexpr uint32_t MASK = IDXBITS == 10 ? 0x1FF80u : 0x1FFC0u;
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t* tab = reinterpret_cast<uint32_t*>(smem);
  uint32_t* xq = reinterpret_cast<uint32_t*>(smem + kReplicatedTableBytes);  // [cols_per_set][TW / 2] int16 pairs
  float* xscale = reinterpret_cast<float*>(xq + static_cast<size_t>(A.cols_per_set) * (TW / 2));   // [cols][TW / GW]
  float* xg = xscale + static_cast<size_t>(A.cols_per_set) * (TW / GW);      // [cols][TW / GW] sums (offset formats)
  uint64_t* full = reinterpret_cast<uint64_t*>(xg + (HAS_OFFSET ? A.cols_per_set * (TW / GW) : 0));
  uint64_t* empty = full + kGemv1MaxSlots;
  UnitMeta* meta = reinterpret_cast<UnitMeta*>(empty + kGemv1MaxSlots);      // [kGemv1MaxUnits]
  uint32_t* bufs = reinterpret_cast<uint32_t*>(meta + kGemv1MaxUnits);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int set = blockIdx.x % A.nsets, bi = blockIdx.x / A.nsets;
  const int nb_set = (gridDim.x - set + A.nsets - 1) / A.nsets;              // blocks of this set
  const int ncol = (M.KT - set + A.nsets - 1) / A.nsets;                     // tile columns of this set
  const int nunits = (M.N / kTileRows) * ncol * SPLIT;                       // units of this set
  const int nmine = bi < nunits ? (nunits - bi + nb_set - 1) / nb_set : 0;   // units of this block: bi + k nb_set

  // unit of the set -> (tile row, column index in the set, segment), segment fastest
  auto coords = [&](int u, int& tr, int& j, int& seg) {
    seg = u % SPLIT;
    const int v = u / SPLIT;
    j = v % ncol;
    tr = v / ncol;
  };

  // 1. every thread: where the block's units live (global loads in parallel), barriers
  for (int k = threadIdx.x; k < nmine; k += blockDim.x) {
    int tr, j, seg;
    coords(bi + k * nb_set, tr, j, seg);
    const int t = tr * M.KT + set + A.nsets * j;
    const uint32_t* gb = M.group_base + static_cast<size_t>(t) * (2 * SPLIT) + 2 * seg;
    const uint32_t g0 = __ldg(gb), g1 = __ldg(gb + 1), g2 = __ldg(gb + 2);
    meta[k] = UnitMeta{g0, static_cast<uint16_t>((g2 - g0) >> 5), static_cast<uint16_t>((g1 - g0) >> 5)};
  }
  if (threadIdx.x < A.slots) {
    mbar_init(smem_addr(full + threadIdx.x), 1);
    mbar_init(smem_addr(empty + threadIdx.x), 1);
  }
  __syncthreads();

  if (warp >= A.warps) {
    // 2a. producers: warp A.warps + i feeds units i, i + producers, ... of the block's list (one lane each: issuing a
    // bulk copy costs a few hundred cycles, so several lanes in different warps keep more copies in flight)
    if (lane == 0) {
      const int pw = warp - A.warps;
      // units further down the list are pulled into L2 ahead of time, so that their copy finds them there
      auto prefetch = [&](int k) {
        if (A.prefetch && k < nmine)
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(M.words + meta[k].src),
                       "r"(meta[k].lines * 128u)
                       : "memory");
      };
      for (int k = pw; k < nmine; k += A.producers) {
        const int slot = k % A.slots, round = k / A.slots;
        prefetch(k + A.prefetch);
        if (round > 0 && !mbar_wait(smem_addr(empty + slot), (round - 1) & 1)) return;
        const UnitMeta um = meta[k];
        bulk_load(smem_addr(bufs + static_cast<size_t>(slot) * A.buf_words), M.words + um.src, um.lines * 128u,
                  smem_addr(full + slot));
      }
    }
    return;
  }

  // 2b. consumers: table and activations first (the first copies are already on their way)
  const int nthr = A.warps * 32;
  {
    // replicate the table: a warp loads 32 entries with one coalesced read, then broadcasts them one by one and every
    // lane stores its own copy (bank = lane, no conflicts).  With 16 copies two entries go out per store.
    constexpr int NIDX = 1 << IDXBITS, PER = IDXBITS == 10 ? 1 : 2;
    for (int i0 = warp * 32; i0 < NIDX; i0 += A.warps * 32) {
      const uint32_t mine = __ldg(M.tab32 + i0 + lane);
#pragma unroll 8
      for (int j = 0; j < 32; j += PER) {
        const uint32_t v = __shfl_sync(0xffffffffu, mine, PER == 1 ? j : j + (lane >> 4));
        tab[(i0 + j) * (32 / PER) + lane] = v;
      }
    }
  }
  // activations -> 16-bit fixed point with one scale per sub-block (GW consecutive weights sit in GW consecutive
  // lanes).  Loads go out eight at a time so that their global-memory latencies overlap.
  constexpr int XB = 8;
  for (int base = 0; base < ncol * TW; base += XB * nthr) {
    float v[XB];
#pragma unroll
    for (int u = 0; u < XB; ++u) {
      const int i = base + u * nthr + threadIdx.x;
      v[u] = 0.f;
      if (i < ncol * TW) {
        const int j = i / TW, k = i - j * TW;
        const size_t src = static_cast<size_t>(set + A.nsets * j) * TW + k;
        v[u] = A.x_is_half ? __half2float(static_cast<const __half*>(A.x)[src]) : static_cast<const float*>(A.x)[src];
      }
    }
#pragma unroll
    for (int u = 0; u < XB; ++u) {
      const int i = base + u * nthr + threadIdx.x;
      if (i < ncol * TW) {   // whole warps take this branch together: sizes are multiples of 32
        float amax = fabsf(v[u]), sum = v[u];
#pragma unroll
        for (int o = 1; o < GW; o <<= 1) {
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          if (HAS_OFFSET) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        const int q = __float2int_rn(v[u] * (amax > 0.f ? 32767.f / amax : 0.f));
        const int qn = __shfl_down_sync(0xffffffffu, q, 1);
        if ((lane & 1) == 0) xq[i >> 1] = (static_cast<uint32_t>(q) & 0xFFFFu) | (static_cast<uint32_t>(qn) << 16);
        if ((lane & (GW - 1)) == 0) {
          xscale[i / GW] = amax * (1.f / 32767.f);
          if (HAS_OFFSET) xg[i / GW] = sum;
        }
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
  const uint8_t* tab_lane = smem + ((lane & ((1 << LOG_R) - 1)) << 2);
  const size_t side_row = static_cast<size_t>(M.K / 256) * SB;
  // side bytes of a unit's two rows: fetched one unit ahead (they come from DRAM in small strided pieces)
  auto side_ptrs = [&](int k, const uint8_t*& pa, const uint8_t*& pb, int& seg) {
    int tr, j;
    coords(bi + k * nb_set, tr, j, seg);
    const size_t col = static_cast<size_t>(set + A.nsets * j) * (TW / 256) * SB;
    pa = M.side + static_cast<size_t>(tr * kTileRows + lane) * side_row + col;
    pb = pa + 32 * side_row;
  };
  UnitSide<FMT, NQ> side_a, side_b, next_a, next_b;
  if (warp < nmine) {
    const uint8_t *pa, *pb;
    int sg;
    side_ptrs(warp, pa, pb, sg);
    side_a.load(pa, sg * NQ);
    side_b.load(pb, sg * NQ);
  }
#pragma unroll 1
  for (int k = warp; k < nmine; k += A.warps) {
    int tr, j, seg;
    coords(bi + k * nb_set, tr, j, seg);
    const int tc = set + A.nsets * j;
    const int na = tr * kTileRows + lane, nb = na + 32;
    if (k + A.warps < nmine) {
      const uint8_t *pa, *pb;
      int sg;
      side_ptrs(k + A.warps, pa, pb, sg);
      next_a.load(pa, sg * NQ);
      next_b.load(pb, sg * NQ);
    }
    const uint32_t* xt = xq + static_cast<size_t>(j) * (TW / 2) + seg * (TW / SPLIT / 2);
    const float* xst = xscale + static_cast<size_t>(j) * (TW / GW) + seg * NSU;
    const float* xgt = xg + static_cast<size_t>(j) * (TW / GW) + seg * NSU;
    const int slot = k % A.slots;
    const uint32_t* buf = bufs + static_cast<size_t>(slot) * A.buf_words;
    if (!mbar_wait(smem_addr(full + slot), (k / A.slots) & 1)) return;
    GroupChain ca, cb;
    ca.init(buf + lane);
    cb.init(buf + meta[k].second * 32u + lane);
    float tot_a = 0.f, tot_b = 0.f;
#pragma unroll 1
    for (int q = 0; q < NQ; ++q) {
      const bool hi = (seg * NQ + q) & 1;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int g = q * 4 + jj;
        int acc_a = 0, acc_b = 0;
        sub_block<FMT, G, SPG, MASK>(ca, cb, tab_lane, xt + g * (GW / 2), acc_a, acc_b);
        float s_a, o_a, s_b, o_b;
        side_a.sub(hi, jj, s_a, o_a);
        side_b.sub(hi, jj, s_b, o_b);
        const float xsc = xst[g];
        const float fa = static_cast<float>(acc_a) * xsc, fb = static_cast<float>(acc_b) * xsc;
        if (HAS_OFFSET) {
          const float gx = xgt[g];
          tot_a += s_a * fa - o_a * gx;
          tot_b += s_b * fb - o_b * gx;
        } else {
          tot_a = fmaf(s_a, fa, tot_a);
          tot_b = fmaf(s_b, fb, tot_b);
        }
      }
      side_a.next(hi);
      side_b.next(hi);
    }
    // every lane has read its last word: hand the buffer back to the producer
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(empty + slot)) : "memory");
    float* prow = A.partials + static_cast<size_t>(tc * SPLIT + seg) * M.N;
    prow[na] = tot_a;
    prow[nb] = tot_b;
    side_a = next_a;
    side_b = next_b;
  }
}

}  // namespace lw
