// Fused decode + dequant + matrix-vector product for ONE activation row (batch 1).  Included by lw_kernels.cu.
//
// Design, each point backed by a measured counter of an earlier variant (Q6_K 14336 x 4096, ncu on B200):
//  * 32-bit decode-table entries (lw::fat_table): the code length sits in the top four bits, so the bit position
//    advances with one multiply-high-and-add (FMA pipe, not the half-rate integer pipe), and the symbol's grid value is
//    stored as a bf16 float, so a weight costs one shift (plus one mask for the first nibble of a pair).  This took the
//    loop from 19 to 10 instructions per symbol.
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

template <int FMT>
__device__ __forceinline__ float fat_first(uint32_t e) {   // grid value of the symbol (or of its low nibble)
  if (FMT == kFmtQ4K) return __uint_as_float((e << 4) & 0xFFF00000u);
  return __uint_as_float(e << 16);
}
__device__ __forceinline__ float fat_second(uint32_t e) { return __uint_as_float(e << 16); }   // high nibble

// One sub-block (SPG symbols) of both chains: acc_a / acc_b += x . f(q).  xq points at the sub-block's activations.
template <int FMT, int G, int SPG, uint32_t MASK>
__device__ __forceinline__ void sub_block(GroupChain& ca, GroupChain& cb, const uint8_t* tab_lane, const float* xq,
                                          float& acc_a, float& acc_b) {
  constexpr bool PAIR = is_paired(FMT);
  float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int c = 0; c < SPG; ++c) {
    if (c % G == 0) {
      ca.begin();
      cb.begin();
    }
    const uint32_t ea = ca.template sym<MASK>(tab_lane), eb = cb.template sym<MASK>(tab_lane);
    if (PAIR) {
      if (c % 2 == 0) x = *reinterpret_cast<const float4*>(xq + 2 * c);
      const float x0 = c % 2 == 0 ? x.x : x.z, x1 = c % 2 == 0 ? x.y : x.w;
      acc_a = fmaf(x0, fat_first<FMT>(ea), acc_a);
      acc_b = fmaf(x0, fat_first<FMT>(eb), acc_b);
      acc_a = fmaf(x1, fat_second(ea), acc_a);
      acc_b = fmaf(x1, fat_second(eb), acc_b);
    } else {
      if (c % 4 == 0) x = *reinterpret_cast<const float4*>(xq + c);
      const float xv = c % 4 == 0 ? x.x : c % 4 == 1 ? x.y : c % 4 == 2 ? x.z : x.w;
      acc_a = fmaf(xv, fat_first<FMT>(ea), acc_a);
      acc_b = fmaf(xv, fat_first<FMT>(eb), acc_b);
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
  uint4 w[kBlocks];
  // sp: side bytes of the row's first super-block in this tile; quad0: first quad of the unit within the tile row
  __device__ __forceinline__ void load(const uint8_t* sp, int quad0) {
    if (FMT == kFmtQ6K) {
      const uint8_t* blk = sp + (quad0 >> 2) * 18;
      d = half_bits_to_float(__ldg(reinterpret_cast<const uint16_t*>(blk + 16)));
#pragma unroll
      for (int q = 0; q < NQ; ++q) sc[q] = ldg_u32_2byte_aligned(blk + 4 * ((quad0 & 3) + q));
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
constexpr int kGemv1MaxWarps = 16;

struct Gemv1Args {
  const void* x;          // activations [K], fp16 or fp32
  float* partials;        // [KT * SPLIT][N]
  int x_is_half;
  int warps;              // warps per block (<= kGemv1MaxWarps)
  uint32_t buf_words;     // staging buffer of one warp, in words
  int nsets;              // tile columns are dealt to `nsets` sets of blocks (bounds the staged activations)
  int cols_per_set;       // ceil(KT / nsets)
};

// Units of a set: (tile row tr, column j of the set, segment seg), enumerated seg-fastest.
template <int FMT, int G, int IDXBITS, int SPLIT>
__global__ void __launch_bounds__(kGemv1MaxWarps * 32, 1) k_gemv1(MatDev M, Gemv1Args A) {
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
  float* xs = reinterpret_cast<float*>(smem + kReplicatedTableBytes);        // [cols_per_set][TW]
  float* xg = xs + static_cast<size_t>(A.cols_per_set) * TW;                 // [cols_per_set][TW / GW]
  uint64_t* bars = reinterpret_cast<uint64_t*>(xg + (HAS_OFFSET ? A.cols_per_set * (TW / GW) : 0));
  uint32_t* bufs = reinterpret_cast<uint32_t*>(bars + kGemv1MaxWarps);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int set = blockIdx.x % A.nsets, bi = blockIdx.x / A.nsets;
  const int nb_set = (gridDim.x - set + A.nsets - 1) / A.nsets;              // blocks of this set
  const int ncol = (M.KT - set + A.nsets - 1) / A.nsets;                     // tile columns of this set
  const int NT = M.N / kTileRows;
  const int nunits = NT * ncol * SPLIT;
  uint32_t* buf = bufs + static_cast<size_t>(warp) * A.buf_words;
  const uint32_t bar_a = smem_addr(bars + warp);

  // unit -> coordinates
  auto coords = [&](int u, int& tr, int& j, int& seg) {
    seg = u % SPLIT;
    const int v = u / SPLIT;
    j = v % ncol;
    tr = v / ncol;
  };
  // start the bulk copy of unit u into this warp's buffer (lane 0)
  auto stage = [&](int u, uint32_t& gb0, uint32_t& gb1) {
    int tr, j, seg;
    coords(u, tr, j, seg);
    const int t = tr * M.KT + set + A.nsets * j;
    const uint32_t* gb = M.group_base + static_cast<size_t>(t) * (2 * SPLIT) + 2 * seg;
    gb0 = __ldg(gb);
    gb1 = __ldg(gb + 1);
    const uint32_t end = __ldg(gb + 2);
    if (lane == 0) bulk_load(smem_addr(buf), M.words + gb0, (end - gb0) * 4u, bar_a);
  };

  int u = warp * nb_set + bi;
  const int ustride = A.warps * nb_set;
  uint32_t gb0 = 0, gb1 = 0;
  if (lane == 0) mbar_init(bar_a, 1);
  __syncwarp();
  if (u < nunits) stage(u, gb0, gb1);   // first copy overlaps the table and activation staging

  for (int i = threadIdx.x; i < kReplicatedTableBytes / 4; i += blockDim.x) tab[i] = __ldg(M.tab32 + (i >> LOG_R));
  for (int i = threadIdx.x; i < ncol * TW; i += blockDim.x) {
    const int j = i / TW, k = i - j * TW;
    const size_t src = static_cast<size_t>(set + A.nsets * j) * TW + k;
    xs[i] = A.x_is_half ? __half2float(static_cast<const __half*>(A.x)[src]) : static_cast<const float*>(A.x)[src];
  }
  __syncthreads();
  if (HAS_OFFSET) {
    for (int g = threadIdx.x; g < ncol * (TW / GW); g += blockDim.x) {
      float a = 0.f;
      for (int k = 0; k < GW; ++k) a += xs[g * GW + k];
      xg[g] = a;
    }
    __syncthreads();
  }
  const uint8_t* tab_lane = smem + ((lane & ((1 << LOG_R) - 1)) << 2);
  const size_t side_row = static_cast<size_t>(M.K / 256) * SB;
  uint32_t parity = 0;
#pragma unroll 1
  for (; u < nunits; u += ustride) {
    int tr, j, seg;
    coords(u, tr, j, seg);
    const int tc = set + A.nsets * j;
    const int na = tr * kTileRows + lane, nb = na + 32;
    const uint8_t* sa = M.side + na * side_row + static_cast<size_t>(tc) * (TW / 256) * SB;
    const uint8_t* sb_ = M.side + nb * side_row + static_cast<size_t>(tc) * (TW / 256) * SB;
    UnitSide<FMT, NQ> side_a, side_b;
    side_a.load(sa, seg * NQ);
    side_b.load(sb_, seg * NQ);
    const float* xt = xs + static_cast<size_t>(j) * TW + seg * (TW / SPLIT);
    const float* xgt = xg + static_cast<size_t>(j) * (TW / GW) + seg * NSU;
    if (!mbar_wait(bar_a, parity)) return;
    parity ^= 1u;
    GroupChain ca, cb;
    ca.init(buf + lane);
    cb.init(buf + (gb1 - gb0) + lane);
    float tot_a = 0.f, tot_b = 0.f;
#pragma unroll 1
    for (int q = 0; q < NQ; ++q) {
      const bool hi = (seg * NQ + q) & 1;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int g = q * 4 + jj;
        float acc_a = 0.f, acc_b = 0.f;
        sub_block<FMT, G, SPG, MASK>(ca, cb, tab_lane, xt + g * GW, acc_a, acc_b);
        float s_a, o_a, s_b, o_b;
        side_a.sub(hi, jj, s_a, o_a);
        side_b.sub(hi, jj, s_b, o_b);
        if (HAS_OFFSET) {
          const float gx = xgt[g];
          tot_a += s_a * acc_a - o_a * gx;
          tot_b += s_b * acc_b - o_b * gx;
        } else {
          tot_a = fmaf(s_a, acc_a, tot_a);
          tot_b = fmaf(s_b, acc_b, tot_b);
        }
      }
      side_a.next(hi);
      side_b.next(hi);
    }
    float* prow = A.partials + static_cast<size_t>(tc * SPLIT + seg) * M.N;
    prow[na] = tot_a;
    prow[nb] = tot_b;
    // the buffer is free once every lane has read its last word; then the next unit's copy may overwrite it
    __syncwarp();
    if (u + ustride < nunits) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      stage(u + ustride, gb0, gb1);
    }
  }
}

}  // namespace lw
