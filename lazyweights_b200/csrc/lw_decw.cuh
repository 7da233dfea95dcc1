// Decode + block dequantisation to fp16 weights with the batch-1 kernel's decoder (lw_gemv1.cuh): replicated 32-bit
// table, grouped refills chosen from the data, unit scales staged with the chains, producer warps feeding a ring of
// staging buffers, units drawn from a shared counter.  Instead of dot products every decoded grid value becomes
// w = s * f(q) - o in float32 (product and difference rounded separately, llama.cpp's block formulas; reference:
// scripts/a2_kq_bundle.py:50-68) and one round to fp16; a lane produces the weights of its two rows 32 bytes at a time,
// which leave through the warp's staging area and a 2-D tensor copy (WarpTileStage, lw_ring.cuh) or, without it, as one
// 32-byte store per lane and row.  Included by lw_decw.cu.
#pragma once
#include "lw_gemv1.cuh"

namespace lw {

struct DecwArgs {
  RingArgs r;       // r.tr0, r.ntr: tile rows to decode
  __half* out;      // [ntr * 64][K]
};

// Collects sixteen weights of one chain: one 32-byte piece of a row.  flush() is the plain-store form (a whole sector:
// a lane writes to its own row, so every store instruction touches 32 different lines, and 16-byte pieces paid for a
// full sector each).
struct HalfPack {
  uint32_t w[8];
  __device__ __forceinline__ void put(int i, float lo, float hi) {   // halfs 2 i, 2 i + 1 of the current sixteen
    const __half2 h = __floats2half2_rn(lo, hi);   // one conversion instruction for both, each rounded to nearest even
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  __device__ __forceinline__ void flush(__half* dst) const {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
  }
};

__device__ __forceinline__ float grid_of_entry(uint32_t e, int which) {
  return static_cast<float>(static_cast<int>(static_cast<int8_t>((e >> (8 * which)) & 255u)));
}

// TILE_OUT: the weights leave through shared memory and the tensor-copy engine (WarpTileStage; TM = the tensor map of the
// launch's output rows) instead of 32-byte stores
template <int FMT, int G, int IDXBITS, int LOG_R, bool TILE_OUT>
__global__ void __launch_bounds__(1024, 1) k_decw(const __grid_constant__ MatDev M, const __grid_constant__ DecwArgs A,
                                                  const __grid_constant__ CUtensorMap TM) {
  const RingArgs& RA = A.r;
  constexpr bool PAIR = is_paired(FMT);
  constexpr int SPLIT = default_split(FMT);
  constexpr int TW = PAIR ? 2 * kTileSyms : kTileSyms;
  constexpr int GW = sub_width(FMT), SPG = sub_syms(FMT), SIDEW = unit_side_words(FMT);
  constexpr int NSU = TW / GW / SPLIT;   // sub-blocks per unit: four, or eight 16-weight ones of a Q6_K pair layout
  constexpr bool PAIR_LAYOUT = is_pair_layout(FMT);
  constexpr int NIDX = 1 << IDXBITS, R = 1 << LOG_R;
  constexpr bool SINGLE = NIDX <= kLutSize;
  constexpr uint32_t MASK = static_cast<uint32_t>(NIDX - 1) << (LOG_R + 2);
  constexpr int kReplicatedTableBytes = NIDX * R * 4;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint32_t* tab = reinterpret_cast<uint32_t*>(smem);
  uint32_t* tab1 = reinterpret_cast<uint32_t*>(smem + kReplicatedTableBytes);
  uint8_t* stage0 = reinterpret_cast<uint8_t*>(tab1 + kLutSize);   // [warps][2 KB] when TILE_OUT; 1024-byte aligned
  RingMem RM;
  RM.carve(stage0 + (TILE_OUT ? RA.warps * WarpTileStage::kBytes : 0), RA);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TableLoad<IDXBITS, LOG_R, SINGLE> table;
  table.issue(M.tab32, warp, lane, RA.warps);
  BlockShare S;
  S.init(M, RA, SPLIT, blockIdx.x, gridDim.x);   // one column set (nsets = 1): there are no activations to stage
  const int nmine = S.nmine;
  const bool consumer = warp < RA.warps;
  const int nthr = RA.warps * 32;

  // 1. the block's list (whole tiles, symbol-by-symbol tiles first) and the ring's barriers
  ring_reset(RM);
  __syncthreads();
  ring_build_list<SPLIT>(M, RA, S, RM);
  __syncthreads();

  if (!consumer) {
    ring_produce(M, RA, RM, nmine, warp - RA.warps, lane);   // 2a. producers
    return;
  }

  // 2b. consumers: the tables
  table.finish(M.tab32, tab, tab1, warp, lane, RA.warps);
  asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
  const uint32_t lane_off = (lane & (R - 1)) << 2;
  WarpTileStage stage;
  stage.init(stage0 + (TILE_OUT ? warp * WarpTileStage::kBytes : 0), lane);
#pragma unroll 1
  for (;;) {
    Unit u;
    const int got = ring_draw(RA, RM, nmine, lane, u);
    if (got == 0) break;
    if (got < 0) {
      if (TILE_OUT) stage.drain(lane);
      return;
    }
    const uint32_t tc = u.j, seg = u.seg, tr = u.tr, cls = u.cls, lines = u.lines, second = u.second;
    const uint32_t* buf = u.buf;
    UnitSide<FMT> side_a, side_b;
    side_a.load(buf + lines * 32u - SIDEW, lane);
    side_b.load(buf + lines * 32u - SIDEW, lane + 32);
    typename ChainOf<PAIR_LAYOUT, IDXBITS>::type ca, cb;
    ca.init(buf + lane, kRingLogCopies - LOG_R);
    cb.init(buf + second * 32u + lane, kRingLogCopies - LOG_R);
    __half* oa = A.out + (static_cast<size_t>(tr - RA.tr0) * kTileRows + lane) * M.K + static_cast<size_t>(tc) * TW +
                 seg * (TW / SPLIT);
    __half* ob = oa + static_cast<size_t>(32) * M.K;
    // symbols per 32-byte store: eight paired symbols (two weights each) or sixteen single ones
    constexpr int PER = PAIR ? 8 : 16;
    // sixteen weights of each of the unit's rows, from column `col` of the unit
    auto out16 = [&](int col, const HalfPack& pa, const HalfPack& pb) {
      if constexpr (TILE_OUT) {
        stage.reuse(lane);
        stage.put(0, pa.w);
        stage.put(1, pb.w);
        stage.send(&TM, (static_cast<int>(tc) * TW + static_cast<int>(seg) * (TW / SPLIT) + col) * 2, static_cast<int>(tr - RA.tr0) * kTileRows, lane);
      } else {
        pa.flush(oa + col);
        pb.flush(ob + col);
      }
    };
    // weights of one decoded symbol pair (chains a and b) into the two packs
    // s * f(q) - o, each operation rounded; formats without offsets have o = 0 and x - 0 = x exactly, so they skip it
    constexpr bool HAS_OFFSET = FMT == kFmtQ4K || FMT == kFmtQ5K || FMT == kFmtQ5KP;
    auto weight = [&](float s, float o, uint32_t e, int which) {
      const float p = __fmul_rn(s, grid_of_entry(e, which));
      return HAS_OFFSET ? __fsub_rn(p, o) : p;
    };
    auto emit = [&](int c, uint32_t ea, uint32_t eb, float s_a, float o_a, float s_b, float o_b, HalfPack& pa, HalfPack& pb) {
      if (PAIR) {
        pa.put(c, weight(s_a, o_a, ea, 0), weight(s_a, o_a, ea, 1));
        pb.put(c, weight(s_b, o_b, eb, 0), weight(s_b, o_b, eb, 1));
      } else {   // two consecutive symbols make one half2: the even one waits (as float bits) for the odd one
        const float wa = weight(s_a, o_a, ea, 0);
        const float wb = weight(s_b, o_b, eb, 0);
        if (c % 2 == 0) {
          pa.w[c / 2] = __float_as_uint(wa);
          pb.w[c / 2] = __float_as_uint(wb);
        } else {
          pa.put(c / 2, __uint_as_float(pa.w[c / 2]), wa);
          pb.put(c / 2, __uint_as_float(pb.w[c / 2]), wb);
        }
      }
    };
    if (PAIR_LAYOUT || cls == 0) {   // a pair layout has no other class
      // the common class: groups of G symbols per refill check, everything unrolled (the phase of the groups is static)
#pragma unroll
      for (int jj = 0; jj < NSU; ++jj) {
        float s_a, o_a, s_b, o_b;
        side_a.sub(jj, s_a, o_a);
        side_b.sub(jj, s_b, o_b);
#pragma unroll
        for (int c0 = 0; c0 < SPG; c0 += PER) {
          HalfPack pa, pb;
#pragma unroll
          for (int c = 0; c < PER; ++c) {
            const int f = jj * SPG + c0 + c;
            if (f % G == 0) {
              ca.begin();
              cb.begin();
            }
            const uint32_t ea = ca.template sym<MASK>(smem, lane_off), eb = cb.template sym<MASK>(smem, lane_off);
            if (f % G == G - 1 || f == NSU * SPG - 1) {
              ca.end();
              cb.end();
            }
            emit(c, ea, eb, s_a, o_a, s_b, o_b, pa, pb);
          }
          out16(jj * GW + (PAIR ? 2 * c0 : c0), pa, pb);
        }
      }
    } else if constexpr (!PAIR_LAYOUT) {
      // the fallback classes, rolled up: window normalised per symbol (exact for any data), or the single-copy table
#pragma unroll 1
      for (int jj = 0; jj < 4; ++jj) {
        float s_a, o_a, s_b, o_b;
        side_a.sub(jj, s_a, o_a);
        side_b.sub(jj, s_b, o_b);
#pragma unroll 1
        for (int c0 = 0; c0 < SPG; c0 += PER) {
          HalfPack pa, pb;
#pragma unroll
          for (int c = 0; c < PER; ++c) {
            uint32_t ea, eb;
            if (cls == 2) {
              ea = ca.slow_sym(tab1, LOG_R + 2);
              eb = cb.slow_sym(tab1, LOG_R + 2);
            } else {
              ca.begin();
              cb.begin();
              ea = ca.template sym<MASK>(smem, lane_off);
              eb = cb.template sym<MASK>(smem, lane_off);
              ca.end();
              cb.end();
            }
            emit(c, ea, eb, s_a, o_a, s_b, o_b, pa, pb);
          }
          out16(jj * GW + (PAIR ? 2 * c0 : c0), pa, pb);
        }
      }
    }
    ring_release(RM, u, lane);
  }
  if (TILE_OUT) stage.drain(lane);
}

}  // namespace lw
