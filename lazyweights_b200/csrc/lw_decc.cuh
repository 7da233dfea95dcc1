// Decode to codes with the batch-1 kernel's decoder (lw_ring.cuh: replicated 32-bit table, grouped refills chosen from
// the data, producer warps feeding a ring of staging buffers): the role of k_decode_hufi, kernels/llmrt.cu:767-806.
// The table here maps a window to the SYMBOL itself (length << 28 | symbol; lw::MatDev::symtab32), not to grid values;
// a pair layout's table already holds two codes per entry.  A lane produces the bytes of its two rows 32 at a time: 32
// symbols, or 16 paired symbols expanded to one 4-bit code per byte (low nibble first, kernels/llmrt.cu:798-800), or 16
// pair symbols of two codes.  They leave through the warp's staging area and a 2-D tensor copy (WarpTileStage,
// lw_ring.cuh) or, without it, as one 32-byte store per lane and row.  Included by lw_decc.cu.
#pragma once
#include "lw_ring.cuh"

namespace lw {

struct DeccArgs {
  RingArgs r;
  uint8_t* out;      // [N][row_bytes]
  int row_bytes;     // Ks, or 2 Ks when paired symbols are expanded
};

struct BytePack {
  uint32_t w[8];
  __device__ __forceinline__ void flush(uint8_t* dst) const {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
  }
};

// TILE_OUT: the bytes leave through shared memory and the tensor-copy engine (WarpTileStage; TM = the output's tensor map)
// instead of 32-byte stores
template <int FMT, int G, int IDXBITS, int LOG_R, bool EXPAND, bool TILE_OUT>
__global__ void __launch_bounds__(1024, 1) k_decode_codes_ring(const __grid_constant__ MatDev M, const __grid_constant__ DeccArgs A,
                                                               const __grid_constant__ CUtensorMap TM) {
  const RingArgs& RA = A.r;
  constexpr int SPLIT = default_split(FMT);
  constexpr int USYM = kTileSyms / SPLIT;                          // symbols per chain
  constexpr int PER = EXPAND ? 16 : 32;                            // symbols per 32-byte store
  constexpr int OUT_PER_SYM = EXPAND ? 2 : 1;
  static_assert(!EXPAND || is_paired(FMT), "only paired symbols expand");
  // a pair layout (two codes of an unpaired format per symbol) is always written one code per byte; its table holds
  // grid values, from which the codes follow: Q6_K stores code - 32 (so code = low six bits with bit 5 flipped),
  // Q5_K the code itself
  constexpr bool PAIR_LAYOUT = is_pair_layout(FMT);
  static_assert(!PAIR_LAYOUT || EXPAND, "a pair layout is written expanded");
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
  const uint32_t* src = PAIR_LAYOUT ? M.tab32 : M.symtab32;
  TableLoad<IDXBITS, LOG_R, SINGLE> table;
  table.issue(src, warp, lane, RA.warps);
  BlockShare S;
  S.init(M, RA, SPLIT, blockIdx.x, gridDim.x);
  const int nmine = S.nmine;
  ring_reset(RM);
  __syncthreads();
  ring_build_list<SPLIT>(M, RA, S, RM);
  __syncthreads();
  if (warp >= RA.warps) {
    ring_produce(M, RA, RM, nmine, warp - RA.warps, lane);
    return;
  }
  // the symbol table, replicated like the value table of the other kernels
  table.finish(src, tab, tab1, warp, lane, RA.warps);
  asm volatile("bar.sync 1, %0;" ::"r"(RA.warps * 32) : "memory");
  const uint32_t lane_off = (lane & (R - 1)) << 2;
  // Symbol c of the current 32 bytes.  Bytes are placed with byte permutes (one instruction per symbol, c is a constant
  // after unrolling); the first symbol of a word just sets it, its upper bytes are replaced by the symbols that follow.
  // Table entries are length << 28 | payload with zero bits between, so byte 1 of a symbol entry is zero.
  auto put = [&](BytePack& p, int c, uint32_t e) {
    if constexpr (PAIR_LAYOUT) {          // two code bytes per entry
      uint32_t& w = p.w[c / 2];
      if (c % 2 == 0) {
        w = e;
      } else {
        w = __byte_perm(w, e, 0x5410);
        if (FMT == kFmtQ6KP) w = (w & 0x3F3F3F3Fu) ^ 0x20202020u;   // the table holds code - 32
      }
    } else if constexpr (EXPAND) {        // a pair symbol to two 4-bit codes, low nibble first
      uint32_t& w = p.w[c / 2];
      if (c % 2 == 0) {
        w = e;
      } else {
        w = __byte_perm(w, e, 0x5410);    // [s0, 0, s1, 0]
        w = (w | (w << 4)) & 0x0F0F0F0Fu;
      }
    } else {
      uint32_t& w = p.w[c / 4];
      w = c % 4 == 0 ? e : __byte_perm(w, e, c % 4 == 1 ? 0x3240 : c % 4 == 2 ? 0x3410 : 0x4210);
    }
  };
  WarpTileStage stage;
  stage.init(stage0 + (TILE_OUT ? warp * WarpTileStage::kBytes : 0), lane);
  // 32 bytes of each of the unit's rows: piece `it` of the unit; oa / ob: the unit's first byte in rows lane, lane + 32
  auto out32 = [&](const Unit& u, int it, const BytePack& pa, const BytePack& pb, uint8_t* oa, uint8_t* ob) {
    if constexpr (TILE_OUT) {
      stage.reuse(lane);
      stage.put(0, pa.w);
      stage.put(1, pb.w);
      stage.send(&TM, (u.j * kTileSyms + u.seg * USYM) * OUT_PER_SYM + it * 32, u.tr * kTileRows, lane);
    } else {
      pa.flush(oa + it * 32);
      pb.flush(ob + it * 32);
    }
  };
#pragma unroll 1
  for (;;) {
    Unit u;
    const int got = ring_draw(RA, RM, nmine, lane, u);
    if (got == 0) break;
    if (got < 0) {
      if (TILE_OUT) stage.drain(lane);
      return;
    }
    typename ChainOf<PAIR_LAYOUT, IDXBITS>::type ca, cb;
    ca.init(u.buf + lane, kRingLogCopies - LOG_R);
    cb.init(u.buf + u.second * 32u + lane, kRingLogCopies - LOG_R);
    uint8_t* oa = A.out + (static_cast<size_t>(u.tr) * kTileRows + lane) * A.row_bytes +
                  (static_cast<size_t>(u.j) * kTileSyms + u.seg * USYM) * OUT_PER_SYM;
    uint8_t* ob = oa + static_cast<size_t>(32) * A.row_bytes;
    if (PAIR_LAYOUT || u.cls == 0) {   // a pair layout has no other class
#pragma unroll
      for (int c0 = 0; c0 < USYM; c0 += PER) {
        BytePack pa, pb;
#pragma unroll
        for (int c = 0; c < PER; ++c) {
          const int f = c0 + c;
          if (f % G == 0) {
            ca.begin();
            cb.begin();
          }
          const uint32_t ea = ca.template sym<MASK>(smem, lane_off), eb = cb.template sym<MASK>(smem, lane_off);
          if (f % G == G - 1 || f == USYM - 1) {
            ca.end();
            cb.end();
          }
          put(pa, c, ea);
          put(pb, c, eb);
        }
        out32(u, c0 / PER, pa, pb, oa, ob);
      }
    } else if constexpr (!PAIR_LAYOUT) {
#pragma unroll 1
      for (int c0 = 0; c0 < USYM; c0 += PER) {
        BytePack pa, pb;
#pragma unroll
        for (int c = 0; c < PER; ++c) {
          uint32_t ea, eb;
          if (u.cls == 2) {
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
          put(pa, c, ea);
          put(pb, c, eb);
        }
        out32(u, c0 / PER, pa, pb, oa, ob);
      }
    }
    ring_release(RM, u, lane);
  }
  if (TILE_OUT) stage.drain(lane);
}

}  // namespace lw
