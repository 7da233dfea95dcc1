// Decode + block dequantisation to fp16 weights with the batch-1 kernel's decoder (lw_gemv1.cuh): replicated 32-bit
// table, grouped refills chosen from the data, unit scales staged with the chains, producer warps feeding a ring of
// staging buffers, units drawn from a shared counter.  Instead of dot products every decoded grid value becomes
// w = s * f(q) - o in float32 (product and difference rounded separately, llama.cpp's block formulas; reference:
// scripts/a2_kq_bundle.py:50-68) and one __float2half_rn; a lane writes the weights of its two rows 32 bytes at a time.
// Included by lw_decw.cu.
#pragma once
#include "lw_gemv1.cuh"

namespace lw {

struct DecwArgs {
  Gemv1Args g;      // x, y, partials unused
  __half* out;      // [(tr1 - tr0) * 64][K]
  int tr0, tr1;     // tile rows to decode
};

// Collects sixteen weights of one chain and stores them as one 32-byte piece (a whole sector: a lane writes to its
// own row, so every store instruction touches 32 different lines, and 16-byte pieces paid for a full sector each).
struct HalfPack {
  uint32_t w[8];
  __device__ __forceinline__ void put(int i, float lo, float hi) {   // halfs 2 i, 2 i + 1 of the current sixteen
    const __half2 h = __halves2half2(__float2half_rn(lo), __float2half_rn(hi));
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

template <int FMT, int G, int IDXBITS, int LOG_R>
__global__ void __launch_bounds__(1024, 1) k_decw(MatDev M, DecwArgs DA) {
  const Gemv1Args& A = DA.g;
  constexpr bool PAIR = is_paired(FMT);
  constexpr int SPLIT = default_split(FMT);
  constexpr int TW = PAIR ? 2 * kTileSyms : kTileSyms;
  constexpr int GW = sub_width(FMT), SPG = sub_syms(FMT), SIDEW = unit_side_words(FMT);
  constexpr int NIDX = 1 << IDXBITS, R = 1 << LOG_R;
  constexpr uint32_t MASK = static_cast<uint32_t>(NIDX - 1) << (LOG_R + 2);
  constexpr int kReplicatedTableBytes = NIDX * R * 4;
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t* tab = reinterpret_cast<uint32_t*>(smem);
  uint32_t* tab1 = reinterpret_cast<uint32_t*>(smem + kReplicatedTableBytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(tab1 + kLutSize);
  uint64_t* empty = full + kGemv1MaxSlots;
  uint32_t* released = reinterpret_cast<uint32_t*>(empty + kGemv1MaxSlots);
  int* next_unit = reinterpret_cast<int*>(released + kGemv1MaxSlots);
  int* list_count = next_unit + 1;
  UnitMeta* meta = reinterpret_cast<UnitMeta*>(next_unit + 4);
  uint32_t* bufs = reinterpret_cast<uint32_t*>(meta + A.max_units);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int set = 0, bi = blockIdx.x, nb_set = gridDim.x, ncol = M.KT;   // one column set: no activations to stage
  const int ntiles = (DA.tr1 - DA.tr0) * ncol;
  const int tmine = bi < ntiles ? (ntiles - bi + nb_set - 1) / nb_set : 0;
  const int nmine = tmine * SPLIT;
  const bool consumer = warp < A.warps;
  const int nthr = A.warps * 32;

  // 1. the block's list (whole tiles, symbol-by-symbol tiles first), exactly as in the batch-1 kernel
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
      const int v = bi + (k / SPLIT) * nb_set;
      j = v % ncol;
      tr = DA.tr0 + v / ncol;
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
    tpos = __shfl_sync(0xffffffffu, tpos, lane - seg);
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
    // 2a. producers: issuer s owns buffers s, s + S, ... and feeds them round by round
    if (lane < A.producer_lanes) {
      const int issuers = A.producers * A.producer_lanes;
      for (int round = 0; round * A.slots < nmine; ++round)
        for (int slot = (warp - A.warps) * A.producer_lanes + lane; slot < A.slots; slot += issuers) {
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

  // 2b. consumers: tables, then the activations of the block's tile columns for all rows
  {
    constexpr int PER = 32 / R;
    for (int i0 = warp * 32; i0 < NIDX; i0 += A.warps * 32) {
      const uint32_t mine = __ldg(M.tab32 + i0 + lane);
#pragma unroll 8
      for (int j = 0; j < 32; j += PER) {
        const uint32_t v = __shfl_sync(0xffffffffu, mine, j + (lane >> LOG_R));
        tab[(i0 + j) * R + lane] = v;
      }
      tab1[i0 + lane] = mine;
    }
    for (int idx = NIDX + static_cast<int>(threadIdx.x); idx < kLutSize; idx += nthr) tab1[idx] = __ldg(M.tab32 + idx);
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nthr) : "memory");
  const uint32_t lane_off = (lane & (R - 1)) << 2;
#pragma unroll 1
  for (;;) {
    int k = 0;
    if (lane == 0) k = atomicAdd(next_unit, 1);
    k = __shfl_sync(0xffffffffu, k, 0);
    if (k >= nmine) break;
    const uint4 raw = *reinterpret_cast<const uint4*>(meta + k);
    const uint32_t lines = raw.y & 0xFFFFu, second = raw.y >> 16, tr = raw.z & 0xFFFFu, round = raw.z >> 16;
    const uint32_t tc = raw.w & 255u, seg = (raw.w >> 8) & 255u, slot = (raw.w >> 16) & 255u;
    const uint32_t cls = second >> 14;
    const uint32_t* buf = bufs + static_cast<size_t>(slot) * A.buf_words;
    if (round > 0 && !wait_released(released + slot, round, A.err)) return;
    if (!mbar_wait(smem_addr(full + slot), round & 1, A.err)) return;
    UnitSide<FMT> side_a, side_b;
    side_a.load(buf + lines * 32u - SIDEW, lane);
    side_b.load(buf + lines * 32u - SIDEW, lane + 32);
    GroupChain ca, cb;
    ca.init(buf + lane);
    cb.init(buf + (second & 0x3FFFu) * 32u + lane);
    __half* oa = DA.out + (static_cast<size_t>(tr - DA.tr0) * kTileRows + lane) * M.K + static_cast<size_t>(tc) * TW +
                 seg * (TW / SPLIT);
    __half* ob = oa + static_cast<size_t>(32) * M.K;
    // symbols per 32-byte store: eight paired symbols (two weights each) or sixteen single ones
    constexpr int PER = PAIR ? 8 : 16;
    // weights of one decoded symbol pair (chains a and b) into the two packs
    auto emit = [&](int c, uint32_t ea, uint32_t eb, float s_a, float o_a, float s_b, float o_b, HalfPack& pa, HalfPack& pb) {
      if (PAIR) {
        pa.put(c, __fsub_rn(__fmul_rn(s_a, grid_of_entry(ea, 0)), o_a), __fsub_rn(__fmul_rn(s_a, grid_of_entry(ea, 1)), o_a));
        pb.put(c, __fsub_rn(__fmul_rn(s_b, grid_of_entry(eb, 0)), o_b), __fsub_rn(__fmul_rn(s_b, grid_of_entry(eb, 1)), o_b));
      } else {   // two consecutive symbols make one half2: the even one waits (as float bits) for the odd one
        const float wa = __fsub_rn(__fmul_rn(s_a, grid_of_entry(ea, 0)), o_a);
        const float wb = __fsub_rn(__fmul_rn(s_b, grid_of_entry(eb, 0)), o_b);
        if (c % 2 == 0) {
          pa.w[c / 2] = __float_as_uint(wa);
          pb.w[c / 2] = __float_as_uint(wb);
        } else {
          pa.put(c / 2, __uint_as_float(pa.w[c / 2]), wa);
          pb.put(c / 2, __uint_as_float(pb.w[c / 2]), wb);
        }
      }
    };
    if (cls == 0) {
      // the common class: groups of G symbols per refill check, everything unrolled (the phase of the groups is static)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
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
            if (f % G == G - 1 || f == 4 * SPG - 1) {
              ca.end();
              cb.end();
            }
            emit(c, ea, eb, s_a, o_a, s_b, o_b, pa, pb);
          }
          const int col = jj * GW + (PAIR ? 2 * c0 : c0);
          pa.flush(oa + col);
          pb.flush(ob + col);
        }
      }
    } else {
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
              ea = ca.slow_sym(tab1, static_cast<uint32_t>(M.pad));
              eb = cb.slow_sym(tab1, static_cast<uint32_t>(M.pad));
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
          const int col = jj * GW + (PAIR ? 2 * c0 : c0);
          pa.flush(oa + col);
          pb.flush(ob + col);
        }
      }
    }
    __syncwarp();
    if (lane == 0) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(empty + slot)) : "memory");
      asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_addr(released + slot)), "r"(round + 1u) : "memory");
    }
  }
}

}  // namespace lw
