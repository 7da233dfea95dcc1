// Decode + dequantise + small-M GEMM on the fifth-generation tensor cores (tcgen05), for 9..64 activation rows:
// the role of the reference's decode + k_gemm_raw8 / k_gemm2_raw8 path (kernels/llmrt.cu:211-343, :1827-1841), without
// the decoded weights ever leaving the SM.  Included by lw_gemm_t5.cu.
//
//   D[weight row, token] = sum_k W[weight row, k] X[token, k]     tcgen05.mma, kind::f16, M = 128, N = tokens, K = 16
//
//  * W is the A operand and lives in TENSOR MEMORY: a decoding lane owns a weight row, so after sixteen decoded weights
//    it holds exactly one row of a 128 x 16 A tile in eight registers and writes it with one tcgen05.st (no shared-memory
//    operand tile, no layout shuffle).  A warp can only reach the 32 tensor-memory lanes of its quadrant (warp % 4),
//    so four consumer warps form a TEAM that decodes the same column segment of four consecutive tile rows: warp q
//    fills lanes 32 q .. 32 q + 31.  A lane decodes two rows (l and l + 32 of its tile), hence two A tiles per step:
//    tile "a" = rows l of the four tile rows, tile "b" = rows l + 32; they accumulate into two D tiles.
//  * X is the B operand, converted once per block to fp16 in shared memory in the canonical K-major layout without
//    swizzle (8 x 16-byte core matrices; 128 bytes between K-adjacent core matrices, 8192 between 8-token groups) for
//    the block's 512 weight columns.
//  * D (fp32) lives in tensor memory, double-buffered: while the teams decode the next four tile rows, the previous
//    D is read back with tcgen05.ld and written as one plane of partial products P[column set][token][N]; the planes are
//    added by k_sum_partials (ordered, no atomics).
//  * One warp issues every MMA (one elected lane): it waits for a team's A slot (mbarrier, four arrivals), issues the two
//    MMAs and commits them to the slot's "empty" barrier, so slots are reused as soon as the tensor core has read them.
//  * The coded chains come through the staging ring of lw_ring.cuh (bulk copies by producer warps); the decoder is the
//    batch-1 kernel's (replicated 32-bit table, grouped refills, unit classes), the dequantisation the decode-to-weights
//    kernel's: w = s f(q) - o in float32, product and difference rounded separately, one rounding to fp16.
//  * Every wait is bounded; a warp that gives up sets the device error word and a block-wide flag that makes every other
//    loop of the block end, so that the block always reaches the point where its tensor memory is released.
#pragma once
#include <type_traits>

#include "lw_ring.cuh"

namespace lw {

constexpr int kT5Teams = 4;                 // teams of four consumer warps
constexpr int kT5Consumers = 4 * kT5Teams;  // consumer warps 0 .. 15
constexpr int kT5Producers = 2;             // warps 16, 17 issue the bulk copies
constexpr int kT5Threads = (kT5Consumers + kT5Producers + 1) * 32;   // + the MMA warp (18)
constexpr int kT5ASlots = 4;                // A slots per team (16 tensor-memory columns each: tile a, tile b)
constexpr int kT5SetK = 512;                // weight columns per block (column set)
constexpr int kT5MaxTokens = 64;
constexpr uint32_t kT5TmemCols = 512;

struct GemmT5Args {
  RingArgs r;          // r.nsets = K / 512 column sets; r.tr0 / r.ntr unused (all tile rows)
  const void* x;       // activations [m][K], fp16 or fp32
  float* planes;       // P[K / 512][m][N]
  const float* row_scale;   // fp32 x only (else null): factor per row that keeps it inside fp16's range
  int x_is_half;
  int m;               // tokens (rows of x), 1 .. ntok
  int ntok;            // N of the MMA: m rounded up to a multiple of 16
};

// ------------------------------------------------------------------------------------------------ tcgen05 wrappers

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_dst)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 16 registers of this thread -> its tensor-memory lane, 16 consecutive columns from taddr
__device__ __forceinline__ void tmem_store16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
      "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_store() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_load8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_load() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[128 x N] (+)= A[128 x 16] (tensor memory) . B[N x 16]^T (shared memory descriptor), fp16 inputs, fp32 accumulate
__device__ __forceinline__ void mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
// the barrier is arrived on once every MMA this thread has issued so far has completed
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// Shared-memory matrix descriptor of a K-major operand without swizzle: core matrices of 8 rows x 16 bytes,
// `lbo` bytes between core matrices adjacent in K, `sbo` bytes between 8-row groups (all multiples of 16).
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((saddr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);   // bit 46: descriptor version of this architecture
}
// Instruction descriptor: fp32 accumulator, fp16 A and B, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t idesc_f16_m128(int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __halves2half2(__float2half_rn(lo), __float2half_rn(hi));
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float entry_value(uint32_t e, int which) {
  return static_cast<float>(static_cast<int>(static_cast<int8_t>((e >> (8 * which)) & 255u)));
}

// bounded waits that also end when another warp of the block has given up
__device__ __forceinline__ bool t5_wait(uint64_t* bar, uint32_t parity, const RingArgs& A, volatile int* abort_flag) {
  const uint32_t addr = smem_addr(bar);
  for (uint32_t i = 0; i < A.wait_limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  atomicOr(A.err, 1u);
  *abort_flag = 1;
  return false;
}
// the same for a whole warp: every lane gets the same answer, so that the warp stays converged for the .aligned
// tensor-memory instructions that follow
__device__ __forceinline__ bool t5_wait_warp(uint64_t* bar, uint32_t parity, const RingArgs& A, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, t5_wait(bar, parity, A, abort_flag));
}

// LOG_R: copies of the decode table in THIS kernel (8: half of what the chains' leading zero bits allow, because the
// activations need the shared memory; lw::kRingLogCopies - LOG_R = the extra shift of every lookup).
template <int FMT, int G, int IDXBITS, int LOG_R>
__global__ void __launch_bounds__(kT5Threads, 1) k_gemm_t5(const __grid_constant__ MatDev M, const __grid_constant__ GemmT5Args A) {
  const RingArgs& RA = A.r;
  constexpr bool PAIR = is_paired(FMT);
  constexpr int SPLIT = default_split(FMT);
  constexpr int TW = PAIR ? 2 * kTileSyms : kTileSyms;            // weights per tile row
  constexpr int GW = sub_width(FMT), SPG = sub_syms(FMT), SIDEW = unit_side_words(FMT);
  constexpr int COLS = kT5SetK / TW;                              // tile columns per column set
  constexpr int TU = COLS * SPLIT;                                // team-units per item (four tile rows x one column set)
  constexpr int KU = TW / SPLIT;                                  // weights a unit covers along K
  constexpr int STEPS = KU / 16;                                  // K = 16 steps per team-unit
  constexpr int SYM16 = PAIR ? 8 : 16;                            // symbols per step and chain
  static_assert(TU % kT5Teams == 0 && KU % 16 == 0 && GW % 16 == 0, "team-units are dealt evenly; steps stay inside a sub-block");
  constexpr int NIDX = 1 << IDXBITS, R = 1 << LOG_R;
  constexpr uint32_t MASK = static_cast<uint32_t>(NIDX - 1) << (LOG_R + 2);
  constexpr int kReplicatedTableBytes = NIDX * R * 4;
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t* tab = reinterpret_cast<uint32_t*>(smem);
  // the single-copy table serves the units that hold an 11-bit code under a 1024-window table; with 2048 windows
  // replicated there are no such units and no such table
  constexpr bool SINGLE = IDXBITS < kMaxLen;
  uint32_t* tab1 = reinterpret_cast<uint32_t*>(smem + kReplicatedTableBytes);       // [2048] single copy (if SINGLE)
  uint8_t* xs = reinterpret_cast<uint8_t*>(tab1 + (SINGLE ? kLutSize : 0));        // B operand: [ntok][512] fp16, canonical
  const int ntok = A.ntok;
  uint64_t* a_full = reinterpret_cast<uint64_t*>(xs + static_cast<size_t>(ntok) * kT5SetK * 2);   // [teams][slots]
  uint64_t* a_empty = a_full + kT5Teams * kT5ASlots;
  uint64_t* d_full = a_empty + kT5Teams * kT5ASlots;              // [2]
  uint64_t* d_empty = d_full + 2;                                 // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 2); // tensor-memory base address, abort flag
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  RingMem RM;
  RM.carve(tmem_slot + 4, RA);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TableLoad<IDXBITS, LOG_R, SINGLE> table;
  table.issue(M.tab32, warp, lane, kT5Consumers);
  const int NT = M.N / kTileRows, NRG = NT / 4;                   // row groups of four tile rows
  const int set = blockIdx.x % RA.nsets, bi = blockIdx.x / RA.nsets;
  const int nb_set = (gridDim.x - set + RA.nsets - 1) / RA.nsets;
  const int items = bi < NRG ? (NRG - bi + nb_set - 1) / nb_set : 0;   // row groups bi, bi + nb_set, ...
  const int nmine = items * TU * 4;                               // units of this block, in list order

  // ---- set-up: barriers, the unit list, tensor memory
  if (threadIdx.x == 0) {
    for (int i = 0; i < kT5Teams * kT5ASlots; ++i) {
      mbar_init(smem_addr(a_full + i), 4);
      mbar_init(smem_addr(a_empty + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_addr(d_full + i), 1);
      mbar_init(smem_addr(d_empty + i), kT5Consumers);
    }
    tmem_slot[1] = 0u;
  }
  // list entry k = ((item * TU + team-unit) * 4 + quadrant): tile row 4 rg + quadrant, tile column and segment of the
  // team-unit; staging buffer k % slots, round k / slots
  for (int k = threadIdx.x; k < nmine; k += blockDim.x) {
    const int q = k & 3, s = k >> 2, u = s % TU, it = s / TU;
    const int rg = bi + it * nb_set, tr = 4 * rg + q, tc = set * COLS + u / SPLIT, seg = u % SPLIT;
    const int t = tr * M.KT + tc;
    const uint32_t* gb = M.group_base + static_cast<size_t>(t) * (2 * SPLIT) + 2 * seg;
    const uint32_t g0 = __ldg(gb), g1 = __ldg(gb + 1), g2 = __ldg(gb + 2);
    const uint32_t cls = __ldg(M.unit_slow + static_cast<size_t>(t) * SPLIT + seg);
    RM.meta[k] = UnitMeta{g0,
                          static_cast<uint16_t>((g2 - g0) >> 5),
                          static_cast<uint16_t>(((g1 - g0) >> 5) | (cls << 14)),
                          static_cast<uint16_t>(tr),
                          static_cast<uint16_t>(k / RA.slots),
                          static_cast<uint8_t>(u),
                          static_cast<uint8_t>(seg),
                          static_cast<uint8_t>(k % RA.slots),
                          0};
  }
  if (threadIdx.x < RA.slots) {
    mbar_init(smem_addr(RM.full + threadIdx.x), 1);
    mbar_init(smem_addr(RM.empty + threadIdx.x), 1);
    RM.released[threadIdx.x] = 0u;
  }
  if (warp == kT5Consumers + kT5Producers) tmem_alloc(tmem_slot, kT5TmemCols);   // the MMA warp owns the allocation
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot[0];
  // tensor-memory columns: D buffers [2][a | b][ntok] from 0, A rings [team][slot][a 8 | b 8] from 256
  const uint32_t d_col0 = 0, a_col0 = 256;

  if (warp >= kT5Consumers && warp < kT5Consumers + kT5Producers) {
    ring_produce(M, RA, RM, nmine, warp - kT5Consumers, lane);        // ---- producers: the staging ring
  }

  // ---- X -> fp16 in the canonical K-major layout (all warps but the producers, which are already copying)
  if (warp < kT5Consumers || warp == kT5Consumers + kT5Producers) {
    const int nthr = (kT5Consumers + 1) * 32;
    const int tid = warp < kT5Consumers ? threadIdx.x : kT5Consumers * 32 + lane;
    // one thread converts eight consecutive K values of one token: one 16-byte row of a core matrix
    for (int i = tid; i < ntok * (kT5SetK / 8); i += nthr) {
      const int n = i / (kT5SetK / 8), kc = i % (kT5SetK / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (n < A.m) {
        const size_t src = static_cast<size_t>(n) * M.K + static_cast<size_t>(set) * kT5SetK + kc * 8;
        if (A.x_is_half) {
          v = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(A.x) + src));
        } else {
          const float4 f0 = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(A.x) + src));
          const float4 f1 = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(A.x) + src) + 1);
          const float rs = A.row_scale ? A.row_scale[n] : 1.f;   // not __ldg: written by the kernel just before
          v = make_uint4(pack_half2(f0.x * rs, f0.y * rs), pack_half2(f0.z * rs, f0.w * rs), pack_half2(f1.x * rs, f1.y * rs),
                         pack_half2(f1.z * rs, f1.w * rs));
        }
      }
      *reinterpret_cast<uint4*>(xs + (n >> 3) * (kT5SetK / 8 * 128) + kc * 128 + (n & 7) * 16) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads xs through the async proxy
  }
  if (warp < kT5Consumers) table.finish(M.tab32, tab, tab1, warp, lane, kT5Consumers);
  if (warp < kT5Consumers || warp == kT5Consumers + kT5Producers)
    asm volatile("bar.sync 1, %0;" ::"r"((kT5Consumers + 1) * 32) : "memory");

  if (warp == kT5Consumers + kT5Producers) {
    // ---- the MMA warp: one lane issues; the others wait at the end
    if (lane == 0) {
      const uint32_t idesc = idesc_f16_m128(ntok);
      const uint32_t xs_addr = smem_addr(xs);
      uint32_t a_count[kT5Teams] = {0u, 0u, 0u, 0u};
      bool ok = true;
      for (int it = 0; it < items && ok; ++it) {
        const int db = it & 1;
        if (it >= 2) ok = t5_wait(d_empty + db, ((it >> 1) - 1) & 1, RA, abort_flag);   // the epilogue of item it - 2 is done
        tc_fence_after();
        const uint32_t d_a = tmem + d_col0 + db * 2 * ntok, d_b = d_a + ntok;
        bool first = true;
        for (int rd = 0; rd < TU / kT5Teams && ok; ++rd)
          for (int j = 0; j < STEPS && ok; ++j)
            for (int t = 0; t < kT5Teams && ok; ++t) {
              const int u = rd * kT5Teams + t;                        // the team-unit this team is on
              const uint32_t n = a_count[t]++, sl = n % kT5ASlots, ph = (n / kT5ASlots) & 1u;
              ok = t5_wait(a_full + t * kT5ASlots + sl, ph, RA, abort_flag);
              if (!ok) break;
              tc_fence_after();
              const uint32_t koff = (u / SPLIT) * TW + (u % SPLIT) * KU + 16 * j;   // K offset inside the column set
              const uint64_t bdesc = smem_desc_kmajor(xs_addr + (koff >> 3) * 128, 128, kT5SetK / 8 * 128);
              const uint32_t a_a = tmem + a_col0 + (t * kT5ASlots + sl) * 16;
              mma_ts_f16(d_a, a_a, bdesc, idesc, !first);
              mma_ts_f16(d_b, a_a + 8, bdesc, idesc, !first);
              mma_commit(a_empty + t * kT5ASlots + sl);
              first = false;   // only the item's very first pair of MMAs overwrites D
            }
        if (ok) mma_commit(d_full + db);
      }
    }
    __syncwarp();
  } else if (warp < kT5Consumers) {
    // ---- consumers: team = warp / 4, quadrant = warp % 4
    const int team = warp >> 2, quad = warp & 3;
    const uint32_t lane_off = (lane & (R - 1)) << 2;
    const uint32_t my_lanes = static_cast<uint32_t>(32 * quad) << 16;
    uint32_t a_n = 0;       // A slots this team has used
    bool ok = true;
    // writes the plane of item `it` (tokens x 256 weight rows of its row group) from D buffer it % 2
    auto epilogue = [&](int it) {
      const int db = it & 1;
      if (!t5_wait_warp(d_full + db, (it >> 1) & 1, RA, abort_flag)) return false;
      tc_fence_after();
      const int rg = bi + it * nb_set;
      float* plane = A.planes + static_cast<size_t>(set) * A.m * M.N;
      // D buffer: columns [0, ntok) = tile a (rows l), [ntok, 2 ntok) = tile b (rows l + 32); team t reads a quarter
      const int per_team = 2 * ntok / kT5Teams;
      for (int c0 = team * per_team; c0 < (team + 1) * per_team; c0 += 8) {
        uint32_t v[8];
        tmem_load8(tmem + my_lanes + d_col0 + db * 2 * ntok + c0, v);
        tmem_wait_load();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = c0 + i, half = c >= ntok ? 1 : 0, tok = c - half * ntok;
          if (tok < A.m)
            plane[static_cast<size_t>(tok) * M.N + (4 * rg + quad) * kTileRows + half * 32 + lane] = __uint_as_float(v[i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_empty + db);
      return true;
    };
    for (int it = 0; it < items && ok; ++it) {
      for (int rd = 0; rd < TU / kT5Teams && ok; ++rd) {
        const int u = rd * kT5Teams + team;
        const int k = ((it * TU + u) << 2) + quad;
        const uint4 raw = *reinterpret_cast<const uint4*>(RM.meta + k);
        const uint32_t lines = raw.y & 0xFFFFu, second = (raw.y >> 16) & 0x3FFFu, cls = raw.y >> 30, round = raw.z >> 16;
        const uint32_t slot = (raw.w >> 16) & 255u;
        const uint32_t* buf = RM.bufs + static_cast<size_t>(slot) * RA.buf_words;
        bool here = round == 0 || wait_released(RM.released + slot, round, RA.err, RA.wait_limit);
        here = here && mbar_wait(smem_addr(RM.full + slot), round & 1, RA.err, RA.wait_limit);
        if (!__all_sync(0xffffffffu, here)) {
          *abort_flag = 1;
          ok = false;
          break;
        }
        UnitSide<FMT> side_a, side_b;
        side_a.load(buf + lines * 32u - SIDEW, lane);
        side_b.load(buf + lines * 32u - SIDEW, lane + 32);
        typename ChainOf<is_pair_layout(FMT), IDXBITS>::type ca, cb;
        ca.init(buf + lane, kRingLogCopies - LOG_R);
        cb.init(buf + second * 32u + lane, kRingLogCopies - LOG_R);
        // One unit: STEPS times sixteen weights of rows l (chain a) and l + 32 (chain b) -> one A slot each.  CLS = the
        // unit's class: 0 groups of G symbols per refill check (fully unrolled, the phase of the groups is static),
        // 1 the window normalised per symbol (exact for any data), 2 symbol by symbol through the single-copy table.
        auto run_unit = [&](auto cls_tag) {
          constexpr int CLS = decltype(cls_tag)::value;
#pragma unroll(CLS == 0 ? STEPS : 1)
          for (int j = 0; j < STEPS; ++j) {
            const int jj = 16 * j / GW;                                   // the sub-block (scale) of this step
            float s_a, o_a, s_b, o_b;
            side_a.sub(jj, s_a, o_a);
            side_b.sub(jj, s_b, o_b);
            uint32_t w[16];                                               // [0..8) tile a, [8..16) tile b, half2 each
#pragma unroll
            for (int c = 0; c < SYM16; ++c) {
              const int f = j * SYM16 + c;                                // symbol index within the chain
              uint32_t ea, eb;
              if constexpr (CLS == 0) {
                if (f % G == 0) {
                  ca.begin();
                  cb.begin();
                }
                ea = ca.template sym<MASK>(smem, lane_off);
                eb = cb.template sym<MASK>(smem, lane_off);
                if (f % G == G - 1 || f == STEPS * SYM16 - 1) {
                  ca.end();
                  cb.end();
                }
              } else if constexpr (CLS == 1) {
                ca.begin();
                cb.begin();
                ea = ca.template sym<MASK>(smem, lane_off);
                eb = cb.template sym<MASK>(smem, lane_off);
                ca.end();
                cb.end();
              } else {
                ea = ca.slow_sym(tab1, LOG_R + 2);
                eb = cb.slow_sym(tab1, LOG_R + 2);
              }
              if (PAIR) {
                w[c] = pack_half2(__fsub_rn(__fmul_rn(s_a, entry_value(ea, 0)), o_a), __fsub_rn(__fmul_rn(s_a, entry_value(ea, 1)), o_a));
                w[8 + c] = pack_half2(__fsub_rn(__fmul_rn(s_b, entry_value(eb, 0)), o_b), __fsub_rn(__fmul_rn(s_b, entry_value(eb, 1)), o_b));
              } else {
                const float wa = __fsub_rn(__fmul_rn(s_a, entry_value(ea, 0)), o_a);
                const float wb = __fsub_rn(__fmul_rn(s_b, entry_value(eb, 0)), o_b);
                if (c % 2 == 0) {
                  w[c / 2] = __float_as_uint(wa);
                  w[8 + c / 2] = __float_as_uint(wb);
                } else {
                  w[c / 2] = pack_half2(__uint_as_float(w[c / 2]), wa);
                  w[8 + c / 2] = pack_half2(__uint_as_float(w[8 + c / 2]), wb);
                }
              }
            }
            // the team's next A slot, once the tensor core has read its previous contents
            const uint32_t sl = a_n % kT5ASlots, use = a_n / kT5ASlots;
            ++a_n;
            if (use > 0 && !t5_wait_warp(a_empty + team * kT5ASlots + sl, (use - 1) & 1u, RA, abort_flag)) return false;
            tc_fence_after();
            tmem_store16(tmem + my_lanes + a_col0 + (team * kT5ASlots + sl) * 16, w);
            tmem_wait_store();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_full + team * kT5ASlots + sl);
          }
          return true;
        };
        if (is_pair_layout(FMT) || cls == 0) ok = run_unit(std::integral_constant<int, 0>{});   // a pair layout has no other class
        else if (cls == 1 || !SINGLE) ok = run_unit(std::integral_constant<int, 1>{});
        else ok = run_unit(std::integral_constant<int, 2>{});
        if (!ok) break;
        // every lane has read its last word: hand the staging buffer back
        __syncwarp();
        if (lane == 0) {
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(RM.empty + slot)) : "memory");
          asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_addr(RM.released + slot)), "r"(round + 1u) : "memory");
        }
        if (rd == 0 && it > 0) ok = epilogue(it - 1);   // the previous item's D, while the tensor core works on this one
      }
    }
    if (ok && items > 0) epilogue(items - 1);
  }
  // ---- everyone meets here (also after a wait gave up), then the tensor memory is released
  tc_fence_before();
  __syncthreads();
  if (warp == kT5Consumers + kT5Producers) {
    tc_fence_after();
    tmem_dealloc(tmem, kT5TmemCols);
  }
}

}  // namespace lw
