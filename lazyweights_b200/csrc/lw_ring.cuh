// The producer / consumer machinery shared by the persistent decode kernels (batch-1 product lw_gemv1.cuh, 2..8-row
// product lw_gemvm.cuh, decode to weights lw_decw.cuh, decode to codes lw_decc.cuh, many-row tensor-core product
// lw_gemm_tc5.cuh): the block's list of work units, the ring of staging buffers that producer lanes fill with bulk
// copies, the replicated decode table and the grouped chain reader.  One copy of this code, so that an ordering rule
// learnt once (wait_released below) holds everywhere.
//
// Block = consumer warps + producer warps.  Unit k of the block's list goes through staging buffer k % slots
// ("round" k / slots of that buffer).  Producer lanes each own a subset of the buffers and, round after round, wait
// until a buffer is free and start the bulk copy of its next unit; a consumer warp draws the next unit of the list from
// a shared counter, waits for the buffer to fill, decodes, and frees it.  With more buffers than consumers the copies
// run ahead of the decoding, so no warp waits for DRAM in steady state.  Everything a unit needs (coordinates, buffer,
// round) is worked out once, in parallel, when the block starts: the per-unit path has no integer division.
//
// A parity wait on an mbarrier is only exact for a waiter that is at most one phase away, and here the waiters of
// consecutive rounds of a buffer are different threads.  So every buffer also has a plain counter of the rounds that
// were released: both sides first wait until it reaches their round (exact at any distance), after which the barrier
// is known to be in the phase the parity wait assumes.  Every wait is bounded: a warp that gives up sets the device
// error word and leaves.
#pragma once
#include <cuda.h>
#include "lw_device.cuh"

namespace lw {

constexpr int kRingLogCopies = 4;        // the layout's pad allows up to 16 copies of the decode table
// Copies a kernel keeps: 16 of a 1024-window table, 8 of a 2048-window table, 4 of a 4096-window table (pair layouts)
// - 64 KB either way.  (Measured on the pair layout of Q6_K, 14336 x 4096: 8 copies of its 4096-window table = 128 KB
// leave 10 consumer warps, 23.3 instead of 20.1 us per product; so do units of half the size with either table.)  With 16 copies of the
// large table (128 KB) too few staging buffers fit beside it, and a block is left with 10 consumer warps instead of 28:
// measured on a paired 4-bit matrix, the decode loop then waits on its own dependency chain (2.5 warps per scheduler).
#ifndef LW_LOG_COPIES_11
#define LW_LOG_COPIES_11 3
#endif
__host__ __device__ constexpr int ring_log_copies(int index_bits) {
  return index_bits == 12 ? 2 : index_bits == 11 ? LW_LOG_COPIES_11 : kRingLogCopies;   // 64 KB in every case
}
constexpr int kRingMaxWarps = 28;        // consumer warps; up to four more warps produce
constexpr int kRingMaxSlots = 64;        // staging buffers in the ring
constexpr int kRingMaxUnits = 1024;      // work units one block can be dealt in one launch

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

// What every kernel of the family is told about its block shape and staging ring.
struct RingArgs {
  unsigned int* err;      // device error word (bit 0: a bounded wait gave up)
  uint32_t wait_limit;    // polls after which a wait gives up
  int warps;              // consumer warps per block
  int producers;          // producer warps per block
  int producer_lanes;     // lanes of a producer warp that issue copies
  int slots;              // staging buffers in the ring (>= warps)
  uint32_t buf_words;     // one staging buffer, in words
  int nsets;              // tile columns are dealt to `nsets` sets of blocks (bounds the staged activations)
  int cols_per_set;       // ceil(KT / nsets)
  int max_units;          // capacity of the block's unit list (>= units of any block, multiple of 2)
  int tr0, ntr;           // tile rows this launch covers: tr0 .. tr0 + ntr - 1
  int drop_unit;          // test switch: block 0 never copies this unit of its list (-1: none), so that the waits
                          // for it run out and the give-up path can be exercised without a fault
};

// Shared-memory pieces of the ring (carved by the kernel; sizes: ring_fixed_bytes below).
struct RingMem {
  uint64_t* full;         // [kRingMaxSlots] a buffer's copy has landed
  uint64_t* empty;        // [kRingMaxSlots] a buffer's consumer is done
  uint32_t* released;     // [kRingMaxSlots] rounds released so far
  int* next_unit;         // the list's shared counter; next_unit[1..2] = slow / other tiles placed so far
  UnitMeta* meta;         // [max_units]
  uint32_t* bufs;         // [slots][buf_words]
  // p: 16-byte aligned; a kernel's own shared arrays come before the ring
  __device__ __forceinline__ void carve(void* p, const RingArgs& A) {
    full = reinterpret_cast<uint64_t*>(p);
    empty = full + kRingMaxSlots;
    released = reinterpret_cast<uint32_t*>(empty + kRingMaxSlots);
    next_unit = reinterpret_cast<int*>(released + kRingMaxSlots);
    meta = reinterpret_cast<UnitMeta*>(next_unit + 4);
    bufs = reinterpret_cast<uint32_t*>(meta + A.max_units);
  }
};
__host__ __device__ constexpr size_t ring_fixed_bytes(int max_units) {
  return 2 * kRingMaxSlots * 8 + kRingMaxSlots * 4 + 16 + static_cast<size_t>(max_units) * sizeof(UnitMeta);
}

// The share of one block: blocks b, b + nsets, ... serve the tile columns set, set + nsets, ... of the launch's rows.
struct BlockShare {
  int set, bi, nb_set, ncol, ntiles, tmine, nmine;
  // bidx of nblocks: this block among the blocks that work on the matrix (the whole grid, or a part of it when one
  // launch covers several matrices)
  __device__ __forceinline__ void init(const MatDev& M, const RingArgs& A, int split, int bidx, int nblocks) {
    set = bidx % A.nsets;
    bi = bidx / A.nsets;
    nb_set = (nblocks - set + A.nsets - 1) / A.nsets;                 // blocks of this set
    ncol = (M.KT - set + A.nsets - 1) / A.nsets;                      // tile columns of this set
    ntiles = A.ntr * ncol;                                            // tiles of this set
    tmine = bi < ntiles ? (ntiles - bi + nb_set - 1) / nb_set : 0;    // tiles of this block: bi + k nb_set
    nmine = tmine * split;                                            // its units
  }
};

__device__ __forceinline__ bool wait_released(const uint32_t* released, uint32_t round, unsigned int* err,
                                              uint32_t limit) {
  const uint32_t addr = smem_addr(released);
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    if (v >= round) return true;
    __nanosleep(100);   // do not take issue slots from the warps this one is waiting for
  }
  atomicOr(err, 1u);
  return false;
}

// Clears the counters of the list.  Call before the __syncthreads that precedes ring_build_list.
__device__ __forceinline__ void ring_reset(const RingMem& R) {
  if (threadIdx.x == 0) {
    R.next_unit[0] = 0;
    R.next_unit[1] = 0;
    R.next_unit[2] = 0;
  }
}

// The block's list: tiles bi, bi + nb_set, ... of the set, their SPLIT units in segment order, with the tiles that
// hold a symbol-by-symbol unit moved to the front (such a unit takes several times longer: started last, it would keep
// the whole block waiting).  The order within the two classes is whatever the counters hand out; results do not depend
// on it.  Also initialises the barriers of the ring.  All threads of the block call this between two __syncthreads.
template <int SPLIT>
__device__ __forceinline__ void ring_build_list(const MatDev& M, const RingArgs& A, const BlockShare& S,
                                                const RingMem& R) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* list_count = R.next_unit + 1;
  for (int k0 = warp * 32; k0 < S.nmine; k0 += (blockDim.x >> 5) * 32) {
    const int k = k0 + lane, seg = lane % SPLIT;
    const bool valid = k < S.nmine, leader = seg == 0;
    int tr = 0, j = 0;
    uint32_t g0 = 0, g1 = 0, g2 = 0, cls = 0;
    bool slow = false;
    if (valid) {
      const int v = S.bi + (k / SPLIT) * S.nb_set;   // tile of the set -> (tile row, column index in the set)
      j = v % S.ncol;
      tr = A.tr0 + v / S.ncol;
      const int t = tr * M.KT + S.set + A.nsets * j;
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
    int tpos = slow ? base_s + __popc(bs & below) : S.tmine - 1 - (base_f + __popc(bf & below));
    tpos = __shfl_sync(0xffffffffu, tpos, lane - seg);   // the tile's position, from its leader
    if (valid) {
      const int pos = tpos * SPLIT + seg;
      R.meta[pos] = UnitMeta{g0,
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
    mbar_init(smem_addr(R.full + threadIdx.x), 1);
    mbar_init(smem_addr(R.empty + threadIdx.x), 1);
    R.released[threadIdx.x] = 0u;
  }
}

// Producers: issuer s = pwarp * producer_lanes + lane owns buffers s, s + S, ... (S issuers) and feeds them round by
// round, i.e. in the order of the block's list.  Issuing a bulk copy takes a few hundred cycles, so several issuers
// keep more copies in flight.  pwarp = index of the calling warp among the producer warps.
__device__ __forceinline__ void ring_produce(const MatDev& M, const RingArgs& A, const RingMem& R, int nmine, int pwarp,
                                             int lane) {
  if (lane >= A.producer_lanes) return;
  const int issuers = A.producers * A.producer_lanes;
  for (int round = 0; round * A.slots < nmine; ++round)
    for (int slot = pwarp * A.producer_lanes + lane; slot < A.slots; slot += issuers) {
      const int k = round * A.slots + slot;
      if (k >= nmine) break;
      if (round > 0) {
        if (!wait_released(R.released + slot, round, A.err, A.wait_limit)) return;
        if (!mbar_wait(smem_addr(R.empty + slot), (round - 1) & 1, A.err, A.wait_limit)) return;
      }
      if (k == A.drop_unit && blockIdx.x == 0) continue;
      const UnitMeta um = R.meta[k];
      bulk_load(smem_addr(R.bufs + static_cast<size_t>(slot) * A.buf_words), M.words + um.src, um.lines * 128u,
                smem_addr(R.full + slot));
    }
}

// One drawn unit, unpacked.
struct Unit {
  uint32_t lines, second, tr, round, j, seg, slot, cls;
  int k;
  const uint32_t* buf;
};

// Consumers: the next unit of the list, its buffer filled.  Returns 0 when the list is exhausted, -1 when a wait gave
// up (the warp must leave), 1 otherwise.
__device__ __forceinline__ int ring_draw(const RingArgs& A, const RingMem& R, int nmine, int lane, Unit& u) {
  int k = 0;
  if (lane == 0) k = atomicAdd(R.next_unit, 1);
  k = __shfl_sync(0xffffffffu, k, 0);
  if (k >= nmine) return 0;
  const uint4 raw = *reinterpret_cast<const uint4*>(R.meta + k);
  u.k = k;
  u.lines = raw.y & 0xFFFFu;
  u.second = (raw.y >> 16) & 0x3FFFu;
  u.cls = raw.y >> 30;
  u.tr = raw.z & 0xFFFFu;
  u.round = raw.z >> 16;
  u.j = raw.w & 255u;
  u.seg = (raw.w >> 8) & 255u;
  u.slot = (raw.w >> 16) & 255u;
  u.buf = R.bufs + static_cast<size_t>(u.slot) * A.buf_words;
  if (u.round > 0 && !wait_released(R.released + u.slot, u.round, A.err, A.wait_limit)) return -1;
  if (!mbar_wait(smem_addr(R.full + u.slot), u.round & 1, A.err, A.wait_limit)) return -1;
  return 1;
}

// Every lane has read its last word: hand the buffer back to the producer.
__device__ __forceinline__ void ring_release(const RingMem& R, const Unit& u, int lane) {
  __syncwarp();
  if (lane == 0) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(R.empty + u.slot)) : "memory");
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_addr(R.released + u.slot)), "r"(u.round + 1u)
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------- replicated table
//
// 32-bit decode-table entries (lw::fat_table): the code length sits in the top four bits, so the bit position advances
// with one multiply-high-and-add (FMA pipe, not the half-rate integer pipe), and the grid values of the symbol are
// signed bytes.  The table is replicated so that lanes read their own banks: with one copy, 32 lanes looking up 32
// pseudo-random windows collide about 3.4 ways and the shared-memory pipe (one 128-byte wavefront per clock per SM) is
// the bound.  R = 2^LOG_R copies of a table of 2^IDXBITS windows: entry address = (window << (LOG_R + 2)) |
// (lane % R) << 2.  Every chain starts with pad = LOG_R + 2 zero bits, which puts the window on exactly those address
// bits of the funnel-shifted word: the entry address is one three-input logic operation.
//
// Spreads 32 entries held by a warp (lane l holds entry i0 + l): broadcast one by one, every lane stores its own copy
// (bank = lane, no conflicts).  With 16 copies two entries go out per store.  tab1 = the single-copy table.
template <int LOG_R, bool SINGLE = true>
__device__ __forceinline__ void table_spread(uint32_t* tab, uint32_t* tab1, int i0, uint32_t mine, int lane) {
  constexpr int R = 1 << LOG_R, PER = 32 / R;   // entries per store: lane l writes copy l % R of entry i0 + j + l / R
#pragma unroll 8
  for (int j = 0; j < 32; j += PER) {
    const uint32_t v = __shfl_sync(0xffffffffu, mine, j + (lane >> LOG_R));
    tab[(i0 + j) * R + lane] = v;
  }
  if (SINGLE) tab1[i0 + lane] = mine;
}

// The whole table, by `nwarps` warps (warp, lane = the caller's position among them).  SINGLE = false: no single-copy
// table (a kernel whose replicated table already holds all 2048 windows has no use for it).
template <int IDXBITS, int LOG_R, bool SINGLE = true>
__device__ __forceinline__ void table_fill(const MatDev& M, uint32_t* tab, uint32_t* tab1, int warp, int lane,
                                           int nwarps) {
  constexpr int NIDX = 1 << IDXBITS;
  for (int i0 = warp * 32; i0 < NIDX; i0 += nwarps * 32)
    table_spread<LOG_R, SINGLE>(tab, tab1, i0, __ldg(M.tab32 + i0 + lane), lane);
  if (SINGLE)
    for (int idx = NIDX + warp * 32 + lane; idx < kLutSize; idx += nwarps * 32) tab1[idx] = __ldg(M.tab32 + idx);
}

// The same in two steps, for kernels that have set-up to do between them: issue() starts up to PRE loads per lane right
// at the kernel's start (their latency, a DRAM miss for the first block that touches the table, then overlaps the unit
// list's own loads and barriers), finish() spreads them and loads whatever a small block has left.
template <int IDXBITS, int LOG_R, bool SINGLE = true, int PRE = 8>
struct TableLoad {
  static constexpr int NIDX = 1 << IDXBITS;
  uint32_t pre[PRE];
  __device__ __forceinline__ void issue(const uint32_t* src, int warp, int lane, int nwarps) {
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int i0 = (i * nwarps + warp) * 32;
      pre[i] = warp < nwarps && i0 < NIDX ? __ldg(src + i0 + lane) : 0u;
    }
  }
  __device__ __forceinline__ void finish(const uint32_t* src, uint32_t* tab, uint32_t* tab1, int warp, int lane, int nwarps) const {
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int i0 = (i * nwarps + warp) * 32;
      if (i0 < NIDX) table_spread<LOG_R, SINGLE>(tab, tab1, i0, pre[i], lane);
    }
    for (int i0 = (PRE * nwarps + warp) * 32; i0 < NIDX; i0 += nwarps * 32)
      table_spread<LOG_R, SINGLE>(tab, tab1, i0, __ldg(src + i0 + lane), lane);
    if (SINGLE)
      for (int idx = NIDX + warp * 32 + lane; idx < kLutSize; idx += nwarps * 32) tab1[idx] = __ldg(src + idx);
  }
};

// ------------------------------------------------------------------------------------------------ tile stores
//
// Output of the decode-only kernels.  A lane owns two rows of a tile, so a plain store instruction of a warp touches 32
// different lines and passes the load/store pipe once per line - the pipe the table lookups already fill.  Instead a
// warp collects 32 bytes of each of its 64 rows in shared memory (2 KB, two 16-byte stores per lane and row) and one lane
// hands the 64 x 32-byte box to the tensor-copy engine (cp.async.bulk.tensor shared -> global, a plain store of this GPU's
// own memory), which writes whole sectors without the load/store pipe.  The tensor map (built on the host per output
// buffer, bytes as elements: [rows][row bytes]) uses the 32-byte swizzle: the 16-byte half of a row is exchanged where
// address bit 7 is set, which is exactly what spreads the lanes' 16-byte stores over all banks.
// wait_group is a hardware wait on the issuing lane's own copies, not a spin on memory.
struct WarpTileStage {
  static constexpr int kBytes = 2048;
  uint32_t base, row_a, swz;   // shared addresses: the warp's area (1024-byte aligned), this lane's first row
  __device__ __forceinline__ void init(const void* warp_area, int lane) {
    base = smem_addr(warp_area);
    row_a = base + lane * 32;          // row lane; row lane + 32 is 1024 bytes further (same address bit 7)
    swz = ((lane >> 2) & 1) * 16;
  }
  // the box sent last has been read: the area may be written again
  __device__ __forceinline__ void reuse(int lane) const {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
  }
  __device__ __forceinline__ void put(int second, const uint32_t (&w)[8]) const {
    const uint32_t a = row_a + second * 1024;
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a + swz), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a + (16u ^ swz)), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
  }
  // x: byte column (a multiple of 32), y: first of the 64 rows
  __device__ __forceinline__ void send(const void* tensor_map, int x, int y, int lane) const {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tensor_map), "r"(x), "r"(y), "r"(base)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  // before the warp exits: its copies are complete
  __device__ __forceinline__ void drain(int lane) const {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
};

// ------------------------------------------------------------------------------------------------ chain reader
//
// Refills are checked once per group of G symbols: the 64-bit window is normalised to the chain's bit position when a
// group starts (two funnel shifts), the G symbols only add their lengths to a local offset, one predicated word shift
// follows.  That is exact only while every symbol of a group starts within 31 bits of the group and one word per group
// keeps up; the loader (lw::walk_blob) checks both for every chain of the matrix, picks the largest G that leaves few
// exceptions, and flags the work units that hold one: those run with groups of two symbols, which is exact for any
// data.  With the 10-bit table, a unit that holds an 11-bit code is decoded symbol by symbol through the single-copy
// table of all 2048 windows.
struct GroupChain {
  const uint32_t* p;
  uint32_t w0, w1, w2, bp;   // three stream words; bp = bits consumed so far (its low five bits place the window)
  uint32_t a, b, off;        // window normalised to bp, offset inside the group
  // bp0: pad bits to skip.  A chain is laid out with kRingLogCopies + 2 leading zero bits; a kernel whose table has
  // fewer copies (2^LOG_R) wants the window LOG_R + 2 bits up in the shifted word, i.e. starts kRingLogCopies - LOG_R
  // bits into the pad.
  __device__ __forceinline__ void init(const uint32_t* chain_words, uint32_t bp0 = 0) {
    w0 = chain_words[0];
    w1 = chain_words[32];
    w2 = chain_words[64];
    p = chain_words + 96;
    bp = bp0;
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

// The reader of the pair layouts (lw::build_pairs): every group starts by loading its three words from the chain at
// the word its bit position has reached - no refill, no branch, nothing kept between groups but the position - so a
// group may use up any number of words.  What remains of the grouping rule is that its last symbol starts within 31
// bits of its first: always true for groups of three symbols of at most 12 bits.  (Measured on the 11-bit codes of
// the bundle formats this reader is a few per cent slower than GroupChain: two more shared-memory loads per group.  A
// variant of GroupChain that holds a fourth word and refills up to twice per group was measured on the pair layout too:
// 119 M instead of 81 M instructions for eight 14336 x 4096 products, 22.4 instead of 18.3 us each.)
struct ReloadChain {
  const uint32_t* base;
  uint32_t bp;
  uint32_t a, b, off;
  __device__ __forceinline__ void init(const uint32_t* chain_words, uint32_t bp0 = 0) {
    base = chain_words;
    bp = bp0;
  }
  __device__ __forceinline__ void begin() {
    const uint32_t* q = base + (bp >> 5) * 32u;
    const uint32_t w0 = q[0], w1 = q[32], w2 = q[64];
    a = __funnelshift_r(w0, w1, bp);
    b = __funnelshift_r(w1, w2, bp);
    off = 0;
  }
  template <uint32_t MASK>
  __device__ __forceinline__ uint32_t sym(const uint8_t* tab, uint32_t lane_off) {
    const uint32_t t = __funnelshift_r(a, b, off);
    const uint32_t e = *reinterpret_cast<const uint32_t*>(tab + ((t & MASK) | lane_off));
    off = __umulhi(e, 16u) + off;
    return e;
  }
  __device__ __forceinline__ void end() { bp += off; }
  __device__ __forceinline__ uint32_t slow_sym(const uint32_t* tab32, uint32_t pad) {
    const uint32_t* q = base + (bp >> 5) * 32u;
    const uint32_t e = tab32[(__funnelshift_r(q[0], q[32], bp) >> pad) & (kLutSize - 1)];
    bp += e >> 28;
    return e;
  }
};

// Pair layouts with an 11-bit code are laid out WITHOUT pad bits: three symbols of at most 11 bits need 33 bits after
// the bit position, which the two words a group starts in always hold (position mod 32 <= 31, 31 + 33 = 64), so a group
// loads two words instead of three; the price is one instruction per lookup (the window is shifted up onto the table's
// address bits instead of being read where the pad put it) in a kernel whose issue slots are half empty and whose
// shared-memory pipe is full.
struct ReloadChain2 {
  const uint32_t* base;
  uint32_t bp;
  uint32_t a, b, off;
  __device__ __forceinline__ void init(const uint32_t* chain_words, uint32_t = 0) {
    base = chain_words;
    bp = 0;
  }
  __device__ __forceinline__ void begin() {
    const uint32_t* q = base + (bp >> 5) * 32u;
    const uint32_t w0 = q[0], w1 = q[32];
    a = __funnelshift_r(w0, w1, bp);
    b = w1 >> (bp & 31u);
    off = 0;
  }
  template <uint32_t MASK>
  __device__ __forceinline__ uint32_t sym(const uint8_t* tab, uint32_t lane_off) {
    constexpr int SH = __builtin_ctz(MASK);
    const uint32_t t = __funnelshift_r(a, b, off);
    const uint32_t e = *reinterpret_cast<const uint32_t*>(tab + (((t << SH) & MASK) | lane_off));
    off = __umulhi(e, 16u) + off;
    return e;
  }
  __device__ __forceinline__ void end() { bp += off; }
  __device__ __forceinline__ uint32_t slow_sym(const uint32_t* tab32, uint32_t) {
    const uint32_t* q = base + (bp >> 5) * 32u;
    const uint32_t e = tab32[__funnelshift_r(q[0], q[32], bp) & (kLutSize - 1)];
    bp += e >> 28;
    return e;
  }
};

// The reader of a kernel instantiation: pair layouts by the width of their code, everything else GroupChain.
template <bool PAIR_LAYOUT, int IDXBITS>
struct ChainOf {
  using type = GroupChain;
};
template <>
struct ChainOf<true, 12> {
  using type = ReloadChain;
};
template <>
struct ChainOf<true, 11> {
  using type = ReloadChain2;
};
// zero bits at the start of every chain of a pair layout
__host__ __device__ constexpr int pair_pad_bits(int index_bits) { return index_bits == 11 ? 0 : kRingLogCopies + 2; }

// Scales of the unit's two rows (row `lane` and row `lane + 32`), read from the block that follows the unit's chain
// words in its staging buffer (layout: lw::unit_side_words).  sub(j) = (scale, offset) of sub-block j (a constant
// after unrolling): weight = scale * f(code) - offset, every operation rounded separately in float32 (llama.cpp's
// block formulas; reference: scripts/a2_kq_bundle.py:50-68, kernels/llmrt.cu:126-149).
template <int FMT>
struct UnitSide {
  uint32_t sc, mn, dd;   // Q6KP: mn = scales of sub-blocks 4..7
  __device__ __forceinline__ void load(const uint32_t* sb, int row) {
    if (FMT == kFmtQ4K || FMT == kFmtQ5K || FMT == kFmtQ5KP) {
      dd = sb[row];
      sc = sb[64 + row];
      mn = sb[128 + row];
    } else if (FMT == kFmtQ6KP) {
      sc = sb[row];
      mn = sb[64 + row];
      dd = reinterpret_cast<const uint16_t*>(sb)[256 + row];
    } else {
      sc = sb[row];
      dd = reinterpret_cast<const uint16_t*>(sb)[128 + row];
      mn = 0;
    }
  }
  __device__ __forceinline__ void sub(int j, float& s, float& o) const {
    const uint32_t q = ((FMT == kFmtQ6KP && j >= 4 ? mn : sc) >> (8 * (j & 3))) & 255u;
    if (FMT == kFmtQ6K || FMT == kFmtQ6KP) {
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

}  // namespace lw
