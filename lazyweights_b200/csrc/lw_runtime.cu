// Decoder runtime around the coded matrices (the "next" rows of the path: what rt_forward needs).
//
// Mirrors the token step of the reference runtime (kernels/llmrt.cu:2291-2436): embedding gather, RMSNorm with the
// residual add folded in (:1288-1301), rotate-half RoPE + fp16 KV-cache write (:1305-1332), causal grouped-query
// attention with per-query arithmetic that does not depend on the number of tokens in the pass (:1336-1498), SwiGLU
// (:1500-1505), coded matrices through the fused decode + product kernels.  Activations fp32, KV cache fp16
// [layer][kv head][position][head dim].  Tensor parallelism: a rank opens ITS shard of the model as a bundle whose
// cfg carries the local head / FFN / vocabulary sizes; partial outputs of `o` and `down` are summed with NCCL
// all-reduce and the logits are gathered (rt_tp_init).
#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <sstream>
#include <thread>

#include "../../include/lwb200.h"
#include "lw_model.h"

namespace lw {

// ------------------------------------------------------------------------------------------------ NCCL by dlopen
// The process (PyTorch) already carries an NCCL; binding it at run time avoids a second copy at link time.
struct Nccl {
  void* lib = nullptr;
  int (*GetUniqueId)(void*) = nullptr;
  int (*CommInitRank)(void**, int, const void*, int) = nullptr;   // ncclUniqueId is passed by value: see init()
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  int (*CommGetAsyncError)(void*, int*) = nullptr;   // optional
  int (*CommAbort)(void*) = nullptr;                 // optional
  const char* (*GetErrorString)(int) = nullptr;
  void* init_rank_sym = nullptr;
  bool load() {
    if (lib) return true;
    for (const char* n : {"libnccl.so.2", "libnccl.so"}) {
      lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (lib) break;
    }
    if (!lib) return false;
    GetUniqueId = reinterpret_cast<int (*)(void*)>(dlsym(lib, "ncclGetUniqueId"));
    init_rank_sym = dlsym(lib, "ncclCommInitRank");
    AllReduce = reinterpret_cast<decltype(AllReduce)>(dlsym(lib, "ncclAllReduce"));
    AllGather = reinterpret_cast<decltype(AllGather)>(dlsym(lib, "ncclAllGather"));
    CommDestroy = reinterpret_cast<decltype(CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
    GetErrorString = reinterpret_cast<decltype(GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
    CommGetAsyncError = reinterpret_cast<decltype(CommGetAsyncError)>(dlsym(lib, "ncclCommGetAsyncError"));
    CommAbort = reinterpret_cast<decltype(CommAbort)>(dlsym(lib, "ncclCommAbort"));
    return GetUniqueId && init_rank_sym && AllReduce && AllGather && CommDestroy;
  }
};
static Nccl g_nccl;
struct UniqueId { char bytes[128]; };
constexpr int kNcclFloat = 7, kNcclSum = 0;

// error word of this file's kernels (bit 0: the peer all-reduce gave up waiting for a rank)
__device__ unsigned int g_rt_error;

struct Runtime {
  int L = 0, D = 0, H = 0, Hk = 0, Dh = 0, I = 0, V = 0;   // heads, FFN width and vocabulary are the LOCAL sizes
  int Tmax = 0, max_batch = 0, pos = 0, window = 0;
  int tp_rank = 0, tp_world = 1;
  int Vfull = 0, Vmax = 0;           // whole vocabulary; largest shard (ranks may hold 63 or 62 tile rows, say)
  std::vector<int> voff, vcnt;       // first row and rows of every rank's vocabulary shard
  bool time_collectives = false;     // next pass: direct launches with CUDA events around every collective
  // peer-memory all-reduce (rt_tp_peer_open): every rank's exchange buffer mapped into every other rank
  void* peer_local = nullptr;                 // this rank's buffer (cudaMalloc; exported with cudaIpcGetMemHandle)
  void* peer_base[8] = {nullptr};             // the ranks' buffers as seen from this process (own = peer_local)
  bool peer_ready = false;
  size_t peer_bytes = 0;
  std::vector<cudaEvent_t> coll_events;
  double collective_us = 0.0;        // time inside collectives during the last such pass
  int collective_calls = 0;
  float eps = 1e-5f, attn_scale = 1.f;
  void* comm = nullptr;
  float *h = nullptr, *xn = nullptr, *att = nullptr, *o = nullptr, *qkv = nullptr, *g = nullptr, *u = nullptr;
  float *logits = nullptr, *logits_all = nullptr, *cosv = nullptr, *sinv = nullptr, *lnf = nullptr;
  float* attn_part = nullptr;   // [max_batch][H][max_chunks][Dh + 2]
  unsigned int* attn_done = nullptr;   // [max_batch][H] chunk blocks finished per (token, head group); zero between passes
  int max_chunks = 1;
  int* ids = nullptr;          // device: max_batch token ids, then the position of the pass (read by the kernels, so
                               // that a captured graph replays at any position, as kernels/llmrt.cu:1308 does)
  int* h_ids = nullptr;        // pinned host copy of the same
  int* gen = nullptr;          // [Tmax] tokens generated by rt_decode_greedy (device)
  int wait_timeout_ms = 0;     // rt_tp_set_timeout: overrides LW_TP_TIMEOUT_MS for this handle (0: the default)
  bool tp_failed = false;      // a guarded wait gave up: the communicator is gone
  cudaStream_t stream = nullptr;
  bool graphs = true;
  std::map<long long, cudaGraphExec_t> graph_exec;
  std::map<long long, int> graph_seen;
  long long graph_launches = 0, graph_captures = 0;
  __half *kc = nullptr, *vc = nullptr, *embed16 = nullptr;
  uint8_t* embed8 = nullptr;
  float *embed_rs = nullptr, *embed_rsub = nullptr;
  int embed_groups = 0, embed_rows = 0;
  std::vector<float*> ln1, ln2;
  std::vector<int> m_qkv, m_q, m_k, m_v, m_o, m_gate, m_up, m_down;
  int m_head = -1;
  std::vector<void*> owned;   // device allocations to free
  std::vector<int> eos;
};

// ----------------------------------------------------------------------------------------------------- kernels

__global__ void k_embed16(const int* __restrict__ ids, const __half* __restrict__ E, float* __restrict__ h, int D) {
  const __half* row = E + static_cast<size_t>(ids[blockIdx.x]) * D;
  for (int k = threadIdx.x; k < D; k += blockDim.x) h[static_cast<size_t>(blockIdx.x) * D + k] = __half2float(row[k]);
}

// raw8 embedding with per-group scale / offset, rounded to fp16 like the reference's gather (kernels/llmrt.cu:1261-1274)
__global__ void k_embed8(const int* __restrict__ ids, const uint8_t* __restrict__ E, const float* __restrict__ rs,
                         const float* __restrict__ rsub, float* __restrict__ h, int D, int G) {
  const int id = ids[blockIdx.x], sub = D / G;
  for (int k = threadIdx.x; k < D; k += blockDim.x) {
    const float v = (static_cast<float>(E[static_cast<size_t>(id) * D + k]) - rsub[static_cast<size_t>(id) * G + k / sub]) *
                    rs[static_cast<size_t>(id) * G + k / sub];
    h[static_cast<size_t>(blockIdx.x) * D + k] = __half2float(__float2half_rn(v));
  }
}

// Programmatic dependent launch (see lw_device.cuh): every kernel of a pass lets its successor be set up at once and
// waits for its predecessor before it reads or writes anything.
__device__ __forceinline__ void dep_begin() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static void launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// h += res (if res), out = h * rsqrt(mean(h^2) + eps) * g.  One block of 1024 threads per token; every thread keeps up
// to eight elements in registers (float4 loads), so the row is read once.  Longer rows fall back to a second read.
constexpr int kNormThreads = 1024;
__global__ void __launch_bounds__(kNormThreads)
    k_rmsnorm(float* __restrict__ h, const float* __restrict__ res, const float* __restrict__ g,
              float* __restrict__ out, int D, float eps) {
  dep_begin();
  __shared__ float red[33];
  float* hr = h + static_cast<size_t>(blockIdx.x) * D;
  const float* rr = res ? res + static_cast<size_t>(blockIdx.x) * D : nullptr;
  float* orow = out + static_cast<size_t>(blockIdx.x) * D;
  const bool vec = (D & 3) == 0 && D <= 8 * kNormThreads;
  float4 v[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  float ss = 0.f;
  if (vec) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = (i * kNormThreads + threadIdx.x) * 4;
      if (k < D) {
        v[i] = *reinterpret_cast<const float4*>(hr + k);
        if (rr) {
          const float4 r4 = *reinterpret_cast<const float4*>(rr + k);
          v[i].x += r4.x;
          v[i].y += r4.y;
          v[i].z += r4.z;
          v[i].w += r4.w;
          *reinterpret_cast<float4*>(hr + k) = v[i];
        }
        ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
      }
    }
  } else {
    for (int k = threadIdx.x; k < D; k += blockDim.x) {
      float x = hr[k];
      if (rr) {
        x += rr[k];
        hr[k] = x;
      }
      ss += x * x;
    }
  }
  for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) red[32] = rsqrtf(t / D + eps);
  }
  __syncthreads();
  const float r = red[32];
  if (vec) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = (i * kNormThreads + threadIdx.x) * 4;
      if (k < D) {
        const float4 g4 = *reinterpret_cast<const float4*>(g + k);
        *reinterpret_cast<float4*>(orow + k) = make_float4(v[i].x * r * g4.x, v[i].y * r * g4.y, v[i].z * r * g4.z,
                                                           v[i].w * r * g4.w);
      }
    }
  } else {
    for (int k = threadIdx.x; k < D; k += blockDim.x) orow[k] = hr[k] * r * g[k];
  }
}

// ---------------------------------------------------------------------------------- all-reduce fused with the norm
//
// Tensor-parallel ranks hold partial outputs of the row-parallel matrices (o, down); their sum is the residual the next
// RMSNorm adds.  Instead of a library all-reduce followed by the norm kernel, ONE kernel per rank does both over peer
// memory (one-shot, all-to-all): every rank stores its partial row into its slot of EVERY rank's exchange buffer (plain
// stores through NVLink), publishes a flag per destination (release at system scope), waits until the flags of all ranks
// have arrived in its own buffer, adds the slots in rank order (every rank adds the same numbers in the same order: the
// ranks' results are identical, as after an all-reduce) and goes on with the norm.  At one token the payload is 16 KB per
// rank and destination: the cost is latency, and this is two NVLink traversals (data, then flag) instead of a library
// call's protocol.  Only ordinary loads and stores touch peer memory - no multicast of any kind.
//
// Exchange buffer of a rank: [kPeerMaxBlocks epoch counters][flags: 2 parities x kPeerMaxBlocks x 8 ranks][slots:
// 2 parities x 8 ranks x kPeerMaxBlocks rows x D floats].  Block j (token row j) keeps its own epoch: the number of
// all-reduces it has taken part in; slot and flag parity = epoch & 1, so a rank that is one all-reduce ahead never
// overwrites data a slower rank still reads (it cannot be two ahead: it needs the slower rank's contribution first).
// The wait is bounded: after `limit` polls the block sets the device error word and continues with what it has.
constexpr int kPeerMaxBlocks = 8, kPeerMaxRanks = 8;
struct PeerView {
  float* slots[kPeerMaxRanks];       // rank p's slot area, as mapped here
  uint32_t* flags[kPeerMaxRanks];    // rank p's flag area
  uint32_t* epoch;                   // this rank's epoch counters
  int world, rank, D;
};
__host__ __device__ constexpr size_t peer_flag_words() { return 2 * kPeerMaxBlocks * kPeerMaxRanks; }
__host__ __device__ inline size_t peer_slot_floats(int D) { return static_cast<size_t>(2) * kPeerMaxRanks * kPeerMaxBlocks * D; }

__global__ void __launch_bounds__(kNormThreads)
    k_allreduce_rmsnorm(PeerView P, const float* __restrict__ part, float* __restrict__ h, const float* __restrict__ g,
                        float* __restrict__ out, float eps, unsigned int* err, uint32_t limit) {
  dep_begin();
  __shared__ float red[33];
  __shared__ uint32_t s_epoch;
  const int j = blockIdx.x, D = P.D;
  if (threadIdx.x == 0) s_epoch = P.epoch[j];
  __syncthreads();
  const uint32_t e = s_epoch, parity = e & 1u;
  const size_t row = (static_cast<size_t>(parity) * kPeerMaxRanks * kPeerMaxBlocks + static_cast<size_t>(j)) * D;   // + rank * kPeerMaxBlocks * D
  // 1. my partial row into my slot of every rank's buffer
  const float* mine = part + static_cast<size_t>(j) * D;
  for (int k = threadIdx.x * 4; k < D; k += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(mine + k);
    for (int p = 0; p < P.world; ++p)
      *reinterpret_cast<float4*>(P.slots[p] + row + static_cast<size_t>(P.rank) * kPeerMaxBlocks * D + k) = v;
  }
  __threadfence_system();
  __syncthreads();
  // 2. publish: flag (parity, block j, source rank) of every destination := e + 1
  const size_t flag_at = (static_cast<size_t>(parity) * kPeerMaxBlocks + j) * kPeerMaxRanks;
  if (threadIdx.x < P.world) {
    uint32_t* dst = P.flags[threadIdx.x] + flag_at + P.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(e + 1u) : "memory");
  }
  // 3. wait for every rank's flag in my own buffer
  if (threadIdx.x < P.world) {
    const uint32_t* src = P.flags[P.rank] + flag_at + threadIdx.x;
    bool ok = false;
    for (uint32_t i = 0; i < limit && !ok; ++i) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
      ok = v == e + 1u;
    }
    if (!ok) atomicOr(err, 1u);
  }
  __syncthreads();
  // 4. sum in rank order + residual, then the norm (as k_rmsnorm)
  float* hr = h + static_cast<size_t>(j) * D;
  float* orow = out + static_cast<size_t>(j) * D;
  const float* my_slots = P.slots[P.rank] + row;
  float ss = 0.f;
  for (int k = threadIdx.x * 4; k < D; k += blockDim.x * 4) {
    float4 acc = *reinterpret_cast<const float4*>(hr + k);
    for (int r = 0; r < P.world; ++r) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(my_slots + static_cast<size_t>(r) * kPeerMaxBlocks * D + k));
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    *reinterpret_cast<float4*>(hr + k) = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) {
      red[32] = rsqrtf(t / D + eps);
      P.epoch[j] = e + 1u;
    }
  }
  __syncthreads();
  const float r = red[32];
  for (int k = threadIdx.x * 4; k < D; k += blockDim.x * 4) {
    const float4 hv = *reinterpret_cast<const float4*>(hr + k);
    const float4 g4 = *reinterpret_cast<const float4*>(g + k);
    *reinterpret_cast<float4*>(orow + k) = make_float4(hv.x * r * g4.x, hv.y * r * g4.y, hv.z * r * g4.z, hv.w * r * g4.w);
  }
}

// rotate-half RoPE on q (in place) and k (into the cache), v into the cache.  grid (heads + 2 kv heads, tokens).
__global__ void k_rope_cache(float* __restrict__ qkv, const float* __restrict__ cosv, const float* __restrict__ sinv,
                             __half* __restrict__ kc, __half* __restrict__ vc, const int* __restrict__ posp, int H, int Hk,
                             int Dh, int Tmax) {
  dep_begin();
  const int head = blockIdx.x, j = blockIdx.y, p = *posp + j, half = Dh / 2;
  float* row = qkv + static_cast<size_t>(j) * (H + 2 * Hk) * Dh + static_cast<size_t>(head) * Dh;
  if (head < H + Hk) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float c = cosv[static_cast<size_t>(p) * half + i], s = sinv[static_cast<size_t>(p) * half + i];
      const float a = row[i], b = row[i + half];
      const float ra = a * c - b * s, rb = b * c + a * s;
      if (head < H) {
        row[i] = ra;
        row[i + half] = rb;
      } else {
        __half* dst = kc + (static_cast<size_t>(head - H) * Tmax + p) * Dh;
        dst[i] = __float2half_rn(ra);
        dst[i + half] = __float2half_rn(rb);
      }
    }
  } else {
    __half* dst = vc + (static_cast<size_t>(head - H - Hk) * Tmax + p) * Dh;
    for (int i = threadIdx.x; i < Dh; i += blockDim.x) dst[i] = __float2half_rn(row[i]);
  }
}

// Causal attention, split over the context so that a long context fills the GPU (one query token of one head is a
// single reduction otherwise).  k_attn: block (group of query heads, token, chunk of kAttnChunk positions) -> the chunk's
// score maximum, its sum of exponentials and the unnormalised weighted sum of v; the block that finishes LAST for a
// (head group, token) merges the chunks with the usual running-maximum rescaling (a counter per (token, head group)
// that the last block sets back to zero), so no second kernel and no wait: every block but one just leaves.  Per-query
// arithmetic does not depend on how many tokens the pass carries, nor on which block happens to be last (the merge
// always runs over the chunks in order).  Chunks of 64 positions: 256 blocks for a context of 2048 and 8 kv heads
// (with 128 positions and a separate merge kernel attention took 0.51 of 3.51 ms per token of the 7B-shaped model).
constexpr int kAttnChunk = 64, kAttnThreads = 256, kAttnMaxDh = 128;
constexpr int kAttnStride = kAttnMaxDh / 2 + 1;   // words per staged row: odd, so 32 consecutive rows hit 32 banks

// GH query heads that share one kv head (grouped-query attention) per block: the chunk's keys, then its values, are
// staged once in shared memory (16-byte loads) and serve all of them.
template <int GH>
__global__ void __launch_bounds__(kAttnThreads)
    k_attn(const float* __restrict__ qkv, const __half* __restrict__ kc, const __half* __restrict__ vc,
           float* __restrict__ part, float* __restrict__ att, unsigned int* __restrict__ done,
           const int* __restrict__ posp, int H, int Hk, int Dh, int Tmax, float scale, int window, int max_chunks) {
  dep_begin();
  __shared__ uint32_t kv[kAttnChunk * kAttnStride];
  __shared__ float qs[GH][kAttnMaxDh];
  __shared__ float sc[GH][kAttnChunk];
  __shared__ unsigned int s_last;
  constexpr int SLOTS = kAttnThreads / kAttnChunk;          // head slots of the score phase (4)
  constexpr int HS = (GH + SLOTS - 1) / SLOTS;              // heads per slot (1)
  constexpr int HV = GH >= 2 ? GH / 2 : 1;                  // heads per thread of the value phase: two halves of the block
  const int head0 = blockIdx.x * GH, j = blockIdx.y, c = blockIdx.z, kh = head0 / (H / Hk), last = *posp + j;
  const int lo = window > 0 ? max(0, last - window + 1) : 0;
  const int p0 = lo + c * kAttnChunk, n = min(kAttnChunk, last + 1 - p0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto out_of = [&](int h, int chunk) { return part + ((static_cast<size_t>(j) * H + head0 + h) * max_chunks + chunk) * (Dh + 2); };
  if (n <= 0) {   // chunk beyond this token's causal range
    if (threadIdx.x < GH) {
      float* out = out_of(threadIdx.x, c);
      out[0] = -INFINITY;
      out[1] = 0.f;
    }
  } else {
    const float* q = qkv + static_cast<size_t>(j) * (H + 2 * Hk) * Dh + static_cast<size_t>(head0) * Dh;
    for (int i = threadIdx.x; i < GH * Dh; i += kAttnThreads) qs[i / Dh][i % Dh] = q[i];
    const int cpr = Dh / 8;   // 16-byte pieces per row
    auto stage = [&](const __half* src) {
      for (int idx = threadIdx.x; idx < kAttnChunk * cpr; idx += kAttnThreads) {
        const int t = idx / cpr, ch = idx - t * cpr;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (t < n) v = __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(t) * Dh) + ch);
        uint32_t* d = kv + t * kAttnStride + ch * 4;
        d[0] = v.x;
        d[1] = v.y;
        d[2] = v.z;
        d[3] = v.w;
      }
    };
    stage(kc + (static_cast<size_t>(kh) * Tmax + p0) * Dh);
    // the chunk's values are requested now and parked in registers while the scores are computed: their DRAM latency
    // hides behind the score phase instead of following it
    constexpr int VPT = kAttnChunk * (kAttnMaxDh / 8) / kAttnThreads;   // 16-byte pieces per thread (4)
    uint4 vreg[VPT];
    {
      const __half* vsrc = vc + (static_cast<size_t>(kh) * Tmax + p0) * Dh;
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const int idx = threadIdx.x + u * kAttnThreads, t = idx / cpr, ch = idx - t * cpr;
        vreg[u] = make_uint4(0u, 0u, 0u, 0u);
        if (idx < kAttnChunk * cpr && t < n) vreg[u] = __ldg(reinterpret_cast<const uint4*>(vsrc + static_cast<size_t>(t) * Dh) + ch);
      }
    }
    __syncthreads();
    {   // scores of position t against the heads of this thread's slot
      const int t = threadIdx.x & (kAttnChunk - 1), slot = threadIdx.x / kAttnChunk;
      if (slot * HS < GH) {
        float acc[HS];
#pragma unroll
        for (int h = 0; h < HS; ++h) acc[h] = 0.f;
        const uint32_t* kr = kv + t * kAttnStride;
        for (int w = 0; w < Dh / 2; ++w) {
          const float2 kk = __half22float2(*reinterpret_cast<const __half2*>(kr + w));
#pragma unroll
          for (int h = 0; h < HS; ++h) {
            if (slot * HS + h < GH) {
              const float2 qq = *reinterpret_cast<const float2*>(&qs[slot * HS + h][2 * w]);
              acc[h] = fmaf(qq.x, kk.x, acc[h]);
              acc[h] = fmaf(qq.y, kk.y, acc[h]);
            }
          }
        }
#pragma unroll
        for (int h = 0; h < HS; ++h)
          if (slot * HS + h < GH) sc[slot * HS + h][t] = t < n ? acc[h] * scale : -INFINITY;
      }
    }
    __syncthreads();
    if (warp < GH) {   // one warp per head: maximum, exponentials, their sum
      constexpr int PER = kAttnChunk / 32;
      float s4[PER], mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        s4[i] = sc[warp][lane + 32 * i];
        mx = fmaxf(mx, s4[i]);
      }
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const float e = __expf(s4[i] - mx);   // exp(-inf) = 0 for the positions past n
        sc[warp][lane + 32 * i] = e;
        sum += e;
      }
      for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) {
        float* out = out_of(warp, c);
        out[0] = mx;
        out[1] = sum;
      }
    }
    __syncthreads();   // scores final, keys no longer needed
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int idx = threadIdx.x + u * kAttnThreads, t = idx / cpr, ch = idx - t * cpr;
      if (idx < kAttnChunk * cpr) {
        uint32_t* d = kv + t * kAttnStride + ch * 4;
        d[0] = vreg[u].x;
        d[1] = vreg[u].y;
        d[2] = vreg[u].z;
        d[3] = vreg[u].w;
      }
    }
    __syncthreads();
    const int t = threadIdx.x & (kAttnMaxDh - 1), hp = threadIdx.x / kAttnMaxDh;   // t = output dimension
    if (hp * HV < GH && t < Dh) {
      float acc[HV];
#pragma unroll
      for (int h = 0; h < HV; ++h) acc[h] = 0.f;
      const __half* vcol = reinterpret_cast<const __half*>(kv) + t;
      for (int p = 0; p < n; ++p) {
        const float v = __half2float(vcol[p * (2 * kAttnStride)]);
#pragma unroll
        for (int h = 0; h < HV; ++h) acc[h] = fmaf(sc[hp * HV + h][p], v, acc[h]);
      }
#pragma unroll
      for (int h = 0; h < HV; ++h) out_of(hp * HV + h, c)[2 + t] = acc[h];
    }
  }
  // the last block of this (token, head group) merges all chunks
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* cnt = done + static_cast<size_t>(j) * gridDim.x + blockIdx.x;
    const unsigned int old = atomicAdd(cnt, 1u);
    s_last = old == gridDim.z - 1 ? 1u : 0u;
    if (s_last) *cnt = 0u;   // ready for the next pass
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Merge.  The chunks' maxima and sums first (one load per thread), the weights exp(m_c - max) by one warp per head,
  // then every output sums its chunks with the loads of 16 chunks in flight at a time (they are L2 round trips: one
  // after the other, as a plain loop over the chunks issues them, they took longer than the attention itself).
  const int nchunks = gridDim.z;
  float* wgt = reinterpret_cast<float*>(kv);              // [GH][nchunks] weights (the staging area is free now)
  float* sums = wgt + GH * nchunks;                        // [GH][nchunks]
  float* tot_s = qs[0];                                    // [GH]
  constexpr int kMergeMax = kAttnChunk * kAttnStride / (2 * GH);   // chunks whose weights fit the staging area
  if (nchunks <= kMergeMax) {
    for (int i = threadIdx.x; i < GH * nchunks; i += kAttnThreads) {
      const int h = i / nchunks, ch = i - h * nchunks;
      const float* pc = out_of(h, ch);
      wgt[i] = __ldcg(pc);
      sums[i] = __ldcg(pc + 1);
    }
    __syncthreads();
    if (warp < GH) {
      float mx = -INFINITY;
      for (int ch = lane; ch < nchunks; ch += 32) mx = fmaxf(mx, wgt[warp * nchunks + ch]);
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float tot = 0.f;
      for (int ch = lane; ch < nchunks; ch += 32) {
        const float sm = sums[warp * nchunks + ch];
        const float w = sm > 0.f ? __expf(wgt[warp * nchunks + ch] - mx) : 0.f;
        wgt[warp * nchunks + ch] = w;
        tot += sm * w;
      }
      for (int o = 16; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
      if (lane == 0) tot_s[warp] = tot;
    }
    __syncthreads();
    for (int o = threadIdx.x; o < GH * Dh; o += kAttnThreads) {
      const int h = o / Dh, d = o - h * Dh;
      const float* col = out_of(h, 0) + 2 + d;
      const float* w = wgt + h * nchunks;
      float a = 0.f;
      for (int c0 = 0; c0 < nchunks; c0 += 16) {
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = c0 + u < nchunks ? __ldcg(col + static_cast<size_t>(c0 + u) * (Dh + 2)) : 0.f;
#pragma unroll
        for (int u = 0; u < 16; ++u) a = fmaf(c0 + u < nchunks ? w[c0 + u] : 0.f, v[u], a);   // in chunk order
      }
      att[static_cast<size_t>(j) * H * Dh + static_cast<size_t>(head0 + h) * Dh + d] = a / tot_s[h];
    }
    return;
  }
  for (int o = threadIdx.x; o < GH * Dh; o += kAttnThreads) {   // very long contexts: chunk by chunk
    const int h = o / Dh, d = o - h * Dh;
    float mx = -INFINITY;
    for (int ch = 0; ch < nchunks; ++ch) mx = fmaxf(mx, __ldcg(out_of(h, ch)));
    float tot = 0.f, a = 0.f;
    for (int ch = 0; ch < nchunks; ++ch) {
      const float* pc = out_of(h, ch);
      const float sum = __ldcg(pc + 1);
      if (sum > 0.f) {
        const float w = __expf(__ldcg(pc) - mx);
        tot += sum * w;
        a += __ldcg(pc + 2 + d) * w;
      }
    }
    att[static_cast<size_t>(j) * H * Dh + static_cast<size_t>(head0 + h) * Dh + d] = a / tot;
  }
}

// Greedy decoding on the device: the id of the largest logit (the lowest id among equals, like a host arg-max) becomes
// the next pass's token, the position advances, the token is appended to the list of generated tokens.  logits: one row;
// with W ranks the rank-major gather of their slices (slot r: Vmax floats, the first (base + (r < rem)) * 64 valid, ids
// from (r * base + min(r, rem)) * 64).  ids[0] = token of the next pass, ids[B] = its position, ids[B + 1] = tokens
// generated so far.  One block.
__global__ void __launch_bounds__(1024) k_argmax_next(const float* __restrict__ logits, int W, int Vmax, int base, int rem,
                                                      int* __restrict__ ids, int B, int* __restrict__ gen) {
  dep_begin();
  __shared__ float sv[32];
  __shared__ int si[32];
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  for (int r = 0; r < W; ++r) {
    const int cnt = (base + (r < rem ? 1 : 0)) * kTileRows, off = (r * base + min(r, rem)) * kTileRows;
    const float* row = logits + static_cast<size_t>(r) * Vmax;
    // eight loads in flight per thread (they are L2 / DRAM round trips: one after the other they took 18 us for 32000
    // logits), compared in the order of the ids
    for (int i0 = threadIdx.x; i0 < cnt; i0 += 8 * blockDim.x) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * blockDim.x;
        v[u] = i < cnt ? row[i] : -INFINITY;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (v[u] > best) {   // ids grow along the loops: a later equal value never replaces an earlier one
          best = v[u];
          best_id = off + i0 + u * static_cast<int>(blockDim.x);
        }
    }
  }
  auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
  for (int o = 16; o; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, best, o);
    const int j = __shfl_xor_sync(0xffffffffu, best_id, o);
    if (better(w, j, best, best_id)) {
      best = w;
      best_id = j;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = best_id;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x >> 5) ? sv[threadIdx.x] : -INFINITY;
    best_id = threadIdx.x < (blockDim.x >> 5) ? si[threadIdx.x] : 0x7fffffff;
    for (int o = 16; o; o >>= 1) {
      const float w = __shfl_xor_sync(0xffffffffu, best, o);
      const int j = __shfl_xor_sync(0xffffffffu, best_id, o);
      if (better(w, j, best, best_id)) {
        best = w;
        best_id = j;
      }
    }
    if (threadIdx.x == 0) {
      if (best_id == 0x7fffffff) best_id = 0;   // every logit NaN: any valid id keeps the next gather in range
      ids[0] = best_id;
      ids[B] += 1;
      gen[ids[B + 1]++] = best_id;
    }
  }
}

__global__ void k_silu_mul(float* __restrict__ g, const float* __restrict__ u, size_t n) {
  dep_begin();
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i < n) {
    const float v = g[i];
    g[i] = v / (1.f + __expf(-v)) * u[i];
  }
}

// ---------------------------------------------------------------------------------------------------- host side

static int cfg_int(const Model* M, const char* k, int def) {
  auto it = M->man.cfg.find(k);
  return it == M->man.cfg.end() ? def : atoi(it->second.c_str());
}
static double cfg_f(const Model* M, const char* k, double def) {
  auto it = M->man.cfg.find(k);
  return it == M->man.cfg.end() ? def : atof(it->second.c_str());
}

template <class T>
static int dalloc(Runtime* R, T** p, size_t count) {
  const cudaError_t e = cudaMalloc(reinterpret_cast<void**>(p), std::max<size_t>(count, 1) * sizeof(T));
  if (e != cudaSuccess) return cuda_fail("cudaMalloc (runtime)", e);
  R->owned.push_back(*p);
  return kOk;
}

// an uncoded tensor of the bundle -> device memory (f32 / f16 / raw8 as stored)
static int upload(Model* M, Runtime* R, const char* name, const char* enc, size_t elem, void** out, const TensorEntry** te) {
  const TensorEntry* t = M->man.find(name);
  if (!t || t->enc != enc) {
    set_error("bundle has no %s tensor %s", enc, name);
    return kErrFormat;
  }
  if (static_cast<size_t>(t->nbytes) != static_cast<size_t>(t->N) * t->K * elem) {
    set_error("tensor %s: %lld bytes do not match its shape", name, t->nbytes);
    return kErrFormat;
  }
  std::vector<uint8_t> host;
  int rc = read_blob(M->fd, *t, host);
  if (rc) return rc;
  uint8_t* d = nullptr;
  if ((rc = dalloc(R, &d, static_cast<size_t>(t->nbytes)))) return rc;
  const cudaError_t e = cudaMemcpy(d, host.data(), t->nbytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return cuda_fail("cudaMemcpy (runtime tensor)", e);
  *out = d;
  if (te) *te = t;
  return kOk;
}

static int find_matrix(Model* M, const std::string& n) {
  auto it = M->by_name.find(n);
  return it == M->by_name.end() ? -1 : it->second;
}

int runtime_init(Model* M, int max_ctx, int max_batch) {
  if (const int rc = validate_model(M->man)) return rc;   // shapes of everything the passes index
  auto R = new Runtime();
  M->rt = R;
  R->L = cfg_int(M, "n_layers", 0);
  R->D = cfg_int(M, "hidden", 0);
  R->H = cfg_int(M, "n_heads", 0);
  R->Hk = cfg_int(M, "n_kv_heads", R->H);
  R->Dh = cfg_int(M, "head_dim", R->H ? R->D / R->H : 0);
  R->I = cfg_int(M, "inter", 0);
  R->V = cfg_int(M, "vocab", 0);
  R->eps = static_cast<float>(cfg_f(M, "eps", 1e-5));
  R->attn_scale = static_cast<float>(cfg_f(M, "attn_scale", R->Dh ? 1.0 / std::sqrt(static_cast<double>(R->Dh)) : 1.0));
  const int rope_rows = cfg_int(M, "rope_rows", 4096);
  R->Tmax = std::max(1, std::min(max_ctx > 0 ? max_ctx : rope_rows, rope_rows));
  R->max_batch = std::max(1, max_batch);
  R->max_chunks = (R->Tmax + kAttnChunk - 1) / kAttnChunk;
  R->tp_world = std::max(1, cfg_int(M, "tp_world", 1));
  R->tp_rank = cfg_int(M, "tp_rank", 0);
  // Vocabulary shards: tile rows (64 vocabulary rows) dealt as evenly as possible, the first (tile rows % world)
  // ranks hold one more (32000 rows on 8 ranks: 63 tile rows on ranks 0..3, 62 on ranks 4..7).
  R->Vfull = cfg_int(M, "vocab_full", R->V * R->tp_world);
  {
    const int units = R->Vfull / kTileRows, base = units / R->tp_world, rem = units % R->tp_world;
    for (int r = 0; r < R->tp_world; ++r) {
      R->voff.push_back((r * base + std::min(r, rem)) * kTileRows);
      R->vcnt.push_back((base + (r < rem ? 1 : 0)) * kTileRows);
      R->Vmax = std::max(R->Vmax, R->vcnt.back());
    }
    if (R->Vfull % kTileRows || R->tp_rank < 0 || R->tp_rank >= R->tp_world || R->vcnt[R->tp_rank] != R->V) {
      set_error("bundle cfg: vocab %d is not rank %d's share of vocab_full %d over %d ranks", R->V, R->tp_rank, R->Vfull,
                R->tp_world);
      return kErrFormat;
    }
  }
  {
    auto it = M->man.cfg.find("eos");
    std::stringstream es(it == M->man.cfg.end() ? "" : it->second);
    std::string x;
    while (std::getline(es, x, ',')) R->eos.push_back(atoi(x.c_str()));
  }
  if (R->L <= 0 || R->D <= 0 || R->H <= 0 || R->Hk <= 0 || R->Dh <= 0 || R->I <= 0 || R->V <= 0 || R->H % R->Hk ||
      R->Dh % 8 || R->Dh > kAttnMaxDh) {
    set_error("bundle cfg: bad model shape (head_dim must be a multiple of 8, at most %d)", kAttnMaxDh);
    return kErrFormat;
  }
  int rc;
  const size_t B = R->max_batch, QKV = static_cast<size_t>(R->H + 2 * R->Hk) * R->Dh;
  if ((rc = dalloc(R, &R->h, B * R->D)) || (rc = dalloc(R, &R->xn, B * R->D)) ||
      (rc = dalloc(R, &R->att, B * R->H * R->Dh)) || (rc = dalloc(R, &R->o, B * R->D)) ||
      (rc = dalloc(R, &R->qkv, B * QKV)) || (rc = dalloc(R, &R->g, B * R->I)) || (rc = dalloc(R, &R->u, B * R->I)) ||
      (rc = dalloc(R, &R->logits, B * R->Vmax)) || (rc = dalloc(R, &R->logits_all, B * R->Vmax * R->tp_world)) ||
      (rc = dalloc(R, &R->ids, B + 2)) || (rc = dalloc(R, &R->gen, static_cast<size_t>(R->Tmax))) ||
      (rc = dalloc(R, &R->attn_part, B * R->H * ((R->Tmax + kAttnChunk - 1) / kAttnChunk) * (R->Dh + 2))) ||
      (rc = dalloc(R, &R->attn_done, B * R->H)) ||
      (rc = dalloc(R, &R->kc, static_cast<size_t>(R->L) * R->Hk * R->Tmax * R->Dh)) ||
      (rc = dalloc(R, &R->vc, static_cast<size_t>(R->L) * R->Hk * R->Tmax * R->Dh)))
    return rc;
  if (cudaMemset(R->attn_done, 0, B * R->H * sizeof(unsigned int)) != cudaSuccess)
    return cuda_fail("cudaMemset (attention counters)", cudaGetLastError());
  if (cudaMallocHost(reinterpret_cast<void**>(&R->h_ids), (B + 2 + static_cast<size_t>(R->Tmax)) * sizeof(int)) != cudaSuccess)
    return cuda_fail("cudaMallocHost (ids)", cudaGetLastError());
  if (cudaStreamCreateWithFlags(&R->stream, cudaStreamNonBlocking) != cudaSuccess)
    return cuda_fail("cudaStreamCreate", cudaGetLastError());
  if (const char* e = getenv("LW_GRAPHS")) R->graphs = atoi(e) != 0;
  const TensorEntry* te = nullptr;
  void* p = nullptr;
  if (M->man.find("embed") && M->man.find("embed")->enc == "f16") {
    if ((rc = upload(M, R, "embed", "f16", 2, &p, &te))) return rc;
    R->embed16 = static_cast<__half*>(p);
  } else {
    if ((rc = upload(M, R, "embed", "raw8", 1, &p, &te))) return rc;
    R->embed8 = static_cast<uint8_t*>(p);
    const TensorEntry* ts = nullptr;
    if ((rc = upload(M, R, "embed.rs", "f32", 4, &p, &ts))) return rc;
    R->embed_rs = static_cast<float*>(p);
    R->embed_groups = ts->K;
    if ((rc = upload(M, R, "embed.rsub", "f32", 4, &p, nullptr))) return rc;
    R->embed_rsub = static_cast<float*>(p);
  }
  if (te->K != R->D) {
    set_error("embed has %d columns, hidden is %d", te->K, R->D);
    return kErrFormat;
  }
  R->embed_rows = te->N;
  if ((rc = upload(M, R, "cos", "f32", 4, &p, &te))) return rc;
  R->cosv = static_cast<float*>(p);
  if (te->K != R->Dh / 2 || te->N < R->Tmax) {
    set_error("rotary table has the wrong shape");
    return kErrFormat;
  }
  if ((rc = upload(M, R, "sin", "f32", 4, &p, nullptr))) return rc;
  R->sinv = static_cast<float*>(p);
  if ((rc = upload(M, R, "lnf", "f32", 4, &p, nullptr))) return rc;
  R->lnf = static_cast<float*>(p);
  for (int l = 0; l < R->L; ++l) {
    const std::string pre = "l" + std::to_string(l) + ".";
    if ((rc = upload(M, R, (pre + "ln1").c_str(), "f32", 4, &p, nullptr))) return rc;
    R->ln1.push_back(static_cast<float*>(p));
    if ((rc = upload(M, R, (pre + "ln2").c_str(), "f32", 4, &p, nullptr))) return rc;
    R->ln2.push_back(static_cast<float*>(p));
    R->m_qkv.push_back(find_matrix(M, pre + "qkv"));
    R->m_q.push_back(find_matrix(M, pre + "q"));
    R->m_k.push_back(find_matrix(M, pre + "k"));
    R->m_v.push_back(find_matrix(M, pre + "v"));
    R->m_o.push_back(find_matrix(M, pre + "o"));
    R->m_gate.push_back(find_matrix(M, pre + "gate"));
    R->m_up.push_back(find_matrix(M, pre + "up"));
    R->m_down.push_back(find_matrix(M, pre + "down"));
    const bool attn_ok = R->m_qkv[l] >= 0 || (R->m_q[l] >= 0 && R->m_k[l] >= 0 && R->m_v[l] >= 0);
    if (!attn_ok || R->m_o[l] < 0 || R->m_gate[l] < 0 || R->m_up[l] < 0 || R->m_down[l] < 0) {
      set_error("layer %d: a coded matrix is missing", l);
      return kErrFormat;
    }
  }
  R->m_head = find_matrix(M, "lm_head");
  if (R->m_head < 0) {
    set_error("bundle has no lm_head");
    return kErrFormat;
  }
  return kOk;
}

void runtime_free(Model* M) {
  Runtime* R = M->rt;
  if (!R) return;
  if (R->stream) cudaStreamSynchronize(R->stream);
  for (auto& kv : R->graph_exec) cudaGraphExecDestroy(kv.second);
  if (R->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(R->comm);
  if (R->stream) cudaStreamDestroy(R->stream);
  for (int p = 0; p < kPeerMaxRanks; ++p)
    if (R->peer_base[p] && R->peer_base[p] != R->peer_local) cudaIpcCloseMemHandle(R->peer_base[p]);
  if (R->peer_local) cudaFree(R->peer_local);
  if (R->h_ids) cudaFreeHost(R->h_ids);
  for (void* p : R->owned) cudaFree(p);
  delete R;
  M->rt = nullptr;
}

double runtime_stat(const Model* M, const char* key) {
  if (!M->rt) return 0;
  if (std::strcmp(key, "graph_launches") == 0) return static_cast<double>(M->rt->graph_launches);
  if (std::strcmp(key, "graph_captures") == 0) return static_cast<double>(M->rt->graph_captures);
  if (std::strcmp(key, "collective_us") == 0) return M->rt->collective_us;
  if (std::strcmp(key, "collective_calls") == 0) return static_cast<double>(M->rt->collective_calls);
  if (std::strcmp(key, "time_collectives") == 0) {   // arms the measurement for the next pass
    M->rt->time_collectives = true;
    return 0;
  }
  return -1;
}

// Brackets a collective with events when the pass is being timed (see rt_stat "collective_us").
struct CollTimer {
  Runtime* R;
  cudaStream_t st;
  CollTimer(Runtime* r, cudaStream_t s) : R(r), st(s) { mark(); }
  ~CollTimer() { mark(); }
  void mark() {
    if (!R->time_collectives) return;
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    cudaEventRecord(e, st);
    R->coll_events.push_back(e);
  }
};

static int nccl_check(int r, const char* what) {
  if (r == 0) return kOk;
  set_error("%s: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "NCCL error");
  return kErrCuda;
}

// The device work of one pass over m <= max_batch tokens (ids and position already in R->h_ids): everything is
// enqueued on `st`, nothing here depends on host-side values that change from pass to pass except `nchunks`.
static PeerView peer_view(const Runtime* R) {
  PeerView P;
  for (int p = 0; p < kPeerMaxRanks; ++p) {
    uint8_t* base = static_cast<uint8_t*>(p < R->tp_world ? R->peer_base[p] : nullptr);
    P.flags[p] = base ? reinterpret_cast<uint32_t*>(base + kPeerMaxBlocks * 4) : nullptr;
    P.slots[p] = base ? reinterpret_cast<float*>(base + 4096) : nullptr;
  }
  P.epoch = static_cast<uint32_t*>(R->peer_local);
  P.world = R->tp_world;
  P.rank = R->tp_rank;
  P.D = R->D;
  return P;
}

// h += (sum over ranks of) `res`, out = rmsnorm(h) * g: the norm kernel; with tensor parallelism the ranks' partial
// `res` are summed first - over peer memory inside the same kernel, or by an NCCL all-reduce in front of it.
static int norm_residual(Model* M, Runtime* R, int m, const float* res, bool res_is_partial, const float* g, cudaStream_t st,
                         const char* what) {
  (void)M;
  if (res && res_is_partial && R->tp_world > 1) {
    if (R->peer_ready && m <= kPeerMaxBlocks && R->D % 4 == 0) {
      CollTimer t(R, st);
      unsigned int* err = nullptr;
      if (cudaGetSymbolAddress(reinterpret_cast<void**>(&err), g_rt_error) != cudaSuccess) return cuda_fail("error word", cudaGetLastError());
      launch_dep(k_allreduce_rmsnorm, dim3(m), dim3(kNormThreads), st, peer_view(R), res, R->h, g, R->xn, R->eps, err,
                 uint32_t(1) << 22);
      return kOk;
    }
    if (!R->comm) {
      set_error("tensor-parallel bundle without a communicator: call rt_tp_init");
      return kErrArg;
    }
    CollTimer t(R, st);
    const int rc = nccl_check(g_nccl.AllReduce(res, const_cast<float*>(res), static_cast<size_t>(m) * R->D, kNcclFloat, kNcclSum,
                                               R->comm, st), what);
    if (rc) return rc;
  }
  launch_dep(k_rmsnorm, dim3(m), dim3(kNormThreads), st, R->h, res, g, R->xn, R->D, R->eps);
  return kOk;
}

// greedy: the token and the position are already on the device (written by the previous pass's k_argmax_next), and
// the pass ends with that kernel.
static int enqueue_pass(Model* M, Runtime* R, int m, bool all_logits, int nchunks, cudaStream_t st, bool greedy = false) {
  cudaError_t e = cudaSuccess;
  if (!greedy) e = cudaMemcpyAsync(R->ids, R->h_ids, (R->max_batch + 1) * sizeof(int), cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) return cuda_fail("ids upload", e);
  const int* posp = R->ids + R->max_batch;
  if (R->embed16) k_embed16<<<m, 256, 0, st>>>(R->ids, R->embed16, R->h, R->D);
  else k_embed8<<<m, 256, 0, st>>>(R->ids, R->embed8, R->embed_rs, R->embed_rsub, R->h, R->D, R->embed_groups);
  const size_t QKV = static_cast<size_t>(R->H + 2 * R->Hk) * R->Dh;
  const float* pending = nullptr;   // output of the previous block, added to h by the next norm
  int rc = kOk;
  for (int l = 0; l < R->L; ++l) {
    if ((rc = norm_residual(M, R, m, pending, true, R->ln1[l], st, "all-reduce (down)"))) return rc;
    if (R->m_qkv[l] >= 0) {
      if ((rc = linear_device(M, M->mats[R->m_qkv[l]], R->xn, false, m, R->qkv, static_cast<int>(QKV), st))) return rc;
    } else if (m == 1) {   // one token: q, k and v read the same activations - one launch where their plans agree
      const int idx[3] = {R->m_q[l], R->m_k[l], R->m_v[l]};
      const float* xs[3] = {R->xn, R->xn, R->xn};
      float* ys[3] = {R->qkv, R->qkv + R->H * R->Dh, R->qkv + (R->H + R->Hk) * R->Dh};
      if ((rc = linear_batch_device(M, 3, idx, xs, ys, st))) return rc;
    } else {
      if ((rc = linear_device(M, M->mats[R->m_q[l]], R->xn, false, m, R->qkv, static_cast<int>(QKV), st)) ||
          (rc = linear_device(M, M->mats[R->m_k[l]], R->xn, false, m, R->qkv + R->H * R->Dh, static_cast<int>(QKV), st)) ||
          (rc = linear_device(M, M->mats[R->m_v[l]], R->xn, false, m, R->qkv + (R->H + R->Hk) * R->Dh,
                              static_cast<int>(QKV), st)))
        return rc;
    }
    __half* kc = R->kc + static_cast<size_t>(l) * R->Hk * R->Tmax * R->Dh;
    __half* vc = R->vc + static_cast<size_t>(l) * R->Hk * R->Tmax * R->Dh;
    launch_dep(k_rope_cache, dim3(R->H + 2 * R->Hk, m), dim3(64), st, R->qkv, R->cosv, R->sinv, kc, vc, posp, R->H, R->Hk, R->Dh,
                                                          R->Tmax);
    {
      const int group = R->H / R->Hk;
      if (group % 4 == 0)
        launch_dep(k_attn<4>, dim3(R->H / 4, m, nchunks), dim3(kAttnThreads), st, R->qkv, kc, vc, R->attn_part, R->att, R->attn_done,
                   posp, R->H, R->Hk, R->Dh, R->Tmax, R->attn_scale, R->window, R->max_chunks);
      else if (group % 2 == 0)
        launch_dep(k_attn<2>, dim3(R->H / 2, m, nchunks), dim3(kAttnThreads), st, R->qkv, kc, vc, R->attn_part, R->att, R->attn_done,
                   posp, R->H, R->Hk, R->Dh, R->Tmax, R->attn_scale, R->window, R->max_chunks);
      else
        launch_dep(k_attn<1>, dim3(R->H, m, nchunks), dim3(kAttnThreads), st, R->qkv, kc, vc, R->attn_part, R->att, R->attn_done,
                   posp, R->H, R->Hk, R->Dh, R->Tmax, R->attn_scale, R->window, R->max_chunks);
    }
    if ((rc = linear_device(M, M->mats[R->m_o[l]], R->att, false, m, R->o, R->D, st))) return rc;
    if ((rc = norm_residual(M, R, m, R->o, true, R->ln2[l], st, "all-reduce (o)"))) return rc;
    if (m == 1) {          // one token: gate and up in one launch
      const int idx[2] = {R->m_gate[l], R->m_up[l]};
      const float* xs[2] = {R->xn, R->xn};
      float* ys[2] = {R->g, R->u};
      if ((rc = linear_batch_device(M, 2, idx, xs, ys, st))) return rc;
    } else if ((rc = linear_device(M, M->mats[R->m_gate[l]], R->xn, false, m, R->g, R->I, st)) ||
               (rc = linear_device(M, M->mats[R->m_up[l]], R->xn, false, m, R->u, R->I, st))) {
      return rc;
    }
    const size_t ng = static_cast<size_t>(m) * R->I;
    launch_dep(k_silu_mul, dim3(static_cast<unsigned>((ng + 255) / 256)), dim3(256), st, R->g, R->u, ng);
    if ((rc = linear_device(M, M->mats[R->m_down[l]], R->g, false, m, R->o, R->D, st))) return rc;
    pending = R->o;   // the ranks' partial outputs of `down`: summed by the next norm
  }
  if ((rc = norm_residual(M, R, m, pending, true, R->lnf, st, "all-reduce (down)"))) return rc;
  const int rows = all_logits ? m : 1;
  const float* xlast = all_logits ? R->xn : R->xn + static_cast<size_t>(m - 1) * R->D;
  if ((rc = linear_device(M, M->mats[R->m_head], xlast, false, rows, R->logits, R->V, st))) return rc;
  if (R->comm) {
    // ranks hold consecutive slices of the vocabulary (of 63 or 62 tile rows, say): every rank contributes
    // rows x Vmax floats of which its first rows x V count; gathered rank-major, reordered by the caller
    CollTimer t(R, st);
    if ((rc = nccl_check(g_nccl.AllGather(R->logits, R->logits_all, static_cast<size_t>(rows) * R->Vmax, kNcclFloat,
                                          R->comm, st), "all-gather (logits)")))
      return rc;
  }
  if (greedy) {
    const int units = R->Vfull / kTileRows;
    launch_dep(k_argmax_next, dim3(1), dim3(1024), st, R->comm ? R->logits_all : R->logits, R->tp_world, R->Vmax,
               units / R->tp_world, units % R->tp_world, R->ids, R->max_batch, R->gen);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("forward", e);
  return kOk;
}

// One pass: direct launches the first time a shape (tokens, context bucket, all_logits) occurs, captured into a CUDA
// graph the second time, replayed afterwards (the reference's policy, kernels/llmrt.cu:2294-2341).  The decode + GEMM
// path (more than eight rows) may allocate scratch, so those passes are never captured.
// Waits for the runtime's stream like cudaStreamSynchronize, but with tensor parallelism it gives up: a collective
// whose peer never arrives would otherwise block the host for ever.  While it waits it asks NCCL for asynchronous
// errors; after `timeout_ms` (LW_TP_TIMEOUT_MS, default 60 s) or on such an error it aborts the communicator (the NCCL
// kernels then leave the GPU; this file's own peer kernel has bounded waits and leaves by itself) and reports
// kErrCuda.  The handle is unusable for further tensor-parallel passes after that.
static int guarded_wait(Runtime* R, const char* what) {
  if (R->tp_world <= 1) {
    const cudaError_t e = cudaStreamSynchronize(R->stream);
    return e == cudaSuccess ? kOk : cuda_fail(what, e);
  }
  static const int timeout_ms = [] {
    const char* e = getenv("LW_TP_TIMEOUT_MS");
    return e ? std::max(1, atoi(e)) : 60000;
  }();
  const int limit = R->wait_timeout_ms > 0 ? R->wait_timeout_ms : timeout_ms;
  const auto t0 = std::chrono::steady_clock::now();
  for (unsigned spin = 0;; ++spin) {
    const cudaError_t q = cudaStreamQuery(R->stream);
    if (q == cudaSuccess) return kOk;
    if (q != cudaErrorNotReady) return cuda_fail(what, q);
    int async = 0;
    const bool nccl_failed = R->comm && g_nccl.CommGetAsyncError && (spin & 255u) == 255u &&
                             g_nccl.CommGetAsyncError(R->comm, &async) == 0 && async != 0;
    const long long waited =
        std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (nccl_failed || waited > limit) {
      if (R->comm && g_nccl.CommAbort) {
        g_nccl.CommAbort(R->comm);
        R->comm = nullptr;
      }
      R->tp_failed = true;
      if (nccl_failed)
        set_error("%s: NCCL reports an asynchronous error (%s)", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(async) : "?");
      else
        set_error("%s: the pass did not finish within %d ms - a rank is missing", what, limit);
      return kErrCuda;
    }
    if (waited > 2 && (spin & 15u) == 15u) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

// greedy (one token, ids_host null): a pass of rt_decode_greedy - token and position are on the device already, the
// pass ends with the arg-max that prepares the next one, and the host does not wait between passes.
static int forward_chunk(Model* M, Runtime* R, const int* ids_host, int m, bool all_logits, bool greedy = false) {
  cudaStream_t st = R->stream;
  if (!greedy) {
    cudaStreamSynchronize(st);   // the pinned id buffer is reused
    std::memcpy(R->h_ids, ids_host, m * sizeof(int));
    R->h_ids[R->max_batch] = R->pos;
  }
  const int span = R->window > 0 ? std::min(R->window, R->pos + m) : R->pos + m;
  const int nchunks = (span + kAttnChunk - 1) / kAttnChunk;
  const long long key = (static_cast<long long>(nchunks) << 8) | (m << 1) | (all_logits ? 1 : 0) | (greedy ? 1LL << 62 : 0);
  int rc = kOk;
  auto it = R->graph_exec.find(key);
  if (R->time_collectives && !greedy) {
    // one pass launched directly, with events around every collective; the time between each pair is added up
    rc = enqueue_pass(M, R, m, all_logits, nchunks, st);
    cudaStreamSynchronize(st);
    R->collective_us = 0.0;
    R->collective_calls = static_cast<int>(R->coll_events.size() / 2);
    for (size_t i = 0; i + 1 < R->coll_events.size(); i += 2) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, R->coll_events[i], R->coll_events[i + 1]) == cudaSuccess) R->collective_us += ms * 1e3;
    }
    for (cudaEvent_t e : R->coll_events) cudaEventDestroy(e);
    R->coll_events.clear();
    R->time_collectives = false;
  } else if (it != R->graph_exec.end()) {
    const cudaError_t e = cudaGraphLaunch(it->second, st);
    if (e != cudaSuccess) return cuda_fail("cudaGraphLaunch", e);
    ++R->graph_launches;
  } else if (R->graphs && m <= 8 && ++R->graph_seen[key] >= 2) {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed);
    if (e != cudaSuccess) return cuda_fail("cudaStreamBeginCapture", e);
    rc = enqueue_pass(M, R, m, all_logits, nchunks, st, greedy);
    e = cudaStreamEndCapture(st, &graph);
    if (rc == kOk && e == cudaSuccess && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
      R->graph_exec[key] = exec;
      ++R->graph_captures;
      e = cudaGraphLaunch(exec, st);
      if (e != cudaSuccess) rc = cuda_fail("cudaGraphLaunch", e);
      ++R->graph_launches;
    } else {
      // capture is not possible here (for instance a collective that cannot be captured): run directly from now on
      cudaGetLastError();
      R->graphs = false;
      rc = enqueue_pass(M, R, m, all_logits, nchunks, st, greedy);
    }
    if (graph) cudaGraphDestroy(graph);
  } else {
    rc = enqueue_pass(M, R, m, all_logits, nchunks, st, greedy);
  }
  if (rc) return rc;
  R->pos += m;
  return kOk;
}

}  // namespace lw

using namespace lw;

extern "C" {

int rt_forward(void* handle, const int* ids, int n, float* logits, int all_logits) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !M->rt || !ids || n < 1) {
    set_error("rt_forward: no model runtime in this handle, or bad argument");
    return kErrArg;
  }
  Runtime* R = M->rt;
  if (const int rc = check_device(M)) return rc;
  if (R->tp_failed) {
    set_error("rt_forward: an earlier tensor-parallel pass gave up waiting for a rank; open the shards again");
    return kErrCuda;
  }
  for (int i = 0; i < n; ++i)
    if (ids[i] < 0 || ids[i] >= R->embed_rows) {   // the embedding gather indexes device memory with it
      set_error("rt_forward: token id %d at position %d is outside the embedding's %d rows", ids[i], i, R->embed_rows);
      return kErrArg;
    }
  if (R->pos + n > R->Tmax) return -1;   // context overflow (the reference's -1, kernels/llmrt.cu:2293)
  const int W = R->tp_world, Vfull = R->Vfull;
  std::vector<float> stage;
  for (int i0 = 0; i0 < n; i0 += R->max_batch) {
    const int m = std::min(R->max_batch, n - i0);
    const bool last = i0 + m == n;
    const int rc = forward_chunk(M, R, ids + i0, m, all_logits != 0);
    if (rc) return rc;
    if (!logits || (!all_logits && !last)) continue;
    const int rows = all_logits ? m : 1;
    float* dst = all_logits ? logits + static_cast<size_t>(i0) * Vfull : logits;
    cudaError_t e;
    if (W == 1) {
      e = cudaMemcpyAsync(dst, R->logits, static_cast<size_t>(rows) * R->V * 4, cudaMemcpyDeviceToHost, R->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(R->stream);
    } else {
      stage.resize(static_cast<size_t>(W) * rows * R->Vmax);
      e = cudaMemcpyAsync(stage.data(), R->logits_all, stage.size() * 4, cudaMemcpyDeviceToHost, R->stream);
      if (e == cudaSuccess)
        if (const int rcw = guarded_wait(R, "rt_forward")) return rcw;
      for (int r = 0; r < W && e == cudaSuccess; ++r)
        for (int j = 0; j < rows; ++j)
          std::memcpy(dst + static_cast<size_t>(j) * Vfull + R->voff[r],
                      stage.data() + static_cast<size_t>(r) * rows * R->Vmax + static_cast<size_t>(j) * R->vcnt[r],
                      static_cast<size_t>(R->vcnt[r]) * 4);
    }
    if (e != cudaSuccess) return cuda_fail("logits copy", e);
  }
  if (!logits)
    if (const int rcw = guarded_wait(R, "rt_forward")) return rcw;
  return 0;
}

int rt_decode_greedy(void* handle, int first_token, int n, int* out) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !M->rt || n < 1 || !out) {
    set_error("rt_decode_greedy: no model runtime in this handle, or bad argument");
    return kErrArg;
  }
  Runtime* R = M->rt;
  if (const int rc = check_device(M)) return rc;
  if (R->tp_failed) {
    set_error("rt_decode_greedy: an earlier tensor-parallel pass gave up waiting for a rank; open the shards again");
    return kErrCuda;
  }
  if (first_token < 0 || first_token >= R->embed_rows) {
    set_error("rt_decode_greedy: token id %d is outside the embedding's %d rows", first_token, R->embed_rows);
    return kErrArg;
  }
  if (R->pos + n > R->Tmax) return -1;
  cudaStream_t st = R->stream;
  cudaStreamSynchronize(st);
  const int B = R->max_batch;
  R->h_ids[0] = first_token;
  R->h_ids[B] = R->pos;
  R->h_ids[B + 1] = 0;
  cudaError_t e = cudaMemcpyAsync(R->ids, R->h_ids, (B + 2) * sizeof(int), cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) return cuda_fail("ids upload", e);
  for (int i = 0; i < n; ++i)
    if (const int rc = forward_chunk(M, R, nullptr, 1, false, true)) return rc;
  int* h_gen = R->h_ids + B + 2;
  e = cudaMemcpyAsync(h_gen, R->gen, static_cast<size_t>(n) * sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return cuda_fail("rt_decode_greedy", e);
  if (const int rcw = guarded_wait(R, "rt_decode_greedy")) return rcw;
  std::memcpy(out, h_gen, static_cast<size_t>(n) * sizeof(int));
  return 0;
}

int rt_tp_set_timeout(void* handle, int timeout_ms) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !M->rt || timeout_ms < 0) return kErrArg;
  M->rt->wait_timeout_ms = timeout_ms;
  return 0;
}

// Test hook: the runtime's stream is held up by a host function that sleeps `ms` milliseconds (the GPU is idle
// meanwhile), then the guarded wait of a tensor-parallel handle is called: 0 if the stream drained in time, else the
// status of the give-up path.  For handles without tensor parallelism it only waits.
int lw_debug_stream_stall(void* handle, int ms) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !M->rt || ms < 0 || ms > 5000) return kErrArg;
  Runtime* R = M->rt;
  int* arg = new int(ms);
  const cudaError_t e = cudaLaunchHostFunc(R->stream, [](void* p) {
    int* q = static_cast<int*>(p);
    std::this_thread::sleep_for(std::chrono::milliseconds(*q));
    delete q;
  }, arg);
  if (e != cudaSuccess) {
    delete arg;
    return cuda_fail("cudaLaunchHostFunc", e);
  }
  const int saved_world = R->tp_world;
  if (saved_world <= 1) R->tp_world = 2;   // exercise the bounded wait on a plain handle too
  const int rc = guarded_wait(R, "lw_debug_stream_stall");
  R->tp_world = saved_world;
  const bool failed = R->tp_failed;
  if (saved_world <= 1) R->tp_failed = false;   // nothing was lost on a handle without peers
  cudaStreamSynchronize(R->stream);
  return rc ? rc : (failed ? kErrCuda : 0);
}

void rt_reset(void* handle) {
  Model* M = static_cast<Model*>(handle);
  if (M && M->rt) M->rt->pos = 0;
}
void rt_set_window(void* handle, int w) {
  Model* M = static_cast<Model*>(handle);
  if (M && M->rt && M->rt->window != std::max(0, w)) {
    Runtime* R = M->rt;
    cudaStreamSynchronize(R->stream);
    for (auto& kv : R->graph_exec) cudaGraphExecDestroy(kv.second);   // the window is baked into captured passes
    R->graph_exec.clear();
    R->graph_seen.clear();
    R->window = std::max(0, w);
  }
}
void rt_set_pos(void* handle, int p) {
  Model* M = static_cast<Model*>(handle);
  if (M && M->rt) M->rt->pos = std::max(0, std::min(p, M->rt->pos));
}
int rt_pos(void* handle) {
  Model* M = static_cast<Model*>(handle);
  return M && M->rt ? M->rt->pos : -1;
}
int rt_vocab(void* handle) {
  Model* M = static_cast<Model*>(handle);
  return M && M->rt ? M->rt->Vfull : -1;
}

int lw_tp_unique_id(uint8_t* out128) {
  if (!out128 || !g_nccl.load()) {
    set_error("NCCL is not available in this process");
    return kErrGeneric;
  }
  UniqueId id;
  std::memset(&id, 0, sizeof id);
  const int rc = nccl_check(g_nccl.GetUniqueId(&id), "ncclGetUniqueId");
  if (rc) return rc;
  std::memcpy(out128, id.bytes, 128);
  return kOk;
}

int rt_tp_init(void* handle, int rank, int world, const uint8_t* id128) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !M->rt || !id128 || world < 1 || rank < 0 || rank >= world) {
    set_error("rt_tp_init: bad argument");
    return kErrArg;
  }
  Runtime* R = M->rt;
  if (world != R->tp_world) {
    set_error("bundle was sharded for %d ranks, not %d", R->tp_world, world);
    return kErrArg;
  }
  if (world == 1) return kOk;
  if (!g_nccl.load()) {
    set_error("NCCL is not available in this process");
    return kErrGeneric;
  }
  UniqueId id;
  std::memcpy(id.bytes, id128, 128);
  auto init = reinterpret_cast<int (*)(void**, int, UniqueId, int)>(g_nccl.init_rank_sym);
  const int rc = nccl_check(init(&R->comm, world, id, rank), "ncclCommInitRank");
  if (rc) return rc;
  R->tp_rank = rank;
  return kOk;
}

int rt_tp_peer_export(void* handle, uint8_t* out64) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !M->rt || !out64) return kErrArg;
  Runtime* R = M->rt;
  if (const int rc = check_device(M)) return rc;
  if (R->tp_world < 2 || R->tp_world > kPeerMaxRanks || R->max_batch < 1) {
    set_error("rt_tp_peer_export: needs a shard of 2..8 ranks");
    return kErrArg;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  if (!R->peer_local) {
    R->peer_bytes = 4096 + peer_slot_floats(R->D) * sizeof(float);
    cudaError_t e = cudaMalloc(&R->peer_local, R->peer_bytes);
    if (e != cudaSuccess) return cuda_fail("cudaMalloc (exchange buffer)", e);
    if ((e = cudaMemset(R->peer_local, 0, R->peer_bytes)) != cudaSuccess) return cuda_fail("cudaMemset (exchange buffer)", e);
  }
  cudaIpcMemHandle_t hnd;
  const cudaError_t e = cudaIpcGetMemHandle(&hnd, R->peer_local);
  if (e != cudaSuccess) return cuda_fail("cudaIpcGetMemHandle", e);
  std::memcpy(out64, &hnd, 64);
  return kOk;
}

int rt_tp_peer_open(void* handle, const uint8_t* handles, int world) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !M->rt || !handles) return kErrArg;
  Runtime* R = M->rt;
  if (const int rc = check_device(M)) return rc;
  if (world != R->tp_world || !R->peer_local) {
    set_error("rt_tp_peer_open: call rt_tp_peer_export first; world must match the shard");
    return kErrArg;
  }
  for (int p = 0; p < world; ++p) {
    if (p == R->tp_rank) {
      R->peer_base[p] = R->peer_local;
      continue;
    }
    cudaIpcMemHandle_t hnd;
    std::memcpy(&hnd, handles + 64 * p, 64);
    const cudaError_t e = cudaIpcOpenMemHandle(&R->peer_base[p], hnd, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      R->peer_base[p] = nullptr;
      return cuda_fail("cudaIpcOpenMemHandle", e);
    }
  }
  cudaDeviceSynchronize();
  // captured passes hold the NCCL form of the all-reduce: drop them
  for (auto& kv : R->graph_exec) cudaGraphExecDestroy(kv.second);
  R->graph_exec.clear();
  R->graph_seen.clear();
  R->peer_ready = true;
  return kOk;
}

int rt_tp_error(void* handle) {
  Model* M = static_cast<Model*>(handle);
  if (!M || !M->rt) return kErrArg;
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_rt_error, sizeof v) != cudaSuccess) return cuda_fail("read error word", cudaGetLastError());
  if (v) {
    const unsigned int z = 0;
    cudaMemcpyToSymbol(g_rt_error, &z, sizeof z);
  }
  return static_cast<int>(v);
}

}  // extern "C"
