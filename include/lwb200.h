/* C ABI of liblwb200: Huffman-coded llama.cpp block weights decoded on the GPU (sm_100a), fused with block
 * dequantisation and the matrix-vector / small-M matrix product.
 *
 * The rt_* entry points keep the names, argument meaning and return conventions of the reference runtime's
 * `extern "C"` block (kernels/llmrt.cu:1916-2575) for the per-matrix path, so that a ctypes caller such as
 * scripts/a2_act8_ppl.py:56-77 binds them unchanged.  The lw_* entry points are additions: device-pointer
 * variants for callers that already hold activations on the GPU, the host-side codec, and error reporting.
 *
 * Conventions: plain pointers and sizes only; a handle is an opaque pointer owned by the library and released by
 * rt_close; the library owns all device memory it allocates; callers own every buffer they
 * pass.  One handle is driven by one host thread at a time.  Where the reference prints and exits on a CUDA error
 * or a malformed bundle, these functions return a negative status (or NULL) and leave a message for
 * lw_last_error().  Without a CUDA device every function that needs one fails with LW_ERR_NO_DEVICE: there is no
 * CPU fallback for the GPU path.
 */
#ifndef LWB200_H
#define LWB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  LW_OK = 0,
  LW_ERR = -1,           /* not found / not resident (the reference's -1) */
  LW_ERR_ARG = -2,
  LW_ERR_FORMAT = -3,    /* malformed bundle or blob, rejected on the host before anything is launched */
  LW_ERR_CUDA = -4,
  LW_ERR_TOO_LARGE = -5,
  LW_ERR_NO_DEVICE = -6
};

/* Block formats (side-tensor encodings kq_Q4_K, kq_Q5_K, kq_Q6_K, kq_IQ4_XS; kernels/llmrt.cu:113-121). */
enum { LW_FMT_NONE = 0, LW_FMT_Q4_K = 1, LW_FMT_Q5_K = 2, LW_FMT_Q6_K = 3, LW_FMT_IQ4_XS = 4 };

/* ---- bundle handle ------------------------------------------------------------------------------------- */

/* Opens a bundle directory (manifest.txt + weights.bin, lazyweights/bundle.py:10-21) on the current CUDA device:
 * validates every coded matrix on the host, re-lays it out and uploads it with its `.kqs` side tensor.
 * Replaces rt_open, kernels/llmrt.cu:1921.  budget_mb and floor_mb are accepted for signature compatibility;
 * every matrix is made resident (no streaming on a 180 GB device).  Returns NULL on failure. */
void* rt_open(const char* dir, int max_ctx, int max_batch, long long budget_mb, int floor_mb, int verbose);

/* Frees the handle and all device memory it owns.  Replaces rt_close, kernels/llmrt.cu:2239. */
void rt_close(void* handle);

/* Y[m, N] = X[m, K] . dequant(W)^T with host fp32 buffers; path 0 auto, 1 fused decode+product per chunk of up to
 * eight rows, 2 decode to fp16 weights then GEMM (the reference's paths), 3 (addition) the decode + tcgen05 GEMM for
 * up to 64 rows.  Returns -1 if the matrix is unknown.
 * Replaces rt_test_matmul, kernels/llmrt.cu:2441. */
int rt_test_matmul(void* handle, const char* name, const float* X, int m, float* Y, int path);

/* Decodes a matrix on the GPU to host codes, one code per byte [N, K].  Replaces rt_test_decode,
 * kernels/llmrt.cu:2461. */
int rt_test_decode(void* handle, const char* name, uint8_t* out);

/* Decodes a matrix on `threads` host threads to symbols [N, K / (8 / bits)].  Replaces rt_test_cpu_decode,
 * kernels/llmrt.cu:2543. */
int rt_test_cpu_decode(void* handle, const char* name, int threads, uint8_t* out);

/* GPU decode of every coded matrix into scratch, median seconds per pass over `reps` passes.  Replaces
 * rt_gpu_decode_all, kernels/llmrt.cu:2482. */
double rt_gpu_decode_all(void* handle, int reps);

/* Host decode of every coded matrix on `threads` threads; returns seconds and the symbol count.  Replaces
 * rt_cpu_decode_all, kernels/llmrt.cu:2558. */
double rt_cpu_decode_all(void* handle, int threads, long long* symbols);

/* Counters by name ("resident_bytes", "coded_bytes", "side_bytes", "n_matrices", "graph_launches", "graph_captures");
 * -1 for an unknown key.  Replaces rt_stat, kernels/llmrt.cu:2276.  Additions for tensor-parallel runs:
 * "time_collectives" arms a measurement (returns 0): the next rt_forward pass is launched directly with CUDA events
 * around every collective; afterwards "collective_us" is the time spent between those event pairs and
 * "collective_calls" their number. */
double rt_stat(void* handle, const char* key);

/* ---- decoder runtime (bundles whose cfg describes a model: n_layers, hidden, n_heads, ...) ------------------- */

/* Runs n tokens at the current position through the decoder (chunks of max_batch): embedding, per layer RMSNorm,
 * coded qkv / o / gate / up / down products, rotate-half RoPE, fp16 KV cache, causal grouped-query attention, SwiGLU;
 * final norm and lm_head.  logits (host): n x vocab if all_logits, else vocab values of the last token; may be NULL.
 * Returns 0, -1 on context overflow, or a negative status.  Replaces rt_forward, kernels/llmrt.cu:2291. */
int rt_forward(void* handle, const int* ids, int n, float* logits, int all_logits);

/* Position bookkeeping.  Replace rt_reset, rt_set_window, rt_set_pos, rt_pos, rt_vocab, kernels/llmrt.cu:2269-2274:
 * rt_set_pos only rewinds (the KV cache below the new position is kept); rt_set_window sets a sliding attention
 * window (0 = none). */
/* Greedy decoding without a round trip per token (no counterpart in the reference, whose generation loops pick every
 * token on the host with `argmax`, kernels/llmrt.cu:2663, 2816-2820, 3065-3070): n one-token passes starting with `first_token` at the current
 * position; the arg-max of each pass (lowest id among equal logits, like a host arg-max) is taken on the device and
 * becomes the token of the next pass; out[i] = token chosen by pass i.  The position advances by n.  Equivalent to n
 * calls of rt_forward with an arg-max in between.  With tensor parallelism every rank calls it with the same arguments.
 * Returns 0, -1 on context overflow, or a negative status. */
int rt_decode_greedy(void* handle, int first_token, int n, int* out);

void rt_reset(void* handle);
void rt_set_window(void* handle, int w);
void rt_set_pos(void* handle, int p);
int rt_pos(void* handle);
int rt_vocab(void* handle);

/* Tensor parallelism over NCCL (additions; the reference is single-GPU).  Every rank opens its own shard bundle (cfg
 * tp_world / tp_rank; n_heads, n_kv_heads, inter and vocab are the shard's sizes), rank 0 obtains an id with
 * lw_tp_unique_id, all ranks call rt_tp_init with it.  rt_forward then all-reduces the partial outputs of `o` and
 * `down` and gathers the logits slices into the full vocabulary. */
int lw_tp_unique_id(uint8_t* out128);
int rt_tp_init(void* handle, int rank, int world, const uint8_t* id128);

/* Optional second step: the all-reduces of `o` and `down` over peer memory, fused with the RMSNorm that consumes them
 * (one kernel per rank writes its partial rows into every rank's exchange buffer with plain NVLink stores, waits for
 * the other ranks' flags and sums in rank order; no multicast).  rt_tp_peer_export allocates this rank's exchange buffer
 * and returns its 64-byte CUDA IPC handle; the caller gathers the handles of all ranks (rank-major, world x 64 bytes) and
 * gives them to rt_tp_peer_open, which maps the peers' buffers.  Without this step the all-reduces are NCCL calls.  The
 * logits are gathered by NCCL either way.  rt_tp_error reads and clears the runtime's device error word (1: a rank's
 * flag did not arrive within the poll limit; the pass's logits are then void). */
int rt_tp_peer_export(void* handle, uint8_t* out64);
int rt_tp_peer_open(void* handle, const uint8_t* handles, int world);
int rt_tp_error(void* handle);
/* With tensor parallelism the waits at the end of rt_forward / rt_decode_greedy are bounded: while the pass runs the
 * library polls ncclCommGetAsyncError, and after `timeout_ms` (default: LW_TP_TIMEOUT_MS in the environment, else
 * 60000) without completion - a rank never joined the collective - it aborts the communicator, returns LW_ERR_CUDA and
 * refuses further passes on this handle.  0 restores the default.  No reference counterpart (single GPU). */
int rt_tp_set_timeout(void* handle, int timeout_ms);

/* ---- per-matrix entry points on device pointers (additions) ---------------------------------------------- */

/* Index of a matrix in the handle (>= 0) or -1.  The *_id variants below skip the name lookup. */
int lw_matrix_id(void* handle, const char* name);

/* Shape and sizes of matrix `id`: N rows, K weights per row, block format, coded blob bytes and side bytes as in
 * the manifest (the algorithmic bytes of one product), and the bytes the device layout occupies. */
int lw_matrix_info(void* handle, int id, int* N, int* K, int* fmt, long long* blob_bytes, long long* side_bytes,
                   long long* device_bytes);

/* How the batch-1 kernel decodes matrix `id` (chosen from the data when the bundle is opened; no reference
 * counterpart): symbols per refill group (0 = that kernel is not used), index bits of its replicated table (10 or 11)
 * and the share of work units (64 rows x one column segment) that cannot use that group size and fall back to groups
 * of two symbols or, for 11-bit codes under the 10-bit table, to symbol-by-symbol decoding. */
int lw_matrix_plan(void* handle, int id, int* group, int* index_bits, double* slow_fraction);

/* y[m, N] (fp32, row stride N) = x[m, K] . W^T for 1 <= m <= 8; x is fp16 (x_is_half != 0) or fp32, row-major, on
 * the device; y_dev must be 16-byte aligned.  Launches on `stream` (a cudaStream_t) and does not synchronise.  This
 * is the device-pointer form of the reference's internal matmul(), kernels/llmrt.cu:1794-1826.  Products of one
 * handle must not overlap on the GPU (they share its split-K scratch, and for m = 1 the matrix's tile-row counters):
 * issue them on one stream, as the reference's runtime does. */
int lw_linear(void* handle, int id, const void* x_dev, int x_is_half, int m, float* y_dev, void* stream);

/* n one-row products in as few launches as possible: y_j[N_j] = W_j x_j[K_j] for j < n, matrix j = matrix ids[j] of
 * handles[j] (handles may repeat), every x_j fp16 (x_is_half != 0) or every x_j fp32.  Up to eight products whose
 * matrices share block format and decode plan (lw_matrix_plan) run as ONE kernel launch in which every thread block
 * works on a single matrix: the launch's set-up and tail are paid once and its blocks keep much longer work lists,
 * which is worth about a fifth of the time of products launched one by one (the projections of a decoder layer that read
 * the same activations - gate and up, or q, k and v - are the natural use).  Other combinations are launched one by
 * one; results never depend on the grouping.  The reference runs every product as its own launch
 * (kernels/llmrt.cu:1808-1826); this entry point has no counterpart there. */
int lw_linear_batch(int n, void* const* handles, const int* ids, const void* const* xs_dev, int x_is_half,
                    float* const* ys_dev, void* stream);

/* The same product as lw_linear for callers that must not allocate device memory while they run: code that executes
 * inside a region where the allocator is off limits (a latency-critical serving loop that has already handed all of
 * its memory budget out, a plug-in running under a host framework that owns the device heap, a handle that was opened
 * by someone else and must not grow).  lw_linear draws its split-K scratch from the handle, which rt_open /
 * lw_matrix_create allocated; this entry point uses a fixed 16 MiB scratch array that is part of the library image
 * instead, so nothing is allocated or freed here, by this library or by any library it calls.
 *   - Limit: m <= 8 and at most 4,194,304 partial sums: (K / tile width) x N of them for one row, (K / tile width) x
 *     column segments x m x N for more rows; larger products are refused with LW_ERR_TOO_LARGE and a message (use
 *     lw_linear for those).
 *   - The first call on a device looks the array's device address up (once per device, with that device current); make
 *     that first call before any stream capture begins.
 *   - All calls share the one array and it keeps whatever the previous call left.  Nothing needs clearing (a call
 *     overwrites every partial sum it later reads), but two calls whose kernels overlap on the GPU - different streams,
 *     or different handles on one device - race on it: serialise them on one stream.
 *   - The 16 MiB stay resident on every GPU that loads the library, until the process ends.
 * No counterpart in the reference (its runtime always allocates through cudaMalloc in rt_open / rt_test_matmul). */
int lw_linear_static(void* handle, int id, const void* x_dev, int x_is_half, int m, float* y_dev, void* stream);

/* Fixed-width twin of matrix `id` (the role of the reference's packed `_pk` bundles and their readers LaneR / LaneQ,
 * kernels/llmrt.cu:543-630, :1733-1777): the matrix's codes at a fixed width (8 bits per pair of 4-bit codes, 5 or 6 bits
 * otherwise) in the same device layout, read by the same kernel without any Huffman decoding.  It is the decode-free
 * upper bound of the fused product: the difference between lw_linear (m = 1) and lw_linear_twin is what the entropy
 * decoding costs.  make_twin allocates a second device image of the matrix (larger than the coded one); drop_twin frees
 * it.  lw_linear_twin computes y[N] = W x for one activation row with bit-identical results to lw_linear (same
 * integer sums, same order of float operations), as the reference demands of its twins (kernels/llmrt.cu:895).
 * lw_matrix_twin_bytes: device bytes one twin product reads (-1 without a twin). */
int lw_matrix_make_twin(void* handle, int id);
int lw_matrix_drop_twin(void* handle, int id);
long long lw_matrix_twin_bytes(void* handle, int id);
int lw_linear_twin(void* handle, int id, const void* x_dev, int x_is_half, float* y_dev, void* stream);

/* Decoded and dequantised weights as fp16 [N, K] on the device: float32 block arithmetic (scale * f(q) - offset,
 * each operation rounded) rounded once to fp16.  w_half_dev must be 32-byte aligned (32-byte stores). */
int lw_decode_weights(void* handle, int id, void* w_half_dev, void* stream);

/* Decoded codes on the device, one per byte [N, K] (expand != 0) or symbols [N, K / (8 / bits)] (expand == 0).
 * out_dev must be 32-byte aligned (32-byte stores).  A matrix with a pair layout (lw_matrix_pair_bytes > 0) is decoded
 * through it, two codes per table lookup; the bytes written are the same. */
int lw_decode_codes(void* handle, int id, uint8_t* out_dev, int expand, void* stream);

/* ---- single matrices without a bundle directory (additions) ---------------------------------------------- */

/* Builds a one-matrix handle from a blob in host memory (N rows, Ks symbols per row), an optional side tensor and
 * its block format.  The matrix has id 0.  Released by rt_close.
 * What the device holds (here and in rt_open) is the loader's business: a block-format matrix whose code has 11-bit
 * words is re-coded with words of at most 10 bits (LW_RECODE=0 in the environment: not), Q6_K / Q5_K matrices also get a
 * pair layout (below).  Decoded symbols, products and the byte counts lw_matrix_info reports for the bundle do not change. */
void* lw_matrix_create(const uint8_t* blob, long long blob_bytes, int N, int Ks, int fmt, const uint8_t* side,
                       long long side_bytes);

/* ---- host-side codec (no GPU needed; additions mirroring lazyweights/bundle.py:57-106) -------------------- */

/* Encodes symbols [N, Ks] into a blob.  Returns the blob size in bytes; if out is NULL or cap is too small only the
 * size is returned.  nbits receives the payload bits. */
long long lw_encode_huf8(const uint8_t* sym, int N, int Ks, uint8_t* out, long long cap, long long* nbits);

/* llama.cpp blocks of format fmt (Q4_K 144, Q5_K 176, Q6_K 210, IQ4_XS 136 bytes per 256 weights) <-> codes in weight
 * order [nblk, 256] and the blocks' side bytes [nblk, 16 / 16 / 18 / 8].  join is the exact inverse of split (it
 * refuses codes that do not fit the format).  Replace split / join, scripts/kq_code.py:37-81. */
int lw_block_bytes(int fmt);
int lw_split_blocks(int fmt, const uint8_t* blocks, long long nblk, uint8_t* q, uint8_t* side);
int lw_join_blocks(int fmt, const uint8_t* q, const uint8_t* side, long long nblk, uint8_t* blocks);

/* The n-gram draft cache of speculative decoding (the reference CLI's `--drafter ngramcache`,
 * kernels/llmrt.cu:2604-2661): push every prompt and accepted token, one by one; draft proposes up to kmax tokens,
 * each from the longest n-gram (n = 4..1) of the sequence so far whose most frequent continuation has enough samples
 * and share (lax thresholds: 2 / 2 / 1 / 1 samples, 66 / 50 / 50 / 50 per cent).  Returns the number of drafted tokens. */
void* lw_ngram_create(void);
void lw_ngram_destroy(void* cache);
int lw_ngram_push(void* cache, const int* tokens, int n);
int lw_ngram_draft(void* cache, int* out, int kmax);

/* Full host-side validation of a blob: canonical table, every lane decodes and ends where the next begins. */
int lw_validate_blob(const uint8_t* blob, long long blob_bytes, int N, int Ks);

/* Host only: reads a bundle directory's manifest, checks that every tensor lies inside weights.bin and, if the cfg
 * describes a model, that every tensor the decoder runtime indexes has the shape the cfg implies (coded matrices vs
 * heads / hidden / inter / vocab, norm vectors, rotary tables, embedding and its scale tensors).  rt_open runs the
 * same check before it uploads anything.  The reference exits on such bundles (kernels/llmrt.cu:2146-2171). */
int lw_validate_bundle(const char* dir);

/* Threaded host decode of a blob to symbols [N, Ks] (the algorithm of cpu_decode, kernels/llmrt.cu:2513-2541). */
int lw_cpu_decode(const uint8_t* blob, long long blob_bytes, int N, int Ks, int threads, uint8_t* out);

/* Host only (no GPU needed): validates a blob and builds the device layout that lw_matrix_create would upload, for
 * inspection and for tests that replay the kernels' bit arithmetic on the CPU.  info[0..7] = column segments per tile
 * row, pad bits per chain, symbols per refill group of the batch-1 kernel (0 = not used), index bits of its table,
 * entries of group_base, entries of unit_class, words of scales behind every work unit, longest unit in words.
 * Returns the number of layout words (negative status on error); each array is filled if its capacity suffices
 * (call once with zero capacities to learn the sizes).  `side` may be null for fmt = LW_FMT_NONE.  No reference
 * counterpart (the reference's interleave_huf8 re-layout, kernels/llmrt.cu:1208-1257, is internal to rt_open). */
long long lw_host_layout(const uint8_t* blob, long long blob_bytes, int N, int Ks, int fmt, const uint8_t* side,
                         long long side_bytes, int* info, uint32_t* group_base, long long group_base_cap,
                         uint32_t* words, long long words_cap, uint8_t* unit_class, long long unit_class_cap);

/* The decode table of that layout, lut[2048] = symbol | length << 8 per 11-bit window: the blob's own table, or, where
 * the loader re-coded the matrix with a shorter length limit (LW_RECODE), the table of the code the device holds.
 * Returns the longest code length (negative status on error).  No reference counterpart. */
int lw_host_layout_table(const uint8_t* blob, long long blob_bytes, int N, int Ks, int fmt, const uint8_t* side,
                         long long side_bytes, uint16_t* lut);

/* Pair layout.  For Q6_K and Q5_K matrices whose K is a multiple of 512 the loader keeps a second device layout
 * that every product kernel (one row, 2..8 rows fused, the tensor-core kernel up to 64 rows - where the layout's larger
 * work units fit their shared memory) and the decode to fp16 weights read: two adjacent codes of a row are one symbol of a prefix code built from the matrix's own pair counts (at most
 * 12 bits for pairs of 6-bit codes, 11 for pairs of 5-bit codes), so that the kernel does one table lookup per two
 * weights, as it does for the 4-bit formats whose bundle symbols are pairs already.  The decoded codes are the same;
 * device memory holds the matrix twice (LW_PAIRS=0 in the environment at load: no pair layouts).  No reference
 * counterpart: the reference's kernel decodes these formats one symbol per weight (kernels/llmrt.cu:972-1024).
 * lw_matrix_pair_bytes: bytes of the pair layout that one product reads (0: the matrix has none).
 * lw_host_pairs: host only, builds the layout from decoded codes [N, K] (one per weight; fmt LW_FMT_Q6_K or
 * LW_FMT_Q5_K) for inspection and CPU replay tests.  info[0..7] = column segments per tile row, pad bits per chain,
 * symbols per group, index bits of the table, entries of group_base, longest code, words of scales behind every unit,
 * longest unit in words; table = [1 << index bits] entries length << 28 | value of the second weight << 8 | value of
 * the first (signed bytes).  Returns the number of layout words; arrays are filled if their capacity suffices. */
long long lw_matrix_pair_bytes(void* handle, int id);
long long lw_host_pairs(const uint8_t* codes, int N, int K, int fmt, const uint8_t* side, long long side_bytes, int* info,
                        uint32_t* table, long long table_cap, uint32_t* group_base, long long group_base_cap,
                        uint32_t* words, long long words_cap);

/* ---- diagnostics ------------------------------------------------------------------------------------------ */

/* Message of the last failure on the calling thread. */
const char* lw_last_error(void);

/* Status code of the last rt_open / lw_matrix_create on the calling thread (they can only return NULL). */
int lw_last_status(void);

/* Reads and clears the device error word (bit 0: a bounded wait on a bulk copy gave up).  After a non-zero answer the
 * results of products that were in flight are undefined; the next product of every matrix first zeroes the matrix's
 * tile-row counters again, so later products are correct. */
int lw_kernel_error(void);

/* Number of kernels this library has launched since it was loaded. */
long long lw_launch_count(void);

/* Test switches (no reference counterpart).  Keys: "max_units" (2..1024: units a block is dealt per launch; smaller
 * values make a product run as several launches over ranges of tile rows, the path very tall matrices take),
 * "wait_limit" (polls after which a device-side wait gives up), "drop_unit" (block 0's producers never copy this unit
 * of their list, so the waits for it run out; -1 = none), "t5_min_rows" (1..65: products of at least this many rows,
 * and at most 64, take the decode + tcgen05 kernel; 9 in production), "pairs" (0 / 1: product kernels read the bundle's own code even
 * where a matrix has a pair layout), "reset" (all back to the production values). */
int lw_debug_set(const char* key, long long value);
/* Test hook for the bounded wait above: holds the handle's stream up with a host function that sleeps `ms`
 * milliseconds (0..5000; the GPU is idle meanwhile) and runs the bounded wait with the handle's timeout: 0 if the
 * stream drained in time, LW_ERR_CUDA if the wait gave up first. */
int lw_debug_stream_stall(void* handle, int ms);

/* Launches one warp that waits, `limit` polls each, on a copy barrier nothing completes and on a release counter
 * nothing advances.  Returns 1 (barrier wait gave up) + 2 (counter wait gave up) = 3, or a negative status; the device
 * error word is set as by any wait that gives up (lw_kernel_error then returns 1).  Shows, without a fault, that a
 * lost copy ends a kernel instead of hanging it. */
int lw_debug_wait_probe(long long limit);

#ifdef __cplusplus
}
#endif
#endif
