/* CPU oracle in C.  TEST INFRASTRUCTURE ONLY: the shipped package never links or loads this file.
 *
 * A plain restatement of the reference's CPU path for one coded matrix, used (a) as a second, independent checker
 * beside the NumPy oracle and (b) as the timed CPU baseline of the benchmark ("port"), threaded over all host cores:
 *   orc_decode        the threaded lane decoder: tiles dealt round-robin to threads, one 64-bit unaligned window per
 *                     symbol, 2048-entry table (kernels/llmrt.cu:2513-2541, lazyweights/bundle.py:88-106)
 *   orc_dequant_row   block dequantisation  w = s * f(q) - o  in float32, product and difference rounded separately
 *                     (scripts/a2_kq_bundle.py:50-82)
 *   orc_matvec        decode -> dequant -> y = W x with float32 accumulation per row (the NumPy path of the
 *                     reference's bundle check followed by a float32 product)
 *   orc_pack          the encoder's bit packing for given code lengths and reversed codes: lanes back to back in
 *                     (tile, lane) order, each lane tile row l then l + 32, LSB-first into 32-bit words
 *                     (lazyweights/bundle.py:57-85); the tables come from the NumPy oracle
 * Parity pin: tests/test_oracle_c.py checks these against the reference-made golden vectors in tests/golden.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { TILE_ROWS = 64, TILE_SYMS = 256, LANES = 32, LUT = 2048 };
enum { Q4_K = 1, Q5_K = 2, Q6_K = 3, IQ4_XS = 4 };

static const float IQ4_GRID[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

static int side_bytes(int fmt) { return fmt == Q6_K ? 18 : fmt == IQ4_XS ? 8 : 16; }
static int is_paired(int fmt) { return fmt == Q4_K || fmt == IQ4_XS; }

static float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h >> 15) << 31;
  uint32_t exp = (h >> 10) & 31, man = h & 1023, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 1024));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 1023) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

typedef struct {
  const uint8_t* blob;
  int N, Ks, threads, tid;
  uint8_t* out;
} DecodeJob;

static void decode_tile(const uint8_t* blob, int N, int Ks, int t, uint8_t* out, int out_stride, int out_row0) {
  const int KT = Ks / TILE_SYMS, T = (N / TILE_ROWS) * KT;
  const uint16_t* lut = (const uint16_t*)blob;
  const uint32_t* starts = (const uint32_t*)(blob + 2 * LUT);
  const uint8_t* payload = (const uint8_t*)(starts + (size_t)T * LANES);
  const int tr = t / KT, tc = t % KT;
  for (int lane = 0; lane < LANES; ++lane) {
    uint64_t bp = starts[(size_t)t * LANES + lane];
    for (int half = 0; half < 2; ++half) {
      uint8_t* row = out + (size_t)(tr * TILE_ROWS + half * 32 + lane - out_row0) * out_stride + tc * TILE_SYMS;
      for (int c = 0; c < TILE_SYMS; ++c) {
        uint64_t w;
        memcpy(&w, payload + ((bp >> 5) << 2), 8);
        const uint16_t e = lut[(w >> (bp & 31)) & (LUT - 1)];
        row[c] = (uint8_t)e;
        bp += e >> 8;
      }
    }
  }
}

static void* decode_worker(void* arg) {
  const DecodeJob* j = (const DecodeJob*)arg;
  const int T = (j->N / TILE_ROWS) * (j->Ks / TILE_SYMS);
  for (int t = j->tid; t < T; t += j->threads) decode_tile(j->blob, j->N, j->Ks, t, j->out, j->Ks, 0);
  return NULL;
}

/* blob (with at least 8 readable bytes after its end) -> symbols [N, Ks] */
int orc_decode(const uint8_t* blob, int N, int Ks, int threads, uint8_t* out) {
  if (threads < 1) threads = 1;
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * threads);
  DecodeJob* jobs = (DecodeJob*)malloc(sizeof(DecodeJob) * threads);
  for (int i = 0; i < threads; ++i) {
    jobs[i] = (DecodeJob){blob, N, Ks, threads, i, out};
    pthread_create(&th[i], NULL, decode_worker, &jobs[i]);
  }
  for (int i = 0; i < threads; ++i) pthread_join(th[i], NULL);
  free(th);
  free(jobs);
  return 0;
}

/* symbols [N, Ks] + per-symbol code length and bit-reversed code -> lane_start[T * 32] and payload words (zeroed by
 * the caller, (total_bits + 31) / 32 + 2 of them).  Returns the payload bits. */
long long orc_pack(const uint8_t* sym, int N, int Ks, const uint8_t* len, const uint32_t* rcode, uint32_t* starts,
                   uint32_t* words) {
  const int KT = Ks / TILE_SYMS, NT = N / TILE_ROWS;
  uint64_t acc = 0, pos = 0;
  size_t wi = 0;
  int fill = 0;
  for (int tr = 0; tr < NT; ++tr)
    for (int tc = 0; tc < KT; ++tc)
      for (int lane = 0; lane < LANES; ++lane) {
        starts[((size_t)tr * KT + tc) * LANES + lane] = (uint32_t)pos;
        for (int half = 0; half < 2; ++half) {
          const uint8_t* row = sym + (size_t)(tr * TILE_ROWS + half * 32 + lane) * Ks + tc * TILE_SYMS;
          for (int c = 0; c < TILE_SYMS; ++c) {
            const int s = row[c], l = len[s];
            acc |= (uint64_t)rcode[s] << fill;
            fill += l;
            pos += l;
            if (fill >= 32) {
              words[wi++] = (uint32_t)acc;
              acc >>= 32;
              fill -= 32;
            }
          }
        }
      }
  if (fill) words[wi++] = (uint32_t)acc;
  return (long long)pos;
}

/* (scale, offset) of the sub-blocks of one super-block */
static void sub_scales(int fmt, const uint8_t* p, float* s, float* o) {
  uint16_t h;
  if (fmt == Q4_K || fmt == Q5_K) {
    memcpy(&h, p, 2);
    const float d = half_to_float(h);
    memcpy(&h, p + 2, 2);
    const float dmin = half_to_float(h);
    const uint8_t* q = p + 4;
    for (int j = 0; j < 8; ++j) {
      int sc, mn;
      if (j < 4) {
        sc = q[j] & 63;
        mn = q[j + 4] & 63;
      } else {
        sc = (q[j + 4] & 15) | ((q[j - 4] >> 6) << 4);
        mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
      }
      s[j] = d * (float)sc;
      o[j] = dmin * (float)mn;
    }
  } else if (fmt == Q6_K) {
    memcpy(&h, p + 16, 2);
    const float d = half_to_float(h);
    for (int j = 0; j < 16; ++j) {
      s[j] = d * (float)(int8_t)p[j];
      o[j] = 0.f;
    }
  } else {
    memcpy(&h, p, 2);
    const float d = half_to_float(h);
    memcpy(&h, p + 2, 2);
    const int hi = h;
    for (int j = 0; j < 8; ++j) {
      const int ls = ((p[4 + j / 2] >> (4 * (j & 1))) & 15) | (((hi >> (2 * j)) & 3) << 4);
      s[j] = d * (float)(ls - 32);
      o[j] = 0.f;
    }
  }
}

/* one row of codes [K] + its side bytes -> float32 weights [K] */
void orc_dequant_row(int fmt, const uint8_t* q, const uint8_t* side, int K, float* w) {
  const int SB = side_bytes(fmt), GW = fmt == Q6_K ? 16 : 32;
  for (int b = 0; b < K / 256; ++b) {
    float s[16], o[16];
    sub_scales(fmt, side + (size_t)b * SB, s, o);
    for (int k = 0; k < 256; ++k) {
      const int c = q[b * 256 + k], g = k / GW;
      const float f = fmt == IQ4_XS ? IQ4_GRID[c] : (float)c - (fmt == Q6_K ? 32.f : 0.f);
      volatile float prod = s[g] * f;   /* rounded product, then rounded difference: no fused multiply-add */
      w[b * 256 + k] = prod - o[g];
    }
  }
}

int orc_dequant(int fmt, const uint8_t* q, const uint8_t* side, int N, int K, float* w) {
  const size_t srow = (size_t)(K / 256) * side_bytes(fmt);
  for (int n = 0; n < N; ++n) orc_dequant_row(fmt, q + (size_t)n * K, side + n * srow, K, w + (size_t)n * K);
  return 0;
}

typedef struct {
  const uint8_t* blob;
  const uint8_t* side;
  const float* x;
  float* y;
  int fmt, N, K, m, threads, tid;
} MatvecJob;

/* one tile row (64 matrix rows) at a time: decode its tiles, dequantise each row, accumulate in float32 */
static void* matvec_worker(void* arg) {
  const MatvecJob* j = (const MatvecJob*)arg;
  const int pair = is_paired(j->fmt), Ks = pair ? j->K / 2 : j->K, KT = Ks / TILE_SYMS, NT = j->N / TILE_ROWS;
  const size_t srow = (size_t)(j->K / 256) * side_bytes(j->fmt);
  uint8_t* sym = (uint8_t*)malloc((size_t)TILE_ROWS * Ks);
  uint8_t* q = (uint8_t*)malloc((size_t)j->K);
  float* w = (float*)malloc(sizeof(float) * j->K);
  for (int tr = j->tid; tr < NT; tr += j->threads) {
    for (int tc = 0; tc < KT; ++tc) decode_tile(j->blob, j->N, Ks, tr * KT + tc, sym, Ks, tr * TILE_ROWS);
    for (int r = 0; r < TILE_ROWS; ++r) {
      const int n = tr * TILE_ROWS + r;
      const uint8_t* srcq = sym + (size_t)r * Ks;
      if (pair) {
        for (int k = 0; k < Ks; ++k) {
          q[2 * k] = srcq[k] & 15;
          q[2 * k + 1] = srcq[k] >> 4;
        }
        srcq = q;
      }
      orc_dequant_row(j->fmt, srcq, j->side + n * srow, j->K, w);
      for (int i = 0; i < j->m; ++i) {
        const float* x = j->x + (size_t)i * j->K;
        float acc = 0.f;
        for (int k = 0; k < j->K; ++k) acc += w[k] * x[k];
        j->y[(size_t)i * j->N + n] = acc;
      }
    }
  }
  free(sym);
  free(q);
  free(w);
  return NULL;
}

/* y[m, N] = x[m, K] . W^T from the coded blob and side bytes, on `threads` threads */
int orc_matvec(int fmt, const uint8_t* blob, const uint8_t* side, int N, int K, const float* x, int m, float* y,
               int threads) {
  if (threads < 1) threads = 1;
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * threads);
  MatvecJob* jobs = (MatvecJob*)malloc(sizeof(MatvecJob) * threads);
  for (int i = 0; i < threads; ++i) {
    jobs[i] = (MatvecJob){blob, side, x, y, fmt, N, K, m, threads, i};
    pthread_create(&th[i], NULL, matvec_worker, &jobs[i]);
  }
  for (int i = 0; i < threads; ++i) pthread_join(th[i], NULL);
  free(th);
  free(jobs);
  return 0;
}
