/* illatio_oracle_simd.c -- the CPU baseline's fast form: the row dots of illatio_oracle.c with AVX2 integer
 * instructions, and a pool of threads pinned one to a core.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT (see illatio_oracle.c).  Used only when the benchmark's CPU legs ask for it
 * (orc_set_fast); parity checks run the portable loops.
 *
 * The reference's x86 kernels are IQ2XXS-DOT-AVX2 and Q2K-DOT-AVX2 (src/avx2.lisp:77-150: VPSIGNB / VPMADDUBSW /
 * VPMADDWD, the eight lanes summed per block, then the block's float scales); they are restated here with
 * intrinsics and give the bits of orc_iq2xxs_row_dot_x86 / orc_q2k_row_dot_x86.  For Q8_0, Q4_K and Q6_K the
 * reference has no x86 kernel (its portable loop is its only x86 path); the same integer sums are taken with the
 * same instructions and the float steps stay those of the portable loops, so the results are the portable bits.
 * Threads: one per allowed core, pinned, kept alive between calls, rows split as SHARE does
 * (src/cuda-ds4f.lisp:666-699, src/pool.lisp:162-165).
 */
#define _GNU_SOURCE
#include <pthread.h>
#include <sched.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "iq2xxs_tables.h"

#define QK_K 256
enum { ORC_Q8_0 = 0, ORC_Q4_K = 1, ORC_Q6_K = 2, ORC_Q2_K = 3, ORC_IQ2_XXS = 4 };

float orc_half_to_single(uint16_t h);
float orc_row_dot(int fmt, const uint8_t* w, int ncols, const int8_t* xq, const float* xs, const int32_t* bs);

#if defined(__x86_64__) && defined(__AVX2__)
#include <immintrin.h>

int orc_simd_available(void) { return __builtin_cpu_supports("avx2") ? 1 : 0; }

static inline float f16_at(const uint8_t* w, int64_t i) {
  return orc_half_to_single((uint16_t)(w[i] | (w[i + 1] << 8)));
}
static inline int hsum8(__m256i v) {
  __m128i s = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
  s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4e));
  s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xb1));
  return _mm_cvtsi128_si32(s);
}
/* 32 unsigned bytes times 32 signed bytes: sixteen sums of two products (no saturation for a <= 127) */
static inline __m256i mul_u8_s8(__m256i a, __m256i b) { return _mm256_maddubs_epi16(a, b); }

static float q8_0_dot(const uint8_t* w, int nb, const int8_t* xq, const float* xs) {
  const __m256i ones = _mm256_set1_epi16(1);
  float sum = 0.0f;
  for (int b = 0; b < nb; ++b) {
    const uint8_t* p = w + (int64_t)b * 34;
    const __m256i wv = _mm256_loadu_si256((const __m256i*)(p + 2));
    const __m256i xv = _mm256_loadu_si256((const __m256i*)(xq + b * 32));
    /* |w| * (x with w's sign): VPSIGNB / VPMADDUBSW, as src/avx2.lisp does for its signed operands */
    const __m256i pr = mul_u8_s8(_mm256_abs_epi8(wv), _mm256_sign_epi8(xv, wv));
    const int acc = hsum8(_mm256_madd_epi16(pr, ones));
    sum += (float)acc * (f16_at(p, 0) * xs[b]);
  }
  return sum;
}

static void scale_min_k4(int j, const uint8_t* q, int* sc, int* mn) {
  if (j < 4) { *sc = q[j] & 63; *mn = q[j + 4] & 63; }
  else { *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

static float q4k_dot(const uint8_t* w, int nb, const int8_t* yq, const float* yd, const int32_t* ybs) {
  const __m256i m4 = _mm256_set1_epi8(0xF);
  float sum = 0.0f;
  for (int i = 0; i < nb; ++i) {
    const uint8_t* p = w + (int64_t)i * 144;
    const float ydi = yd[i], d = ydi * f16_at(p, 0), dmin = ydi * f16_at(p, 2);
    int imin = 0, sc[8], mn[8];
    for (int g = 0; g < 8; ++g) scale_min_k4(g, p + 4, &sc[g], &mn[g]);
    for (int g = 0; g < 8; ++g) imin += mn[g] * (ybs[i * 16 + 2 * g] + ybs[i * 16 + 2 * g + 1]);
    sum = sum - dmin * (float)imin;
    __m256i acc = _mm256_setzero_si256();
    for (int k = 0; k < 4; ++k) {
      const __m256i q = _mm256_loadu_si256((const __m256i*)(p + 16 + k * 32));
      const int8_t* y = yq + (int64_t)i * QK_K + k * 64;
      const __m256i lo = mul_u8_s8(_mm256_and_si256(q, m4), _mm256_loadu_si256((const __m256i*)y));
      const __m256i hi = mul_u8_s8(_mm256_and_si256(_mm256_srli_epi16(q, 4), m4), _mm256_loadu_si256((const __m256i*)(y + 32)));
      acc = _mm256_add_epi32(acc, _mm256_madd_epi16(lo, _mm256_set1_epi16((short)sc[2 * k])));
      acc = _mm256_add_epi32(acc, _mm256_madd_epi16(hi, _mm256_set1_epi16((short)sc[2 * k + 1])));
    }
    sum = sum + d * (float)hsum8(acc);
  }
  return sum;
}

static float q6k_dot(const uint8_t* w, int nb, const int8_t* yq, const float* yd, const int32_t* ybs) {
  const __m256i m4 = _mm256_set1_epi8(0xF), m2 = _mm256_set1_epi8(3);
  float sum = 0.0f;
  for (int i = 0; i < nb; ++i) {
    const uint8_t* p = w + (int64_t)i * 210;
    const uint8_t *ql = p, *qh = p + 128;
    const int8_t* sc = (const int8_t*)(p + 192);
    int imins = 0;
    for (int g = 0; g < 16; ++g) imins += ybs[i * 16 + g] * (int)sc[g];
    __m256i acc = _mm256_setzero_si256();
    for (int c = 0; c < 2; ++c) {
      const __m256i h = _mm256_loadu_si256((const __m256i*)(qh + 32 * c));
      for (int part = 0; part < 4; ++part) {
        const __m256i l = _mm256_loadu_si256((const __m256i*)(ql + 64 * c + ((part & 1) ? 32 : 0)));
        const __m256i low = part < 2 ? _mm256_and_si256(l, m4) : _mm256_and_si256(_mm256_srli_epi16(l, 4), m4);
        __m256i hb;  /* bits 2 part, 2 part + 1 of the high bytes, at bit 4 */
        switch (part) {
          case 0: hb = _mm256_slli_epi16(_mm256_and_si256(h, m2), 4); break;
          case 1: hb = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 2), m2), 4); break;
          case 2: hb = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 4), m2), 4); break;
          default: hb = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 6), m2), 4); break;
        }
        const __m256i q6 = _mm256_or_si256(low, hb);
        const __m256i y = _mm256_loadu_si256((const __m256i*)(yq + (int64_t)i * QK_K + c * 128 + part * 32));
        /* the first sixteen weights of the 32 take scale 2 part, the rest 2 part + 1 */
        const __m256i sv = _mm256_set_m128i(_mm_set1_epi16((short)sc[c * 8 + part * 2 + 1]), _mm_set1_epi16((short)sc[c * 8 + part * 2]));
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(mul_u8_s8(q6, y), sv));
      }
    }
    sum = sum + (f16_at(p, 208) * yd[i]) * (float)(hsum8(acc) - 32 * imins);
  }
  return sum;
}

/* Q2K-DOT-AVX2, src/avx2.lisp:112-150 */
static float q2k_dot(const uint8_t* w, int nb, const int8_t* qs, const float* yd, const int32_t* bs) {
  const __m256i m2 = _mm256_set1_epi8(3);
  float total = 0.0f;
  for (int b = 0; b < nb; ++b) {
    const uint8_t* p = w + (int64_t)b * 84;
    int mins = 0;
    for (int j = 0; j < 16; ++j) mins += (p[j] >> 4) * bs[b * 16 + j];
    __m256i acc = _mm256_setzero_si256();
    for (int h = 0; h < 2; ++h) {
      const __m256i q = _mm256_loadu_si256((const __m256i*)(p + 16 + h * 32));
      for (int k = 0; k < 4; ++k) {
        __m256i qk;
        switch (k) {
          case 0: qk = _mm256_and_si256(q, m2); break;
          case 1: qk = _mm256_and_si256(_mm256_srli_epi16(q, 2), m2); break;
          case 2: qk = _mm256_and_si256(_mm256_srli_epi16(q, 4), m2); break;
          default: qk = _mm256_and_si256(_mm256_srli_epi16(q, 6), m2); break;
        }
        const __m256i x = _mm256_loadu_si256((const __m256i*)(qs + (int64_t)b * QK_K + h * 128 + k * 32));
        const __m256i sv = _mm256_set_m128i(_mm_set1_epi16((short)(p[h * 8 + 2 * k + 1] & 15)), _mm_set1_epi16((short)(p[h * 8 + 2 * k] & 15)));
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(mul_u8_s8(qk, x), sv));
      }
    }
    const float yb = yd[b];
    total += ((yb * f16_at(p, 80)) * (float)hsum8(acc)) - ((yb * f16_at(p, 82)) * (float)mins);
  }
  return total;
}

/* IQ2XXS-DOT-AVX2, src/avx2.lisp:77-110 */
static uint64_t g_sign_bytes[128];  /* +1 / -1 per byte, for VPSIGNB */
static pthread_once_t g_sign_once = PTHREAD_ONCE_INIT;
static void sign_bytes_init(void) {
  for (int i = 0; i < 128; ++i) {
    uint64_t v = 0;
    for (int j = 0; j < 8; ++j) v |= (uint64_t)(((ill_ksigns_iq2xs[i] >> j) & 1) ? 0xFF : 0x01) << (8 * j);
    g_sign_bytes[i] = v;
  }
}
static float iq2xxs_dot(const uint8_t* w, int nb, const int8_t* qs, const float* yd) {
  pthread_once(&g_sign_once, sign_bytes_init);
  float total = 0.0f;
  for (int b = 0; b < nb; ++b) {
    const uint8_t* p = w + (int64_t)b * 66;
    __m256i acc = _mm256_setzero_si256();
    for (int ib = 0; ib < 8; ++ib) {
      const uint8_t* so = p + 2 + ib * 8;
      uint32_t aux;
      memcpy(&aux, so + 4, 4);
      const __m256i g = _mm256_set_epi64x((long long)ill_iq2xxs_grid[so[3]], (long long)ill_iq2xxs_grid[so[2]],
                                          (long long)ill_iq2xxs_grid[so[1]], (long long)ill_iq2xxs_grid[so[0]]);
      const __m256i sg = _mm256_set_epi64x((long long)g_sign_bytes[(aux >> 21) & 127], (long long)g_sign_bytes[(aux >> 14) & 127],
                                           (long long)g_sign_bytes[(aux >> 7) & 127], (long long)g_sign_bytes[aux & 127]);
      const __m256i x = _mm256_loadu_si256((const __m256i*)(qs + (int64_t)b * QK_K + ib * 32));
      const __m256i pr = mul_u8_s8(g, _mm256_sign_epi8(x, sg));
      acc = _mm256_add_epi32(acc, _mm256_madd_epi16(pr, _mm256_set1_epi16((short)(2 * (int)(aux >> 28) + 1))));
    }
    total += (f16_at(p, 0) * yd[b]) * (float)hsum8(acc);
  }
  return 0.125f * total;
}

float orc_row_dot_simd(int fmt, const uint8_t* w, int ncols, const int8_t* xq, const float* xs, const int32_t* bs) {
  switch (fmt) {
    case ORC_Q8_0: return q8_0_dot(w, ncols / 32, xq, xs);
    case ORC_Q4_K: return q4k_dot(w, ncols / QK_K, xq, xs, bs);
    case ORC_Q6_K: return q6k_dot(w, ncols / QK_K, xq, xs, bs);
    case ORC_Q2_K: return q2k_dot(w, ncols / QK_K, xq, xs, bs);
    case ORC_IQ2_XXS: return iq2xxs_dot(w, ncols / QK_K, xq, xs);
  }
  return 0.0f;
}
#else
int orc_simd_available(void) { return 0; }
float orc_row_dot_simd(int fmt, const uint8_t* w, int ncols, const int8_t* xq, const float* xs, const int32_t* bs) {
  return orc_row_dot(fmt, w, ncols, xq, xs, bs);
}
#endif

/* ---- a pool of pinned threads ------------------------------------------------------------
 * Workers wait for a generation number to move (spinning for a while, then sleeping on a condition variable),
 * run job INDEX of the posted array and count themselves done.  The caller runs job 0 itself. */
#define POOL_MAX 256
static struct {
  pthread_mutex_t mu;
  pthread_cond_t cv;
  pthread_t th[POOL_MAX];
  int nthreads;                 /* workers alive (job indices 1 .. nthreads) */
  volatile unsigned gen;
  volatile int done;
  void* (*fn)(void*);
  char* jobs;
  size_t job_size;
  int njobs;
} g_pool = {PTHREAD_MUTEX_INITIALIZER, PTHREAD_COND_INITIALIZER, {0}, 0, 0, 0, 0, 0, 0, 0};

static int allowed_cpus(int* out, int max) {
  cpu_set_t set;
  int n = 0;
  if (sched_getaffinity(0, sizeof set, &set) != 0) return 0;
  for (int c = 0; c < CPU_SETSIZE && n < max; ++c)
    if (CPU_ISSET(c, &set)) out[n++] = c;
  return n;
}

static void* pool_worker(void* arg) {
  const int index = (int)(intptr_t)arg;
  unsigned seen = 0;
  for (;;) {
    unsigned spins = 0;
    while (g_pool.gen == seen) {
      if (++spins < 200000) { __builtin_ia32_pause(); continue; }
      pthread_mutex_lock(&g_pool.mu);
      while (g_pool.gen == seen) pthread_cond_wait(&g_pool.cv, &g_pool.mu);
      pthread_mutex_unlock(&g_pool.mu);
    }
    seen = g_pool.gen;
    __sync_synchronize();
    if (index < g_pool.njobs) g_pool.fn(g_pool.jobs + (size_t)index * g_pool.job_size);
    __sync_fetch_and_add(&g_pool.done, 1);
  }
  return 0;
}

/* Runs FN on JOBS[0 .. n) (N <= the pool's size + 1), one a thread, and returns when all are done. */
void orc_pool_run(void* (*fn)(void*), void* jobs, size_t job_size, int n) {
  if (n > POOL_MAX) n = POOL_MAX;
  if (g_pool.nthreads < n - 1) {  /* grow the pool: worker i is pinned to the i-th allowed core */
    int cpus[POOL_MAX];
    const int nc = allowed_cpus(cpus, POOL_MAX);
    for (int i = g_pool.nthreads + 1; i < n; ++i) {
      pthread_create(&g_pool.th[i], 0, pool_worker, (void*)(intptr_t)i);
      if (nc > 0) {
        cpu_set_t one;
        CPU_ZERO(&one);
        CPU_SET(cpus[i % nc], &one);
        pthread_setaffinity_np(g_pool.th[i], sizeof one, &one);
      }
    }
    g_pool.nthreads = n - 1;
  }
  g_pool.fn = fn; g_pool.jobs = (char*)jobs; g_pool.job_size = job_size; g_pool.njobs = n;
  g_pool.done = 0;
  __sync_synchronize();
  pthread_mutex_lock(&g_pool.mu);
  ++g_pool.gen;
  pthread_cond_broadcast(&g_pool.cv);
  pthread_mutex_unlock(&g_pool.mu);
  fn(jobs);  /* job 0 on the calling thread */
  while (g_pool.done < g_pool.nthreads) __builtin_ia32_pause();
}
