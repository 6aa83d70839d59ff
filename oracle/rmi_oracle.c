/*
 * rmi_oracle.c -- CPU restatement (plain C) of the quantized-matmul hot path of
 * rust-model-inference.  TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and
 * the timed CPU baseline.  See rmi_oracle.h for parity status and the per-function
 * reference citations (file:line inside the reference project).
 *
 * Build: gcc -O2 -ffp-contract=off -mavx2 -mfma -mf16c -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: the reference's Rust never contracts a*b+c unless it
 * calls mul_add, and the bit patterns depend on it.
 */
#define _GNU_SOURCE
#include "rmi_oracle.h"

#include <math.h>
#include <pthread.h>
#include <sched.h>
#include <stdatomic.h>
#include <stdlib.h>
#include <string.h>

#if defined(__AVX2__) && defined(__FMA__) && defined(__F16C__)
#include <immintrin.h>
#define ORC_HAVE_AVX2 1
#else
#define ORC_HAVE_AVX2 0
#endif

/* ------------------------------------------------------------------ exp mode */

static int g_exp_mode = ORC_EXP_CR;
void orc_set_exp_mode(int mode) { g_exp_mode = mode; }
int orc_get_exp_mode(void) { return g_exp_mode; }
float orc_expf(float x) {
  if (g_exp_mode == ORC_EXP_LIBM) return expf(x);
  return (float)exp((double)x);
}

/* ------------------------------------------------------------------ f16 */

static inline uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static inline float bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* src/ops/float.rs:193-207: _mm_cvtps_ph(v, 0) / half::f16::from_f32 -- IEEE RNE. */
uint16_t orc_f32_to_f16(float v) {
  uint32_t x = f32_bits(v);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t abs = x & 0x7fffffffu;
  if (abs >= 0x7f800000u) { /* inf / nan */
    if (abs > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((abs >> 13) & 0x3ffu));
    return (uint16_t)(sign | 0x7c00u);
  }
  if (abs >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to >= 65520 -> inf */
  if (abs < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 -> 0 (tie to even) */
  int32_t exp = (int32_t)(abs >> 23) - 127;
  uint32_t man = (abs & 0x7fffffu) | 0x800000u;
  uint32_t shift, half_bits;
  if (exp < -14) { /* subnormal half */
    shift = (uint32_t)(13 + (-14 - exp));
    half_bits = 0;
  } else {
    shift = 13;
    half_bits = (uint32_t)(exp + 15) << 10;
    man &= 0x7fffffu;
  }
  uint32_t q = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) q += 1; /* carry propagates into exponent */
  return (uint16_t)(sign | (half_bits + q));
}

/* src/ops/float.rs:177-191 */
float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_f32(sign);
    /* subnormal: man * 2^-24 */
    float f = (float)man * 5.9604644775390625e-08f;
    return bits_f32(f32_bits(f) | sign);
  }
  if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
  return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

void orc_f32_slice_to_f16(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; i++) dst[i] = orc_f32_to_f16(src[i]);
}

/* src/ops/quant/mod.rs:13-22 */
float orc_f16_from_bytes(const uint8_t* data, size_t len, size_t byte_idx) {
  if (byte_idx + 2 > len) return 0.0f;
  uint16_t bits = (uint16_t)(data[byte_idx] | ((uint16_t)data[byte_idx + 1] << 8));
  float sign = (bits & 0x8000) ? -1.0f : 1.0f;
  int exp = (bits >> 10) & 0x1f;
  float frac = (float)(bits & 0x3ff) / 1024.0f;
  if (exp == 0) return sign * frac * ldexpf(1.0f, -14);
  if (exp == 31) return frac == 0.0f ? sign * INFINITY : sign * NAN;
  return sign * (1.0f + frac) * ldexpf(1.0f, exp - 15);
}

/* ------------------------------------------------------------------ Q8_0 quantizer */

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* src/ops/quant/q8_0.rs:49-71 (scalar), :176-230 (AVX2), :75-165 (NEON) */
void orc_quantize_q8_0(const float* input, size_t n, uint8_t* q8, float* scales, int sem) {
  size_t blocks = n / 32;
  for (size_t b = 0; b < blocks; b++) {
    const float* v = input + b * 32;
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) {
      float a = fabsf(v[i]);
      if (a > amax) amax = a;
    }
    if (sem == ORC_SEM_AVX2 || sem == ORC_SEM_AVX2_BLOCK) {
      /* q8_0.rs:208-229: d = amax/127, id = 127/amax, round-to-nearest-even, clamp [-128,127] */
      float d = amax == 0.0f ? 0.0f : amax / 127.0f;
      float id = amax == 0.0f ? 0.0f : 127.0f / amax;
      scales[b] = orc_f16_to_f32(orc_f32_to_f16(d));
      for (int i = 0; i < 32; i++) {
        float r = nearbyintf(v[i] * id);
        r = clampf(r, -128.0f, 127.0f);
        q8[b * 32 + i] = (uint8_t)(int8_t)(int32_t)r;
      }
    } else if (sem == ORC_SEM_NEON) {
      /* q8_0.rs:108-158: inv = 1/scale, clamp +-127 before and after vcvtnq (RNE) */
      float scale = amax / 127.0f;
      float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
      scales[b] = orc_f16_to_f32(orc_f32_to_f16(scale));
      for (int i = 0; i < 32; i++) {
        float c = clampf(v[i] * inv, -127.0f, 127.0f);
        int32_t r = (int32_t)nearbyintf(c);
        if (r < -127) r = -127;
        if (r > 127) r = 127;
        q8[b * 32 + i] = (uint8_t)(int8_t)r;
      }
    } else {
      /* q8_0.rs:57-69: inverse = 1/scale, f32::round (half away from zero), clamp [-128,127] */
      float scale = amax == 0.0f ? 0.0f : amax / 127.0f;
      float inverse = scale == 0.0f ? 0.0f : 1.0f / scale;
      scales[b] = orc_f16_to_f32(orc_f32_to_f16(scale));
      for (int i = 0; i < 32; i++) {
        float r = clampf(roundf(v[i] * inverse), -128.0f, 127.0f);
        q8[b * 32 + i] = (uint8_t)(int8_t)(int32_t)r;
      }
    }
  }
}

/* ------------------------------------------------------------------ Q8_0 GEMV */

static inline float wd_of(const uint8_t* blk) {
  return orc_f16_to_f32((uint16_t)(blk[0] | ((uint16_t)blk[1] << 8)));
}

/* src/ops/dot.rs:447-456 hsum_ps on lanes a[0..8) */
static inline float hsum8(const float* a) {
  float s0 = a[4] + a[0], s1 = a[5] + a[1], s2 = a[6] + a[2], s3 = a[7] + a[3];
  return (s0 + s1) + (s2 + s3);
}

static float q8_row_avx2(const uint8_t* row, const uint8_t* q8, const float* xs, size_t blocks) {
  /* avx2.rs:82-148 / :157-171: per block da = f16(wd)*xs[b]; eight int32 partial sums of
   * four products each (maddubs + madd); acc[l] = fma(da, f32(partial[l]), acc[l]). */
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t b = 0; b < blocks; b++) {
    const uint8_t* blk = row + b * 34;
    float da = wd_of(blk) * xs[b];
    const int8_t* w = (const int8_t*)(blk + 2);
    const int8_t* x = (const int8_t*)(q8 + b * 32);
    for (int l = 0; l < 8; l++) {
      int32_t p = 0;
      for (int i = 0; i < 4; i++) p += (int32_t)w[4 * l + i] * (int32_t)x[4 * l + i];
      acc[l] = fmaf(da, (float)p, acc[l]);
    }
  }
  return hsum8(acc);
}

static inline int32_t dot32(const int8_t* w, const int8_t* x) {
  int32_t d = 0;
  for (int i = 0; i < 32; i++) d += (int32_t)w[i] * (int32_t)x[i];
  return d;
}

void orc_matmul_q8_0_range(const uint8_t* weight, const uint8_t* input_q8,
                           const float* input_scales, float* output, size_t n_in,
                           size_t row_start, size_t row_end, int sem) {
  size_t blocks = n_in / 32;
  size_t stride = blocks * 34;
  for (size_t row = row_start; row < row_end; row++) {
    const uint8_t* r = weight + row * stride;
    float sum;
    if (sem == ORC_SEM_AVX2) {
      sum = q8_row_avx2(r, input_q8, input_scales, blocks);
    } else if (sem == ORC_SEM_NEON || sem == ORC_SEM_AVX2_BLOCK) {
      /* neon.rs:59-70: sum = fma(f32(dot), wd*xs[b], sum) */
      sum = 0.0f;
      for (size_t b = 0; b < blocks; b++) {
        const uint8_t* blk = r + b * 34;
        int32_t d = dot32((const int8_t*)(blk + 2), (const int8_t*)(input_q8 + b * 32));
        sum = fmaf((float)d, wd_of(blk) * input_scales[b], sum);
      }
    } else {
      /* scalar.rs:42-56: sum += wd * xs[b] * f32(dot)  == ((wd*xs)*dot) + sum */
      sum = 0.0f;
      for (size_t b = 0; b < blocks; b++) {
        const uint8_t* blk = r + b * 34;
        int32_t d = dot32((const int8_t*)(blk + 2), (const int8_t*)(input_q8 + b * 32));
        float t = wd_of(blk) * input_scales[b];
        t = t * (float)d;
        sum = sum + t;
      }
    }
    output[row - row_start] = sum;
  }
}

int orc_has_avx2_fast(void) { return ORC_HAVE_AVX2; }

#if ORC_HAVE_AVX2
static inline float hsum_ps_256(__m256 v) {
  __m128 hi = _mm256_extractf128_ps(v, 1);
  __m128 lo = _mm256_castps256_ps128(v);
  __m128 s = _mm_add_ps(hi, lo);
  __m128 sh = _mm_movehdup_ps(s);
  __m128 s2 = _mm_add_ps(s, sh);
  __m128 s3 = _mm_movehl_ps(sh, s2);
  return _mm_cvtss_f32(_mm_add_ss(s2, s3));
}
static inline float f16c_to_f32(const uint8_t* p) {
  uint16_t h;
  memcpy(&h, p, 2);
  return _cvtsh_ss(h);
}
static inline __m256 q8_block_term(const uint8_t* blk, __m256i qy, __m256i ones) {
  __m256i qx = _mm256_loadu_si256((const __m256i*)(blk + 2));
  __m256i ax = _mm256_sign_epi8(qx, qx);
  __m256i sy = _mm256_sign_epi8(qy, qx);
  return _mm256_cvtepi32_ps(_mm256_madd_epi16(ones, _mm256_maddubs_epi16(ax, sy)));
}
#endif

int orc_matmul_q8_0_range_avx2_fast(const uint8_t* weight, const uint8_t* input_q8,
                                    const float* input_scales, float* output, size_t n_in,
                                    size_t row_start, size_t row_end) {
#if ORC_HAVE_AVX2
  size_t blocks = n_in / 32, stride = blocks * 34;
  const __m256i ones = _mm256_set1_epi16(1);
  size_t row = row_start;
  for (; row + 4 <= row_end; row += 4) {
    const uint8_t* r0 = weight + row * stride;
    const uint8_t *r1 = r0 + stride, *r2 = r1 + stride, *r3 = r2 + stride;
    __m256 c0 = _mm256_setzero_ps(), c1 = c0, c2 = c0, c3 = c0;
    for (size_t b = 0; b < blocks; b++) {
      __m256i qy = _mm256_loadu_si256((const __m256i*)(input_q8 + b * 32));
      float bd = input_scales[b];
      size_t o = b * 34;
      c0 = _mm256_fmadd_ps(_mm256_set1_ps(f16c_to_f32(r0 + o) * bd), q8_block_term(r0 + o, qy, ones), c0);
      c1 = _mm256_fmadd_ps(_mm256_set1_ps(f16c_to_f32(r1 + o) * bd), q8_block_term(r1 + o, qy, ones), c1);
      c2 = _mm256_fmadd_ps(_mm256_set1_ps(f16c_to_f32(r2 + o) * bd), q8_block_term(r2 + o, qy, ones), c2);
      c3 = _mm256_fmadd_ps(_mm256_set1_ps(f16c_to_f32(r3 + o) * bd), q8_block_term(r3 + o, qy, ones), c3);
    }
    float* out = output + (row - row_start);
    out[0] = hsum_ps_256(c0);
    out[1] = hsum_ps_256(c1);
    out[2] = hsum_ps_256(c2);
    out[3] = hsum_ps_256(c3);
  }
  for (; row < row_end; row++) {
    const uint8_t* r0 = weight + row * stride;
    __m256 c0 = _mm256_setzero_ps();
    for (size_t b = 0; b < blocks; b++) {
      __m256i qy = _mm256_loadu_si256((const __m256i*)(input_q8 + b * 32));
      size_t o = b * 34;
      c0 = _mm256_fmadd_ps(_mm256_set1_ps(f16c_to_f32(r0 + o) * input_scales[b]),
                           q8_block_term(r0 + o, qy, ones), c0);
    }
    output[row - row_start] = hsum_ps_256(c0);
  }
  return 1;
#else
  (void)weight; (void)input_q8; (void)input_scales; (void)output; (void)n_in; (void)row_start; (void)row_end;
  return 0;
#endif
}

int orc_quantize_q8_0_avx2_fast(const float* input, size_t n, uint8_t* q8, float* scales) {
#if ORC_HAVE_AVX2
  const __m256 sign_mask = _mm256_set1_ps(-0.0f);
  const __m256 hi = _mm256_set1_ps(127.0f), lo = _mm256_set1_ps(-128.0f);
  const __m256i perm = _mm256_setr_epi32(0, 4, 1, 5, 2, 6, 3, 7);
  for (size_t b = 0; b < n / 32; b++) {
    const float* p = input + b * 32;
    __m256 v[4], m = _mm256_setzero_ps();
    for (int i = 0; i < 4; i++) {
      v[i] = _mm256_loadu_ps(p + 8 * i);
      m = _mm256_max_ps(m, _mm256_andnot_ps(sign_mask, v[i]));
    }
    __m128 m4 = _mm_max_ps(_mm256_extractf128_ps(m, 1), _mm256_castps256_ps128(m));
    m4 = _mm_max_ps(m4, _mm_movehl_ps(m4, m4));
    m4 = _mm_max_ss(m4, _mm_movehdup_ps(m4));
    float amax = _mm_cvtss_f32(m4);
    float d = amax == 0.0f ? 0.0f : amax / 127.0f;
    float id = amax == 0.0f ? 0.0f : 127.0f / amax;
    scales[b] = _cvtsh_ss(_cvtss_sh(d, 0));
    __m256 idv = _mm256_set1_ps(id);
    __m256i q[4];
    for (int i = 0; i < 4; i++) {
      __m256 r = _mm256_round_ps(_mm256_mul_ps(v[i], idv), _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
      q[i] = _mm256_cvtps_epi32(_mm256_min_ps(_mm256_max_ps(r, lo), hi));
    }
    __m256i packed = _mm256_packs_epi16(_mm256_packs_epi32(q[0], q[1]), _mm256_packs_epi32(q[2], q[3]));
    _mm256_storeu_si256((__m256i*)(q8 + b * 32), _mm256_permutevar8x32_epi32(packed, perm));
  }
  return 1;
#else
  (void)input; (void)n; (void)q8; (void)scales;
  return 0;
#endif
}

/* src/ops/kernel/q8_0/parallel.rs:102-139 */
void orc_matmul_q8_0_parallel_rows(const uint8_t* weight, const uint8_t* input_q8,
                                   const float* input_scales, float* output, size_t n_in,
                                   size_t n_out, size_t ith, size_t nth, int sem) {
  if (nth <= 1 || n_out == 0) {
    orc_matmul_q8_0_range(weight, input_q8, input_scales, output, n_in, 0, n_out, sem);
    return;
  }
  size_t per = (n_out + nth - 1) / nth;
  size_t s = ith * per;
  size_t e = s + per < n_out ? s + per : n_out;
  if (s >= e) return;
  orc_matmul_q8_0_range(weight, input_q8, input_scales, output + s, n_in, s, e, sem);
}

void orc_q8_0_block_sums(const uint8_t* weight, const uint8_t* input_q8, int32_t* sums,
                         size_t n_in, size_t row_start, size_t row_end) {
  size_t blocks = n_in / 32, stride = blocks * 34;
  for (size_t row = row_start; row < row_end; row++)
    for (size_t b = 0; b < blocks; b++)
      sums[(row - row_start) * blocks + b] =
          dot32((const int8_t*)(weight + row * stride + b * 34 + 2), (const int8_t*)(input_q8 + b * 32));
}

/* src/ops/kernel/q8_0/scalar.rs:3-29 */
void orc_matmul_q8_0_fallback_range(const uint8_t* weight, const float* input, float* output,
                                    size_t n_in, size_t row_start, size_t row_end) {
  size_t blocks = n_in / 32, stride = blocks * 34;
  for (size_t row = row_start; row < row_end; row++) {
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
      const uint8_t* blk = weight + row * stride + b * 34;
      float d = wd_of(blk);
      float local = 0.0f;
      for (int k = 0; k < 32; k++) {
        float t = (float)(int8_t)blk[2 + k] * input[b * 32 + k];
        local = local + t;
      }
      float t = d * local;
      sum = sum + t;
    }
    output[row - row_start] = sum;
  }
}

/* src/ops/kernel/q8_0/avx2.rs:180-217: two 8-lane accumulators; per block acc0 takes the products of elements
 * 0..7 and 16..23, acc1 those of 8..15 and 24..31, each as fma(d * f32(q), x, acc); lanes added, then hsum_ps. */
void orc_matmul_q8_0_avx2_range(const uint8_t* weight, const float* input, float* output,
                                size_t n_in, size_t row_start, size_t row_end) {
  size_t blocks = n_in / 32, stride = blocks * 34;
  for (size_t row = row_start; row < row_end; row++) {
    float acc0[8] = {0}, acc1[8] = {0};
    for (size_t b = 0; b < blocks; b++) {
      const uint8_t* blk = weight + row * stride + b * 34;
      const int8_t* q = (const int8_t*)(blk + 2);
      const float* x = input + b * 32;
      float d = wd_of(blk);
      for (int l = 0; l < 8; l++) acc0[l] = fmaf(d * (float)q[l], x[l], acc0[l]);
      for (int l = 0; l < 8; l++) acc1[l] = fmaf(d * (float)q[8 + l], x[8 + l], acc1[l]);
      for (int l = 0; l < 8; l++) acc0[l] = fmaf(d * (float)q[16 + l], x[16 + l], acc0[l]);
      for (int l = 0; l < 8; l++) acc1[l] = fmaf(d * (float)q[24 + l], x[24 + l], acc1[l]);
    }
    float s[8];
    for (int l = 0; l < 8; l++) s[l] = acc0[l] + acc1[l];
    output[row - row_start] = hsum8(s);
  }
}

/* src/ops/kernel/q8_0/parallel.rs:317-341 (ops::matmul_q8_0, f32 input): the AVX2 kernel on x86, the scalar
 * kernel everywhere else (there is no NEON variant of this function). */
void orc_matmul_q8_0_f32(const uint8_t* weight, const float* input, float* output, size_t n_in, size_t n_out,
                         int sem) {
  if (sem == ORC_SEM_AVX2) orc_matmul_q8_0_avx2_range(weight, input, output, n_in, 0, n_out);
  else orc_matmul_q8_0_fallback_range(weight, input, output, n_in, 0, n_out);
}

/* ------------------------------------------------------------------ thread pool */
/* Fork-join over nth workers with the reference's (ith, nth) convention
 * (src/core/thread_pool.rs:119-161: every worker runs f(ith, nth), caller is ith 0). */

typedef void (*orc_job_fn)(void* ctx, size_t ith, size_t nth);
typedef struct {
  pthread_t* threads;
  size_t n;
  atomic_ulong gen;
  atomic_ulong done;
  orc_job_fn fn;
  void* ctx;
  atomic_int stop;
} orc_pool;
static orc_pool g_pool;
static pthread_mutex_t g_pool_mu = PTHREAD_MUTEX_INITIALIZER;

typedef struct {
  size_t ith;
} orc_worker_arg;

static void* orc_worker(void* p) {
  size_t ith = ((orc_worker_arg*)p)->ith;
  free(p);
  unsigned long seen = 0;
  for (;;) {
    unsigned spins = 0;
    while (atomic_load_explicit(&g_pool.gen, memory_order_acquire) == seen) {
      if (atomic_load(&g_pool.stop)) return NULL;
      if (++spins > 2000) {
        sched_yield();
        spins = 0;
      }
    }
    seen = atomic_load_explicit(&g_pool.gen, memory_order_acquire);
    g_pool.fn(g_pool.ctx, ith, g_pool.n);
    atomic_fetch_add_explicit(&g_pool.done, 1, memory_order_release);
  }
}

static void orc_pool_resize(size_t n) {
  if (n < 1) n = 1;
  if (g_pool.n == n) return;
  if (g_pool.threads) {
    atomic_store(&g_pool.stop, 1);
    for (size_t i = 1; i < g_pool.n; i++) pthread_join(g_pool.threads[i], NULL);
    free(g_pool.threads);
    g_pool.threads = NULL;
    atomic_store(&g_pool.stop, 0);
  }
  g_pool.n = n;
  atomic_store(&g_pool.gen, 0);
  atomic_store(&g_pool.done, 0);
  g_pool.threads = (pthread_t*)calloc(n, sizeof(pthread_t));
  for (size_t i = 1; i < n; i++) {
    orc_worker_arg* a = (orc_worker_arg*)malloc(sizeof(*a));
    a->ith = i;
    pthread_create(&g_pool.threads[i], NULL, orc_worker, a);
  }
}

static void orc_compute(int threads, orc_job_fn fn, void* ctx) {
  if (threads <= 1) {
    fn(ctx, 0, 1);
    return;
  }
  pthread_mutex_lock(&g_pool_mu);
  orc_pool_resize((size_t)threads);
  g_pool.fn = fn;
  g_pool.ctx = ctx;
  atomic_store(&g_pool.done, 0);
  atomic_fetch_add_explicit(&g_pool.gen, 1, memory_order_release);
  fn(ctx, 0, g_pool.n);
  unsigned spins = 0;
  while (atomic_load_explicit(&g_pool.done, memory_order_acquire) != g_pool.n - 1) {
    if (++spins > 2000) {
      sched_yield();
      spins = 0;
    }
  }
  pthread_mutex_unlock(&g_pool_mu);
}

typedef struct {
  const uint8_t* w;
  const uint8_t* q8;
  const float* xs;
  float* out;
  size_t n_in, n_out;
  int sem;
} gemv_job;

static void gemv_rows(const uint8_t* w, const uint8_t* q8, const float* xs, float* out, size_t n_in,
                      size_t n_out, size_t ith, size_t nth, int sem) {
  /* parallel.rs:124-139 partition; AVX2 semantics go through the intrinsic kernel when built */
  size_t per = nth <= 1 ? n_out : (n_out + nth - 1) / nth;
  size_t s = ith * per;
  size_t e = s + per < n_out ? s + per : n_out;
  if (s >= e) return;
  if (sem == ORC_SEM_AVX2 && orc_matmul_q8_0_range_avx2_fast(w, q8, xs, out + s, n_in, s, e)) return;
  orc_matmul_q8_0_range(w, q8, xs, out + s, n_in, s, e, sem);
}

static void gemv_job_fn(void* p, size_t ith, size_t nth) {
  gemv_job* j = (gemv_job*)p;
  gemv_rows(j->w, j->q8, j->xs, j->out, j->n_in, j->n_out, ith, nth, j->sem);
}

static void quantize_any(const float* x, size_t n, uint8_t* q8, float* scales, int sem) {
  if ((sem == ORC_SEM_AVX2 || sem == ORC_SEM_AVX2_BLOCK) && orc_quantize_q8_0_avx2_fast(x, n, q8, scales)) return;
  orc_quantize_q8_0(x, n, q8, scales, sem);
}

static void pooled_gemv(const uint8_t* w, const uint8_t* q8, const float* xs, float* out,
                        size_t n_in, size_t n_out, int sem, int threads) {
  gemv_job j = {w, q8, xs, out, n_in, n_out, sem};
  orc_compute(threads, gemv_job_fn, &j);
}

/* src/ops/kernel/trait_.rs:78-109 */
void orc_q8_forward_batched(const uint8_t* weight, const float* input, float* output,
                            size_t n_tokens, size_t n_in, size_t n_out, int sem, int threads) {
  uint8_t* q8 = (uint8_t*)malloc(n_in);
  float* xs = (float*)malloc(sizeof(float) * (n_in / 32 + 1));
  for (size_t t = 0; t < n_tokens; t++) {
    quantize_any(input + t * n_in, n_in, q8, xs, sem);
    pooled_gemv(weight, q8, xs, output + t * n_out, n_in, n_out, sem, threads);
  }
  free(q8);
  free(xs);
}

/* src/ops/quant/fuse.rs:25-40 */
size_t orc_fuse_vstack(const uint8_t* a, size_t a_len, size_t a_rows, const uint8_t* b,
                       size_t b_len, size_t b_rows, uint8_t* out) {
  size_t ra = a_len / (a_rows ? a_rows : 1), rb = b_len / (b_rows ? b_rows : 1);
  if (ra != rb) return 0;
  memcpy(out, a, a_len);
  memcpy(out + a_len, b, b_len);
  return a_rows + b_rows;
}

/* src/ops/activation/mod.rs:137-151 */
void orc_silu_mul_inplace(const float* gate, float* up, size_t n) {
  for (size_t i = 0; i < n; i++) {
    float g = gate[i];
    float s = g / (1.0f + orc_expf(-g));
    up[i] = up[i] * s;
  }
}

typedef struct {
  const uint8_t *wg, *wu;
  const uint8_t* q8;
  const float* xs;
  float *gate_out, *up_out; /* named by what they hold, not by the reference's swapped buffers */
  size_t n_embd, n_ff;
  int sem;
} ffn_job;

static void ffn_job_fn(void* p, size_t ith, size_t nth) {
  /* src/models/qwen3.rs:991-1019: both GEMVs on this thread's rows, then SiLU*mul on
   * [ith*n_ff/nth, (ith+1)*n_ff/nth). Safe without a barrier only when the two ranges
   * coincide; the reference has the same property, so do the SiLU after the join instead
   * (same values, no ordering hazard). */
  ffn_job* j = (ffn_job*)p;
  gemv_rows(j->wg, j->q8, j->xs, j->gate_out, j->n_embd, j->n_ff, ith, nth, j->sem);
  gemv_rows(j->wu, j->q8, j->xs, j->up_out, j->n_embd, j->n_ff, ith, nth, j->sem);
}

void orc_ffn_swiglu_q8_0(const uint8_t* w_gate, const uint8_t* w_up, const uint8_t* w_down,
                         const float* x, float* out, float* act, size_t m, size_t n_embd,
                         size_t n_ff, int sem, int threads) {
  size_t nmax = n_embd > n_ff ? n_embd : n_ff;
  uint8_t* q8 = (uint8_t*)malloc(nmax);
  float* xs = (float*)malloc(sizeof(float) * (nmax / 32 + 1));
  float* g = (float*)malloc(sizeof(float) * n_ff);
  float* u = (float*)malloc(sizeof(float) * n_ff);
  for (size_t t = 0; t < m; t++) {
    quantize_any(x + t * n_embd, n_embd, q8, xs, sem);
    ffn_job j = {w_gate, w_up, q8, xs, g, u, n_embd, n_ff, sem};
    orc_compute(threads, ffn_job_fn, &j);
    orc_silu_mul_inplace(g, u, n_ff); /* u = (Wu x) * silu(Wg x) */
    if (act) memcpy(act + t * n_ff, u, sizeof(float) * n_ff);
    quantize_any(u, n_ff, q8, xs, sem);
    pooled_gemv(w_down, q8, xs, out + t * n_embd, n_ff, n_embd, sem, threads);
  }
  free(q8);
  free(xs);
  free(g);
  free(u);
}

/* ------------------------------------------------------------------ K-quants */

/* src/ops/quant/mod.rs:25-33 */
static inline void get_scale_min_k4(int j, const uint8_t* s, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = s[j] & 63;
    *mn = s[j + 4] & 63;
  } else {
    *sc = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
    *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
  }
}

/* src/ops/quant/mod.rs:75-80 */
static inline int32_t nearest_int(float value) {
  float t = value + 12582912.0f;
  return (int32_t)(f32_bits(t) & 0x007fffffu) - 0x00400000;
}

void orc_quantize_row_q8_k(const float* x, size_t n, orc_block_q8k* out, int sem) {
  size_t nb = n / 256;
  for (size_t i = 0; i < nb; i++) {
    const float* blk = x + i * 256;
    float amax = 0.0f, max_val = 0.0f;
    for (int j = 0; j < 256; j++) {
      float ax = fabsf(blk[j]);
      if (ax > amax) {
        amax = ax;
        max_val = blk[j];
      }
    }
    if (amax == 0.0f) {
      memset(&out[i], 0, sizeof(out[i]));
      continue;
    }
    float iscale = -127.0f / max_val;
    for (int j = 0; j < 256; j++) {
      int32_t v;
      if (sem == ORC_SEM_SCALAR) {
        /* mod.rs:103-107 */
        v = nearest_int(iscale * blk[j]);
        if (v > 127) v = 127;
      } else {
        /* mod.rs:171-182: round_ps(nearest even), clamp [-127,127] */
        v = (int32_t)nearbyintf(blk[j] * iscale);
        if (v < -127) v = -127;
        if (v > 127) v = 127;
      }
      out[i].qs[j] = (int8_t)v;
    }
    for (int j = 0; j < 16; j++) {
      int32_t s = 0;
      for (int k = 0; k < 16; k++) s += out[i].qs[j * 16 + k];
      out[i].bsums[j] = (int16_t)s;
    }
    out[i].d = 1.0f / iscale;
  }
}

/* 6-bit scale/min unpack shared by both dot variants (mod.rs:244-264, :739-747) */
static void q4k_unpack_scales(const uint8_t* sb, uint8_t scales[8], uint8_t mins[8]) {
  uint32_t utmp[4];
  memcpy(utmp, sb, 12);
  const uint32_t kmask1 = 0x3f3f3f3f, kmask2 = 0x0f0f0f0f, kmask3 = 0x03030303;
  utmp[3] = ((utmp[2] >> 4) & kmask2) | (((utmp[1] >> 6) & kmask3) << 4);
  uint32_t uaux = utmp[1] & kmask1;
  utmp[1] = (utmp[2] & kmask2) | (((utmp[0] >> 6) & kmask3) << 4);
  utmp[2] = uaux;
  utmp[0] &= kmask1;
  memcpy(scales, &utmp[0], 8);
  memcpy(mins, &utmp[2], 8);
}

/* element e (0..255) of the super-block: group g=e/64, low nibbles are e%64<32 */
static inline int32_t q4k_quant(const uint8_t* qs, int e) {
  int g = e / 64, r = e % 64;
  uint8_t byte = qs[g * 32 + (r & 31)];
  return r < 32 ? (byte & 0xF) : (byte >> 4);
}

void orc_q4k_q8k_block_ints(const uint8_t* blk, const orc_block_q8k* q8k, int32_t* sumi_scaled,
                            int32_t* sumi_mins) {
  uint8_t sc[8], mn[8];
  q4k_unpack_scales(blk + 4, sc, mn);
  int32_t a = 0, m = 0;
  for (int e = 0; e < 256; e++) a += (int32_t)sc[e / 32] * q4k_quant(blk + 16, e) * (int32_t)q8k->qs[e];
  for (int j = 0; j < 16; j++) m += (int32_t)q8k->bsums[j] * (int32_t)mn[j / 2];
  *sumi_scaled = a;
  *sumi_mins = m;
}

float orc_vec_dot_q4k_q8k(const uint8_t* q4k, size_t q4k_len, const orc_block_q8k* q8k, size_t nb,
                          int sem) {
  if (sem == ORC_SEM_SCALAR) {
    /* mod.rs:210-289 */
    float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float sumf = 0.0f;
    for (size_t i = 0; i < nb; i++) {
      size_t boff = i * 144;
      if (boff + 144 > q4k_len) break;
      const uint8_t* blk = q4k + boff;
      float d = orc_f16_from_bytes(q4k, q4k_len, boff);
      float dmin = orc_f16_from_bytes(q4k, q4k_len, boff + 2);
      uint8_t sc[8], mn[8];
      q4k_unpack_scales(blk + 4, sc, mn);
      int32_t sumi = 0;
      for (int j = 0; j < 16; j++) sumi += (int32_t)q8k[i].bsums[j] * (int32_t)mn[j / 2];
      int32_t aux32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int e = 0; e < 256; e++)
        aux32[e & 7] += (int32_t)sc[e / 32] * (int32_t)q8k[i].qs[e] * q4k_quant(blk + 16, e);
      float dd = d * q8k[i].d;
      for (int l = 0; l < 8; l++) {
        float t = dd * (float)aux32[l];
        sums[l] = sums[l] + t;
      }
      float dmin_val = dmin * q8k[i].d;
      float t = dmin_val * (float)sumi;
      sumf = sumf - t;
    }
    for (int l = 0; l < 8; l++) sumf = sumf + sums[l];
    return sumf;
  }
  /* mod.rs:701-799 (AVX2): eight f32 lanes for the scaled sums, four for the mins */
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float acc_m[4] = {0, 0, 0, 0};
  for (size_t i = 0; i < nb; i++) {
    size_t boff = i * 144;
    if (boff + 144 > q4k_len) break;
    const uint8_t* blk = q4k + boff;
    float d = orc_f16_from_bytes(q4k, q4k_len, boff) * q8k[i].d;
    float dmin = -orc_f16_from_bytes(q4k, q4k_len, boff + 2) * q8k[i].d;
    uint8_t sc[8], mn[8];
    q4k_unpack_scales(blk + 4, sc, mn);
    for (int t = 0; t < 4; t++) {
      /* hadd_epi16 (wrapping i16) then madd_epi16 */
      int16_t s0 = (int16_t)(q8k[i].bsums[4 * t] + q8k[i].bsums[4 * t + 1]);
      int16_t s1 = (int16_t)(q8k[i].bsums[4 * t + 2] + q8k[i].bsums[4 * t + 3]);
      int32_t prod = (int32_t)mn[2 * t] * s0 + (int32_t)mn[2 * t + 1] * s1;
      acc_m[t] = fmaf(dmin, (float)prod, acc_m[t]);
    }
    int32_t sumi[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < 4; j++) {
      for (int L = 0; L < 8; L++) {
        int32_t lo = 0, hi = 0;
        for (int e = 4 * L; e < 4 * L + 4; e++) {
          uint8_t byte = blk[16 + j * 32 + e];
          lo += (int32_t)(byte & 0xF) * (int32_t)q8k[i].qs[64 * j + e];
          hi += (int32_t)(byte >> 4) * (int32_t)q8k[i].qs[64 * j + 32 + e];
        }
        sumi[L] += (int32_t)sc[2 * j] * lo + (int32_t)sc[2 * j + 1] * hi;
      }
    }
    for (int L = 0; L < 8; L++) acc[L] = fmaf(d, (float)sumi[L], acc[L]);
  }
  float m0 = acc_m[0] + acc_m[2], m1 = acc_m[1] + acc_m[3];
  float min_val = m0 + m1;
  float main_val = hsum8(acc);
  return main_val + min_val;
}

/* src/ops/quant/mod.rs:456-490 */
void orc_dequantize_row_q4_k(const uint8_t* bytes, size_t bytes_len, float* output, size_t n) {
  size_t nb = n / 256;
  for (size_t bi = 0; bi < nb; bi++) {
    size_t off = bi * 144;
    if (off + 144 > bytes_len) break;
    float d = orc_f16_from_bytes(bytes, bytes_len, off);
    float dmin = orc_f16_from_bytes(bytes, bytes_len, off + 2);
    const uint8_t* sb = bytes + off + 4;
    const uint8_t* qs = bytes + off + 16;
    float* o = output + bi * 256;
    int is = 0;
    for (int q_off = 0; q_off < 128; q_off += 32, is += 2) {
      uint8_t sc1, m1, sc2, m2;
      get_scale_min_k4(is, sb, &sc1, &m1);
      get_scale_min_k4(is + 1, sb, &sc2, &m2);
      float d1 = d * (float)sc1, m1e = dmin * (float)m1;
      float d2 = d * (float)sc2, m2e = dmin * (float)m2;
      for (int l = 0; l < 32; l++) {
        uint8_t ql = qs[q_off + l];
        float a = d1 * (float)(ql & 0xF);
        o[q_off * 2 + l] = a - m1e;
        float b = d2 * (float)(ql >> 4);
        o[q_off * 2 + 32 + l] = b - m2e;
      }
    }
  }
}

/* src/ops/quant/mod.rs:492-508 */
void orc_dequantize_q4_k_weight(const uint8_t* bytes, size_t bytes_len, size_t n_rows, size_t n_cols,
                                float* output) {
  size_t row_bytes = n_cols / 256 * 144;
  for (size_t r = 0; r < n_rows; r++)
    orc_dequantize_row_q4_k(bytes + r * row_bytes, bytes_len - r * row_bytes, output + r * n_cols,
                            n_cols);
}

/* src/core/model.rs:65-85 */
void orc_q4k_forward_dequant(const uint8_t* weight, size_t weight_len, size_t out_features,
                             size_t in_features, const float* input, float* output, float* scratch,
                             size_t scratch_len) {
  size_t n_el = out_features * in_features;
  size_t len = n_el < scratch_len ? n_el : scratch_len;
  (void)len; /* the reference truncates silently; callers here always pass a full scratch */
  orc_dequantize_q4_k_weight(weight, weight_len, out_features, in_features, scratch);
  for (size_t i = 0; i < out_features; i++) {
    float sum = 0.0f;
    const float* w = scratch + i * in_features;
    for (size_t j = 0; j < in_features; j++) {
      float t = w[j] * input[j];
      sum = sum + t;
    }
    output[i] = sum;
  }
}

/* src/ops/kernel/q4_k.rs:56-93 */
void orc_q4k_forward_prepared(const uint8_t* weight, size_t weight_len, const float* input_f32,
                              float* output, size_t n_in, size_t n_out, size_t ith, size_t nth,
                              int sem) {
  size_t per = (n_out + nth - 1) / nth;
  size_t s = ith * per, e = s + per < n_out ? s + per : n_out;
  if (s >= e) return;
  size_t nb = n_in / 256;
  orc_block_q8k* q = (orc_block_q8k*)malloc(sizeof(orc_block_q8k) * nb);
  orc_quantize_row_q8_k(input_f32, n_in, q, sem);
  size_t row_bytes = nb * 144;
  (void)weight_len;
  for (size_t r = s; r < e; r++) output[r] = orc_vec_dot_q4k_q8k(weight + r * row_bytes, row_bytes, q, nb, sem);
  free(q);
}

/* src/ops/kernel/q4_k.rs:20-54 */
void orc_q4k_forward_prequantized(const uint8_t* weight, size_t weight_len, const uint8_t* input_q8,
                                  const float* input_scales, float* output, size_t n_in,
                                  size_t n_out, size_t ith, size_t nth) {
  size_t per = (n_out + nth - 1) / nth;
  size_t s = ith * per, e = s + per < n_out ? s + per : n_out;
  if (s >= e) return;
  float* in = (float*)malloc(sizeof(float) * n_in);
  float* row = (float*)malloc(sizeof(float) * n_in);
  for (size_t i = 0; i < n_in; i++) in[i] = (float)(int8_t)input_q8[i] * input_scales[i / 32];
  size_t row_bytes = n_in / 256 * 144;
  (void)weight_len;
  for (size_t r = s; r < e; r++) {
    orc_dequantize_row_q4_k(weight + r * row_bytes, row_bytes, row, n_in);
    float sum = 0.0f; /* Iterator::sum::<f32>() folds from 0.0 in order */
    for (size_t i = 0; i < n_in; i++) {
      float t = row[i] * in[i];
      sum = sum + t;
    }
    output[r] = sum;
  }
  free(in);
  free(row);
}

/* ------------------------------------------------------------------ Q4_0 */

void orc_q4_0_forward_prequantized(const uint8_t* weight, const uint8_t* input_q8, const float* input_scales,
                                   float* output, size_t n_in, size_t n_out, size_t ith, size_t nth) {
  size_t n_blocks = n_in / 32, row_stride = n_blocks * 18;
  size_t per = (n_out + nth - 1) / nth;
  size_t s = ith * per, e = s + per < n_out ? s + per : n_out;
  if (s >= e) return;
  for (size_t r = s; r < e; r++) {
    float sum = 0.0f;
    for (size_t b = 0; b < n_blocks; b++) {
      const uint8_t* blk = weight + r * row_stride + b * 18;
      float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
      int32_t dot = 0;
      for (int l = 0; l < 16; l++) {
        int x0 = (blk[2 + l] & 0x0F) - 8, x1 = (blk[2 + l] >> 4) - 8;
        dot += x0 * (int32_t)(int8_t)input_q8[b * 32 + l] + x1 * (int32_t)(int8_t)input_q8[b * 32 + 16 + l];
      }
      float t = (float)dot * d;
      t = t * input_scales[b];
      sum = sum + t;
    }
    output[r] = sum;
  }
}

void orc_embedding_lookup_q4_0(const uint8_t* weight, uint32_t token, size_t n_embd, float* out) {
  size_t bpr = n_embd / 32;
  const uint8_t* row = weight + (size_t)token * bpr * 18;
  for (size_t b = 0; b < bpr; b++) {
    const uint8_t* blk = row + b * 18;
    float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
    for (int j = 0; j < 16; j++) {
      float a = (float)(blk[2 + j] & 0x0F) - 8.0f, h = (float)(blk[2 + j] >> 4) - 8.0f;
      out[b * 32 + j] = a * d;
      out[b * 32 + j + 16] = h * d;
    }
  }
}

/* ------------------------------------------------------------------ Q6_K */

/* the 6-bit value (0..63) at position e (0..255) of a super-block: mod.rs:542-555 */
static inline int q6k_value(const uint8_t* blk, int e) {
  const int j = e / 128, r = e % 128, k = r / 32, l = r % 32;
  const uint8_t* ql = blk + j * 64;
  const uint8_t qh = blk[128 + j * 32 + l];
  int lo, hi;
  switch (k) {
    case 0: lo = ql[l] & 0xF; hi = qh & 3; break;
    case 1: lo = ql[l + 32] & 0xF; hi = (qh >> 2) & 3; break;
    case 2: lo = ql[l] >> 4; hi = (qh >> 4) & 3; break;
    default: lo = ql[l + 32] >> 4; hi = (qh >> 6) & 3; break;
  }
  return lo | (hi << 4);
}

void orc_dequantize_row_q6_k(const uint8_t* bytes, size_t bytes_len, float* output, size_t n) {
  size_t nb = n / 256;
  for (size_t b = 0; b < nb; b++) {
    if ((b + 1) * 210 > bytes_len) break;
    const uint8_t* blk = bytes + b * 210;
    float d = orc_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
    for (int e = 0; e < 256; e++) {
      /* scale index: j128*8 + is + {0,2,4,6} with is = l/16  ==  e/16 */
      float sc = (float)(int8_t)blk[192 + e / 16];
      int q = q6k_value(blk, e) - 32;
      float ds = d * sc;
      output[b * 256 + e] = ds * (float)q;
    }
  }
}

void orc_q6k_q8k_block_lanes(const uint8_t* blk, const orc_block_q8k* q8k, int32_t lanes[8]) {
  /* mod.rs:998-1062.  Vector (j, k) covers positions 128j + 32k .. +31; int32 lane L of the madd result
   * covers its bytes 4L..4L+3, bytes 0..15 scaled by scales[8j+2k], bytes 16..31 by scales[8j+2k+1]. */
  const int8_t* sc = (const int8_t*)(blk + 192);
  for (int L = 0; L < 8; L++) {
    int32_t s = 0;
    for (int v = 0; v < 8; v++) {
      int base = 32 * v + 4 * L;
      int32_t p = 0;
      for (int t = 0; t < 4; t++) p += q6k_value(blk, base + t) * (int32_t)q8k->qs[base + t];
      s += (int32_t)sc[2 * v + (L >= 4)] * p;
    }
    int32_t sub = ((int32_t)q8k->bsums[2 * L] * sc[2 * L] + (int32_t)q8k->bsums[2 * L + 1] * sc[2 * L + 1]) * 32;
    lanes[L] = s - sub;
  }
}

float orc_vec_dot_q6k_q8k(const uint8_t* q6k, size_t q6k_len, const orc_block_q8k* q8k, size_t nb, int sem) {
  if (sem == ORC_SEM_SCALAR) {
    /* mod.rs:640-692 */
    float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (size_t i = 0; i < nb; i++) {
      if ((i + 1) * 210 > q6k_len) break;
      const uint8_t* blk = q6k + i * 210;
      int32_t aux32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int g = 0; g < 16; g++) {
        int32_t scale = (int8_t)blk[192 + g];
        for (int t = 0; t < 16; t++) {
          int e = 16 * g + t;
          aux32[t % 8] += scale * (int32_t)q8k[i].qs[e] * (q6k_value(blk, e) - 32);
        }
      }
      float d = orc_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8))) * q8k[i].d;
      for (int l = 0; l < 8; l++) {
        float t = d * (float)aux32[l];
        sums[l] = sums[l] + t;
      }
    }
    float sumf = 0.0f;
    for (int l = 0; l < 8; l++) sumf = sumf + sums[l];
    return sumf;
  }
  /* AVX2, mod.rs:964-1064: eight f32 lanes, one FMA per super-block, hsum_ps at the end */
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t i = 0; i < nb; i++) {
    if ((i + 1) * 210 > q6k_len) break;
    const uint8_t* blk = q6k + i * 210;
    float d = orc_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8))) * q8k[i].d;
    int32_t lanes[8];
    orc_q6k_q8k_block_lanes(blk, &q8k[i], lanes);
    for (int L = 0; L < 8; L++) acc[L] = fmaf(d, (float)lanes[L], acc[L]);
  }
  return hsum8(acc);
}

void orc_q6k_forward_prepared(const uint8_t* weight, size_t weight_len, const float* input_f32, float* output,
                              size_t n_in, size_t n_out, size_t ith, size_t nth, int sem) {
  size_t per = (n_out + nth - 1) / nth;
  size_t s = ith * per, e = s + per < n_out ? s + per : n_out;
  if (s >= e) return;
  size_t nb = n_in / 256;
  orc_block_q8k* q = (orc_block_q8k*)malloc(sizeof(orc_block_q8k) * nb);
  orc_quantize_row_q8_k(input_f32, n_in, q, sem);
  size_t row_bytes = nb * 210;
  (void)weight_len;
  for (size_t r = s; r < e; r++) output[r] = orc_vec_dot_q6k_q8k(weight + r * row_bytes, row_bytes, q, nb, sem);
  free(q);
}

void orc_q6k_forward_prequantized(const uint8_t* weight, size_t weight_len, const uint8_t* input_q8,
                                  const float* input_scales, float* output, size_t n_in, size_t n_out,
                                  size_t ith, size_t nth) {
  size_t per = (n_out + nth - 1) / nth;
  size_t s = ith * per, e = s + per < n_out ? s + per : n_out;
  if (s >= e) return;
  float* in = (float*)malloc(sizeof(float) * n_in);
  float* row = (float*)malloc(sizeof(float) * n_in);
  for (size_t i = 0; i < n_in; i++) in[i] = (float)(int8_t)input_q8[i] * input_scales[i / 32];
  size_t row_bytes = n_in / 256 * 210;
  (void)weight_len;
  for (size_t r = s; r < e; r++) {
    orc_dequantize_row_q6_k(weight + r * row_bytes, row_bytes, row, n_in);
    float sum = 0.0f;
    for (size_t i = 0; i < n_in; i++) {
      float t = row[i] * in[i];
      sum = sum + t;
    }
    output[r] = sum;
  }
  free(in);
  free(row);
}

/* ------------------------------------------------------------------ element-wise ops */

/* src/ops/norm.rs:3-11 */
void orc_rms_norm(const float* input, const float* weight, float* output, size_t n, float eps) {
  double sum_sq = 0.0;
  for (size_t i = 0; i < n; i++) {
    float p = input[i] * input[i];
    sum_sq += (double)p;
  }
  float mean_sq = (float)(sum_sq / (double)n);
  float scale = 1.0f / sqrtf(mean_sq + eps);
  for (size_t i = 0; i < n; i++) {
    float t = input[i] * scale;
    output[i] = t * weight[i];
  }
}

/* src/ops/norm.rs:13-19 (+ scale_mul_avx2 :66-84: (x*scale)*w, same values as the scalar loop) */
void orc_rms_norm_inplace(float* x, const float* weight, size_t n, float eps) {
  orc_rms_norm(x, weight, x, n, eps);
}

/* src/ops/rope.rs:21-37 */
void orc_rope_table(size_t pos, size_t head_dim, float freq_base, float* table) {
  size_t half = head_dim / 2;
  float theta_scale = powf(freq_base, -2.0f / (float)head_dim);
  float theta = (float)pos;
  for (size_t i = 0; i < half; i++) {
    table[2 * i] = cosf(theta);
    table[2 * i + 1] = sinf(theta);
    theta = theta * theta_scale;
  }
}

void orc_rope_neox(float* x, size_t len, size_t pos, size_t head_dim, float freq_base) {
  size_t half = head_dim / 2, n_heads = len / head_dim;
  float table[2 * 512];
  if (half > 512) return;
  orc_rope_table(pos, head_dim, freq_base, table);
  for (size_t h = 0; h < n_heads; h++) {
    float* p = x + h * head_dim;
    for (size_t i = 0; i < half; i++) {
      float c = table[2 * i], s = table[2 * i + 1];
      float x0 = p[i], x1 = p[i + half];
      p[i] = fmaf(x0, c, x1 * -s);
      p[i + half] = fmaf(x0, s, x1 * c);
    }
  }
}

/* src/ops/attention.rs:28-38 */
void orc_softmax(float* x, size_t n) {
  if (n == 0) return;
  float max_val = -INFINITY;
  for (size_t i = 0; i < n; i++) max_val = x[i] > max_val ? x[i] : max_val; /* f32::max */
  float sum = 0.0f;
  for (size_t i = 0; i < n; i++) {
    x[i] = orc_expf(x[i] - max_val);
    sum = sum + x[i];
  }
  if (sum > 0.0f)
    for (size_t i = 0; i < n; i++) x[i] = x[i] / sum;
}

/* src/ops/dot.rs:99-119 */
float orc_dot_f16(const uint16_t* a, const uint16_t* b, size_t n) {
  double sum = 0.0;
  for (size_t i = 0; i < n; i++) {
    float p = orc_f16_to_f32(a[i]) * orc_f16_to_f32(b[i]);
    sum += (double)p;
  }
  return (float)sum;
}

/* src/ops/embedding.rs:12-22 */
void orc_embedding_lookup_q8_0(const uint8_t* weight, uint32_t token, size_t n_embd, float* out) {
  size_t blocks = n_embd / 32;
  const uint8_t* row = weight + (size_t)token * blocks * 34;
  for (size_t b = 0; b < blocks; b++) {
    float d = wd_of(row + b * 34);
    for (int j = 0; j < 32; j++) out[b * 32 + j] = d * (float)(int8_t)row[b * 34 + 2 + j];
  }
}

/* src/models/qwen3.rs:172-191 */
int64_t orc_greedy_token(const float* logits, size_t n) {
  if (n == 0 || !isfinite(logits[0])) return -1;
  size_t best_id = 0;
  float best = logits[0];
  for (size_t i = 1; i < n; i++) {
    if (!isfinite(logits[i])) return -1;
    if (logits[i] > best) {
      best = logits[i];
      best_id = i;
    }
  }
  return (int64_t)best_id;
}

/* ------------------------------------------------------------------ Qwen3 decode */

typedef struct {
  const orc_qwen3_model* m;
  size_t layer, step, capacity;
  float* q;
  float* attn_out;
  uint16_t *k_cache, *v_cache;
  float* scores;       /* [nth][2*score_stride] (second half reused as f16 scratch) */
  size_t score_stride;
  int sem;
  const float *k32, *v32; /* F32 KV caches of the CLI forward (NULL otherwise) */
} attn_job;

static void attn_job_fn(void* p, size_t ith, size_t nth) {
  /* src/models/qwen3.rs:876-933 */
  attn_job* j = (attn_job*)p;
  const orc_qwen3_config* c = &j->m->cfg;
  size_t hd = c->head_dim, kv_stride = c->n_head_kv * hd;
  size_t group = c->n_head / c->n_head_kv;
  float kq_scale = 1.0f / sqrtf((float)hd);
  size_t h0 = ith * c->n_head / nth, h1 = (ith + 1) * c->n_head / nth;
  size_t layer_base = j->layer * j->capacity * kv_stride;
  size_t step = j->step;
  size_t n_padded = (step + 1 + 255) / 256 * 256;
  float* scores = j->scores + ith * 2 * j->score_stride;
  uint16_t* w16 = (uint16_t*)(scores + j->score_stride);
  uint16_t* v16 = w16 + j->score_stride;
  uint16_t q16[1024];
  for (size_t head = h0; head < h1; head++) {
    size_t kvh = head / group;
    orc_f32_slice_to_f16(j->q + head * hd, q16, hd);
    for (size_t t = 0; t < n_padded; t++) scores[t] = -INFINITY;
    for (size_t t = 0; t <= step; t++) {
      const uint16_t* key = j->k_cache + layer_base + t * kv_stride + kvh * hd;
      scores[t] = orc_dot_f16(q16, key, hd) * kq_scale;
    }
    orc_softmax(scores, n_padded);
    for (size_t t = 0; t < n_padded; t++) w16[t] = orc_f32_to_f16(scores[t]);
    for (size_t t = step + 1; t < n_padded; t++) v16[t] = 0;
    float* out = j->attn_out + head * hd;
    for (size_t d = 0; d < hd; d++) {
      for (size_t t = 0; t <= step; t++) v16[t] = j->v_cache[layer_base + t * kv_stride + kvh * hd + d];
      out[d] = orc_dot_f16(v16, w16, n_padded);
    }
  }
}

/* src/ops/dot.rs:79-97, :241-276: f32 x f16 dot in the order of the selected instruction set */
float orc_dot_f16_f32(const float* a, const uint16_t* b, size_t n, int sem) {
  if (sem == ORC_SEM_AVX2) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
      for (int l = 0; l < 8; l++) acc[l] = fmaf(a[i + l], orc_f16_to_f32(b[i + l]), acc[l]);
    float sum = hsum8(acc);
    for (; i < n; i++) {
      float t = a[i] * orc_f16_to_f32(b[i]);
      sum = sum + t;
    }
    return sum;
  }
  if (sem == ORC_SEM_NEON) {
    float acc[4] = {0, 0, 0, 0};
    size_t i = 0;
    for (; i + 4 <= n; i += 4)
      for (int l = 0; l < 4; l++) acc[l] = fmaf(a[i + l], orc_f16_to_f32(b[i + l]), acc[l]);
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]); /* vaddvq_f32 */
    for (; i < n; i++) {
      float t = a[i] * orc_f16_to_f32(b[i]);
      sum = sum + t;
    }
    return sum;
  }
  float s = 0.0f;
  for (size_t i = 0; i < n; i++) {
    float t = a[i] * orc_f16_to_f32(b[i]);
    s = s + t;
  }
  return s;
}

/* src/ops/dot.rs:278-345: y += v * f16(x): fused on AVX2 and NEON, separate multiply and add in the scalar path */
void orc_vec_mad_f16_f32(float* y, const uint16_t* x, float v, size_t n, int sem) {
  for (size_t i = 0; i < n; i++) {
    if (sem == ORC_SEM_SCALAR) {
      float t = v * orc_f16_to_f32(x[i]);
      y[i] = y[i] + t;
    } else {
      y[i] = fmaf(v, orc_f16_to_f32(x[i]), y[i]);
    }
  }
}

static void attn_cli_job_fn(void* p, size_t ith, size_t nth) {
  /* src/app/text.rs:414-453: online soft-max over the cached positions, f32 query, F16 cache */
  attn_job* j = (attn_job*)p;
  const orc_qwen3_config* c = &j->m->cfg;
  size_t hd = c->head_dim, kv_stride = c->n_head_kv * hd;
  size_t group = c->n_head / c->n_head_kv;
  float kq_scale = 1.0f / sqrtf((float)hd);
  size_t h0 = ith * c->n_head / nth, h1 = (ith + 1) * c->n_head / nth;
  size_t layer_base = j->layer * j->capacity * kv_stride;
  for (size_t head = h0; head < h1; head++) {
    size_t kvh = head / group;
    float* out = j->attn_out + head * hd;
    float ms = 0.0f, s_sum = 0.0f;
    for (size_t d = 0; d < hd; d++) out[d] = 0.0f;
    for (size_t t = 0; t <= j->step; t++) {
      const uint16_t* key = j->k_cache + layer_base + t * kv_stride + kvh * hd;
      float score = orc_dot_f16_f32(j->q + head * hd, key, hd, j->sem) * kq_scale;
      if (score > ms) {
        float rescale = orc_expf(ms - score);
        for (size_t d = 0; d < hd; d++) out[d] = out[d] * rescale;
        s_sum = s_sum * rescale;
        ms = score;
      }
      float vs = orc_expf(score - ms);
      orc_vec_mad_f16_f32(out, j->v_cache + layer_base + t * kv_stride + kvh * hd, vs, hd, j->sem);
      s_sum = s_sum + vs;
    }
    float inv_sum = 1.0f / s_sum;
    for (size_t d = 0; d < hd; d++) out[d] = out[d] * inv_sum;
  }
}

/* src/ops/dot.rs:8-76: f32 x f32 dot in the order of the selected instruction set */
float orc_dot_f32(const float* a, const float* b, size_t n, int sem) {
  if (sem == ORC_SEM_AVX2) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
      for (int l = 0; l < 8; l++) acc[l] = fmaf(a[i + l], b[i + l], acc[l]);
    float sum = hsum8(acc);
    for (; i < n; i++) {
      float t = a[i] * b[i];
      sum = sum + t;
    }
    return sum;
  }
  if (sem == ORC_SEM_NEON) {
    float acc[16] = {0}; /* acc0..acc3, four lanes each */
    size_t i = 0;
    for (; i + 16 <= n; i += 16)
      for (int l = 0; l < 16; l++) acc[l] = fmaf(a[i + l], b[i + l], acc[l]);
    float c[4];
    for (int l = 0; l < 4; l++) {
      float c0 = acc[l] + acc[8 + l], c1 = acc[4 + l] + acc[12 + l]; /* acc0+acc2, acc1+acc3 */
      c[l] = c0 + c1;
    }
    float sum = (c[0] + c[1]) + (c[2] + c[3]); /* vaddvq_f32 */
    for (; i < n; i++) {
      float t = a[i] * b[i];
      sum = sum + t;
    }
    return sum;
  }
  float s = 0.0f;
  for (size_t i = 0; i < n; i++) {
    float t = a[i] * b[i];
    s = s + t;
  }
  return s;
}

static void attn_cli_f32_job_fn(void* p, size_t ith, size_t nth) {
  /* src/app/text.rs:458-496: F32 cache: scores padded with -inf to a multiple of 256, soft-max, then one
   * dot over the gathered column of V per output element (a 512-entry stack array in the reference) */
  attn_job* j = (attn_job*)p;
  const orc_qwen3_config* c = &j->m->cfg;
  size_t hd = c->head_dim, kv_stride = c->n_head_kv * hd;
  size_t group = c->n_head / c->n_head_kv;
  float kq_scale = 1.0f / sqrtf((float)hd);
  size_t h0 = ith * c->n_head / nth, h1 = (ith + 1) * c->n_head / nth;
  size_t layer_base = j->layer * j->capacity * kv_stride;
  size_t n_cached = j->step + 1, n_padded = (n_cached + 255) / 256 * 256;
  float* scores = j->scores + ith * 2 * j->score_stride;
  for (size_t head = h0; head < h1; head++) {
    size_t kvh = head / group;
    for (size_t t = 0; t < n_cached; t++)
      scores[t] = orc_dot_f32(j->q + head * hd, j->k32 + layer_base + t * kv_stride + kvh * hd, hd, j->sem) * kq_scale;
    for (size_t t = n_cached; t < n_padded; t++) scores[t] = -INFINITY;
    orc_softmax(scores, n_padded);
    float values[512];
    memset(values, 0, sizeof(values));
    for (size_t d = 0; d < hd; d++) {
      for (size_t t = 0; t < n_cached; t++) values[t] = j->v32[layer_base + t * kv_stride + kvh * hd + d];
      j->attn_out[head * hd + d] = orc_dot_f32(values, scores, n_padded, j->sem);
    }
  }
}

static void attn_logits_job_fn(void* p, size_t ith, size_t nth) {
  /* src/app/logits.rs:474-560: scores (dot_f16_f32 over the F16 cache, dot_f32 over the F32 cache), soft-max
   * over the cached positions, then val += p_t * v_t in position order for every output element */
  attn_job* j = (attn_job*)p;
  const orc_qwen3_config* c = &j->m->cfg;
  size_t hd = c->head_dim, kv_stride = c->n_head_kv * hd;
  size_t group = c->n_head / c->n_head_kv;
  float kq_scale = 1.0f / sqrtf((float)hd);
  size_t h0 = ith * c->n_head / nth, h1 = (ith + 1) * c->n_head / nth;
  size_t layer_base = j->layer * j->capacity * kv_stride;
  size_t n_cached = j->step + 1;
  float* scores = j->scores + ith * 2 * j->score_stride;
  for (size_t head = h0; head < h1; head++) {
    size_t kvh = head / group;
    for (size_t t = 0; t < n_cached; t++) {
      size_t at = layer_base + t * kv_stride + kvh * hd;
      float dot = j->k32 ? orc_dot_f32(j->q + head * hd, j->k32 + at, hd, j->sem)
                         : orc_dot_f16_f32(j->q + head * hd, j->k_cache + at, hd, j->sem);
      scores[t] = dot * kq_scale;
    }
    orc_softmax(scores, n_cached);
    for (size_t d = 0; d < hd; d++) {
      float val = 0.0f;
      for (size_t t = 0; t < n_cached; t++) {
        size_t at = layer_base + t * kv_stride + kvh * hd + d;
        float prod = scores[t] * (j->v32 ? j->v32[at] : orc_f16_to_f32(j->v_cache[at]));
        val = val + prod;
      }
      j->attn_out[head * hd + d] = val;
    }
  }
}

/* Iterator::max_by(partial_cmp): the last maximal index (src/app/text.rs:664-670); -1 on NaN (the reference panics) */
int64_t orc_greedy_token_last(const float* logits, size_t n) {
  if (n == 0) return 0;
  size_t best = 0;
  for (size_t i = 0; i < n; i++) {
    if (isnan(logits[i])) return -1;
    if (i > 0 && logits[i] >= logits[best]) best = i;
  }
  return (int64_t)best;
}

typedef struct {
  const orc_qwen3_layer* w;
  const uint8_t* q8;
  const float* xs;
  float *q, *k, *v;
  size_t n_embd, nq, nk;
  int sem;
} qkv_job;
static void qkv_job_fn(void* p, size_t ith, size_t nth) {
  /* src/models/qwen3.rs:738-774 */
  qkv_job* j = (qkv_job*)p;
  gemv_rows(j->w->wq, j->q8, j->xs, j->q, j->n_embd, j->nq, ith, nth, j->sem);
  gemv_rows(j->w->wk, j->q8, j->xs, j->k, j->n_embd, j->nk, ith, nth, j->sem);
  gemv_rows(j->w->wv, j->q8, j->xs, j->v, j->n_embd, j->nk, ith, nth, j->sem);
}

static int64_t qwen3_generate_variant(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                                      size_t n_gen, uint32_t* out_tokens, int sem, int threads, float* trace,
                                      float* logits_last, int cli);

int64_t orc_qwen3_generate(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                           size_t n_gen, uint32_t* out_tokens, int sem, int threads, float* trace,
                           float* logits_last) {
  return qwen3_generate_variant(model, prompt, n_prompt, n_gen, out_tokens, sem, threads, trace, logits_last, 0);
}

int64_t orc_qwen3_generate_cli(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                               size_t n_gen, uint32_t* out_tokens, int sem, int threads, float* trace,
                               float* logits_last) {
  return qwen3_generate_variant(model, prompt, n_prompt, n_gen, out_tokens, sem, threads, trace, logits_last, 1);
}

/* the same loop with `--kv-cache f32` (src/app/text.rs:183-186, :393-405, :458-496); -2 when the context is
 * longer than the 512 positions the reference's stack array holds (it panics there) */
int64_t orc_qwen3_generate_cli_f32kv(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                                     size_t n_gen, uint32_t* out_tokens, int sem, int threads, float* trace,
                                     float* logits_last) {
  if ((n_prompt + n_gen + 255) / 256 * 256 > 512) return -2;
  return qwen3_generate_variant(model, prompt, n_prompt, n_gen, out_tokens, sem, threads, trace, logits_last, 2);
}

/* the logits tool's copy of the loop (src/app/logits.rs:255-700) over the F16 (kv_f32 = 0) or F32 cache */
int64_t orc_qwen3_generate_logits_tool(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                                       size_t n_gen, uint32_t* out_tokens, int sem, int threads, float* trace,
                                       float* logits_last, int kv_f32) {
  return qwen3_generate_variant(model, prompt, n_prompt, n_gen, out_tokens, sem, threads, trace, logits_last,
                                kv_f32 ? 4 : 3);
}

static int64_t qwen3_generate_variant(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                                      size_t n_gen, uint32_t* out_tokens, int sem, int threads, float* trace,
                                      float* logits_last, int cli) {
  /* src/models/qwen3.rs:440-550 (session buffers), :581-1158 (step loop) */
  const orc_qwen3_config* c = &model->cfg;
  size_t hd = c->head_dim, nq = c->n_head * hd, nk = c->n_head_kv * hd, n_attn = nq;
  size_t kv_stride = nk;
  size_t capacity = n_prompt + n_gen;
  if (capacity == 0 || n_prompt == 0) return 0;
  size_t steps = capacity - 1; /* qwen3.rs:118-126 checked_decoder_steps */
  size_t max_n_in = nq > c->n_ff ? nq : c->n_ff;
  size_t score_stride = (capacity + 255) / 256 * 256;
  if (threads < 1) threads = 1;

  uint16_t* k_cache = (uint16_t*)calloc(c->n_layer * capacity * kv_stride, 2);
  uint16_t* v_cache = (uint16_t*)calloc(c->n_layer * capacity * kv_stride, 2);
  float* x = (float*)calloc(c->n_embd, 4);
  float* normed = (float*)calloc(c->n_embd, 4);
  float* q = (float*)calloc(nq, 4);
  float* k = (float*)calloc(nk, 4);
  float* v = (float*)calloc(nk, 4);
  float* attn_out = (float*)calloc(n_attn, 4);
  float* proj = (float*)calloc(c->n_embd, 4);
  float* gate = (float*)calloc(c->n_ff, 4);
  float* up = (float*)calloc(c->n_ff, 4);
  float* logits = (float*)calloc(c->vocab, 4);
  uint8_t* q8 = (uint8_t*)calloc(max_n_in, 1);
  float* xs = (float*)calloc(max_n_in / 32 + 1, 4);
  float* scores = (float*)calloc((size_t)threads * 2 * score_stride, 4);
  float* k32 = (cli == 2 || cli == 4) ? (float*)calloc(c->n_layer * capacity * kv_stride, 4) : NULL;
  float* v32 = (cli == 2 || cli == 4) ? (float*)calloc(c->n_layer * capacity * kv_stride, 4) : NULL;

  int64_t n_out = 0;
  int failed = 0;
  for (size_t step = 0; step < steps && !failed; step++) {
    size_t pos = step; /* positions are 0..n_prompt-1, then last+1+i (qwen3.rs:128-141) */
    uint32_t tok = step < n_prompt ? prompt[step] : out_tokens[n_out - 1];
    orc_embedding_lookup_q8_0(model->token_embd, tok, c->n_embd, x);
    for (size_t layer = 0; layer < c->n_layer; layer++) {
      const orc_qwen3_layer* w = &model->layers[layer];
      orc_rms_norm(x, w->attn_norm, normed, c->n_embd, c->eps);
      quantize_any(normed, c->n_embd, q8, xs, sem);
      qkv_job qj = {w, q8, xs, q, k, v, c->n_embd, nq, nk, sem};
      orc_compute(threads, qkv_job_fn, &qj);
      if (w->q_norm && w->k_norm) {
        for (size_t h = 0; h < c->n_head; h++) orc_rms_norm_inplace(q + h * hd, w->q_norm, hd, c->eps);
        for (size_t h = 0; h < c->n_head_kv; h++) orc_rms_norm_inplace(k + h * hd, w->k_norm, hd, c->eps);
      }
      orc_rope_neox(q, nq, pos, hd, c->freq_base);
      orc_rope_neox(k, nk, pos, hd, c->freq_base);
      size_t row = layer * capacity * kv_stride + step * kv_stride;
      if (k32) {
        memcpy(k32 + row, k, 4 * nk);
        memcpy(v32 + row, v, 4 * nk);
      } else {
        orc_f32_slice_to_f16(k, k_cache + row, nk);
        orc_f32_slice_to_f16(v, v_cache + row, nk);
      }
      attn_job aj = {model, layer, step, capacity, q, attn_out, k_cache, v_cache, scores, score_stride, sem, k32, v32};
      orc_compute(threads, cli >= 3 ? attn_logits_job_fn : (cli == 2 ? attn_cli_f32_job_fn : (cli ? attn_cli_job_fn : attn_job_fn)), &aj);
      quantize_any(attn_out, n_attn, q8, xs, sem);
      pooled_gemv(w->wo, q8, xs, proj, n_attn, c->n_embd, sem, threads);
      for (size_t i = 0; i < c->n_embd; i++) x[i] = x[i] + proj[i];
      orc_rms_norm(x, w->ffn_norm, normed, c->n_embd, c->eps);
      quantize_any(normed, c->n_embd, q8, xs, sem);
      ffn_job fj = {w->w_gate, w->w_up, q8, xs, gate, up, c->n_embd, c->n_ff, sem};
      orc_compute(threads, ffn_job_fn, &fj);
      orc_silu_mul_inplace(gate, up, c->n_ff);
      quantize_any(up, c->n_ff, q8, xs, sem);
      pooled_gemv(w->w_down, q8, xs, proj, c->n_ff, c->n_embd, sem, threads);
      for (size_t i = 0; i < c->n_embd; i++) x[i] = x[i] + proj[i];
    }
    if (trace) memcpy(trace + step * c->n_embd, x, 4 * c->n_embd);
    if (step + 1 < n_prompt && !(logits_last && step == steps - 1)) continue; /* logits unused */
    orc_rms_norm(x, model->output_norm, normed, c->n_embd, c->eps);
    quantize_any(normed, c->n_embd, q8, xs, sem);
    pooled_gemv(model->output, q8, xs, logits, c->n_embd, c->vocab, sem, threads);
    if (step + 1 < n_prompt) continue;
    /* text loop: last maximal index; Qwen3Session and the logits tool (src/app/logits.rs:766-773): the first */
    int64_t t = (cli == 1 || cli == 2) ? orc_greedy_token_last(logits, c->vocab) : orc_greedy_token(logits, c->vocab);
    if (t < 0) {
      failed = 1;
      break;
    }
    if ((size_t)n_out >= n_gen) break;
    out_tokens[n_out++] = (uint32_t)t;
  }
  if (logits_last) memcpy(logits_last, logits, 4 * c->vocab);
  free(k_cache); free(v_cache); free(x); free(normed); free(q); free(k); free(v);
  free(attn_out); free(proj); free(gate); free(up); free(logits); free(q8); free(xs); free(scores);
  free(k32); free(v32);
  return failed ? -1 : n_out;
}

void orc_embedding_lookup_q6_k(const uint8_t* weight, uint32_t token, size_t n_embd, float* out) {
  size_t row_bytes = n_embd / 256 * 210;
  orc_dequantize_row_q6_k(weight + (size_t)token * row_bytes, row_bytes, out, n_embd);
}
