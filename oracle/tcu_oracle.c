/*
 * tcu_oracle.c -- CPU oracle and timed CPU baseline.  TEST INFRASTRUCTURE ONLY;
 * see tcu_oracle.h for what it restates and why parity is "unpinned".
 *
 * Build: make -C oracle   (gcc -O3 -mf16c -fopenmp -shared)
 */
#define _GNU_SOURCE
#include "tcu_oracle.h"

#include <math.h>
#include <sched.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ fp16 */

uint16_t tcu_oracle_f64_to_f16(double x) {
  uint64_t b;
  memcpy(&b, &x, 8);
  const uint16_t sign = (uint16_t)((b >> 48) & 0x8000u);
  const int exp       = (int)((b >> 52) & 0x7ff);
  uint64_t man        = b & ((1ull << 52) - 1);
  if (exp == 0x7ff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0u));
  if (exp == 0) return sign; /* double subnormals are far below half's range */
  const int e = exp - 1023;
  if (e > 15) return (uint16_t)(sign | 0x7c00u);
  man |= 1ull << 52;
  int shift = 42; /* keep 1+10 significand bits */
  int hexp  = e + 15;
  if (e < -14) { /* half subnormal: fixed exponent, fewer bits */
    shift += -14 - e;
    hexp = 0;
  }
  if (shift > 63) return sign;
  uint64_t q          = man >> shift;
  const uint64_t rem  = man & ((1ull << shift) - 1);
  const uint64_t half = 1ull << (shift - 1);
  if (rem > half || (rem == half && (q & 1))) q++;
  uint32_t bits;
  if (hexp == 0) {
    bits = (uint32_t)q; /* q == 0x400 encodes the smallest normal on its own */
  } else {
    if (q == (1ull << 11)) { /* carried into the next binade */
      q >>= 1;
      hexp++;
    }
    if (hexp >= 31) return (uint16_t)(sign | 0x7c00u);
    bits = ((uint32_t)hexp << 10) | (uint32_t)(q & 0x3ff);
  }
  return (uint16_t)(sign | bits);
}

uint16_t tcu_oracle_f32_to_f16(float x) {
  return tcu_oracle_f64_to_f16((double)x); /* float -> double is exact */
}

double tcu_oracle_f16_to_f64(uint16_t h) {
  const int sign = h >> 15;
  const int exp  = (h >> 10) & 0x1f;
  const int man  = h & 0x3ff;
  double v;
  if (exp == 0)
    v = ldexp((double)man, -24);
  else if (exp == 31)
    v = man ? NAN : INFINITY;
  else
    v = ldexp((double)(man | 0x400), exp - 25);
  return sign ? -v : v;
}

/* ------------------------------------------------------------- generator */

static inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

uint64_t tcu_oracle_hash(uint64_t seed, uint64_t index) {
  return splitmix64(splitmix64(seed) + index);
}

static inline float dist_value(uint64_t h, int dist) {
  const uint32_t u24 = (uint32_t)(h >> 40);
  switch (dist) {
    case TCU_DIST_UNIFORM_PM1: return (float)((int32_t)u24 - (1 << 23)) * 0x1p-23f;
    case TCU_DIST_UNIFORM_01: return (float)u24 * 0x1p-24f;
    case TCU_DIST_SMALL_INT: return (float)((int32_t)(u24 % 5u) - 2);
    default: return 0.001f;
  }
}

void tcu_oracle_fill_f16(uint16_t *out, size_t n, uint64_t seed, uint64_t first_index,
                         int dist) {
  const uint64_t key = splitmix64(seed);
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++)
    out[i] = tcu_oracle_f32_to_f16(dist_value(splitmix64(key + first_index + i), dist));
}

/* ---------------------------------------------------------------- oracle */

void tcu_oracle_segmented_reduce(const uint16_t *in, double *out, size_t num_segments,
                                 size_t segment_size) {
#pragma omp parallel for schedule(static)
  for (size_t j = 0; j < num_segments; j++) {
    double acc        = 0.0;
    const uint16_t *p = in + j * segment_size;
    for (size_t i = 0; i < segment_size; i++) acc += tcu_oracle_f16_to_f64(p[i]);
    out[j] = acc;
  }
}

void tcu_oracle_segmented_scan(const uint16_t *in, double *out, size_t num_segments,
                               size_t segment_size) {
#pragma omp parallel for schedule(static)
  for (size_t j = 0; j < num_segments; j++) {
    double acc        = 0.0;
    const uint16_t *p = in + j * segment_size;
    double *o         = out + j * segment_size;
    for (size_t i = 0; i < segment_size; i++) {
      acc += tcu_oracle_f16_to_f64(p[i]);
      o[i] = acc;
    }
  }
}

void tcu_oracle_tile256_scan_algebra(const uint16_t *in, double *out) {
  double A[16][16], AU[16][16], LA[16][16];
  for (int i = 0; i < 16; i++)
    for (int j = 0; j < 16; j++) A[i][j] = tcu_oracle_f16_to_f64(in[i * 16 + j]);
  for (int i = 0; i < 16; i++)
    for (int j = 0; j < 16; j++) {
      double au = 0.0, la = 0.0;
      for (int k = 0; k < 16; k++) {
        if (k <= j) au += A[i][k]; /* U[k][j] = 1 for k <= j */
        if (k < i) la += A[k][j];  /* L[i][k] = 1 for k <  i */
      }
      AU[i][j] = au;
      LA[i][j] = la;
    }
  for (int i = 0; i < 16; i++) {
    double carry = 0.0; /* (L.A).1 : every column of row i gets the row sum of L.A */
    for (int k = 0; k < 16; k++) carry += LA[i][k];
    for (int j = 0; j < 16; j++) out[i * 16 + j] = AU[i][j] + carry;
  }
}

/* ---------------------------------------------------------------- checks */

size_t tcu_oracle_check_f32(const float *got, const double *ref, size_t n, double rel,
                            double abs_floor, double *max_abs_err, double *max_rel_err) {
  size_t bad = 0;
  double ma = 0.0, mr = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : bad) reduction(max : ma, mr)
  for (size_t i = 0; i < n; i++) {
    const double g = (double)got[i];
    if (!(g == g) || isinf(g)) {
      bad++;
      continue;
    }
    const double err = fabs(g - ref[i]);
    const double tol = fmax(rel * fabs(ref[i]), abs_floor);
    if (err > tol) bad++;
    if (err > ma) ma = err;
    if (fabs(ref[i]) > abs_floor) {
      const double r = err / fabs(ref[i]);
      if (r > mr) mr = r;
    }
  }
  if (max_abs_err) *max_abs_err = ma;
  if (max_rel_err) *max_rel_err = mr;
  return bad;
}

static inline int half_order_key(uint16_t h) {
  const int mag = h & 0x7fff;
  return (h & 0x8000) ? -mag : mag;
}

size_t tcu_oracle_check_f16(const uint16_t *got, const double *ref, size_t n, int max_ulp,
                            int *worst_ulp) {
  size_t bad = 0;
  int worst  = 0;
#pragma omp parallel for schedule(static) reduction(+ : bad) reduction(max : worst)
  for (size_t i = 0; i < n; i++) {
    const uint16_t g = got[i];
    if ((g & 0x7c00) == 0x7c00 && (g & 0x3ff)) { /* NaN never matches */
      bad++;
      continue;
    }
    const uint16_t r = tcu_oracle_f64_to_f16(ref[i]);
    int d            = half_order_key(g) - half_order_key(r);
    if (d < 0) d = -d;
    if (d > max_ulp) bad++;
    if (d > worst) worst = d;
  }
  if (worst_ulp) *worst_ulp = worst;
  return bad;
}

/* ---------------------------------------------------------- CPU baseline */

int tcu_cpu_available_cores(void) {
  cpu_set_t set;
  CPU_ZERO(&set);
  if (sched_getaffinity(0, sizeof(set), &set) == 0) {
    const int c = CPU_COUNT(&set);
    if (c > 0) return c;
  }
  return 1;
}

static int pick_threads(int threads) {
  return threads > 0 ? threads : tcu_cpu_available_cores();
}

static inline float h2f(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}

static inline uint16_t f2h(float f) {
  const _Float16 v = (_Float16)f;
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}

int tcu_cpu_segmented_reduce(const uint16_t *in, float *out, size_t num_segments,
                             size_t segment_size, int threads) {
  const int t = pick_threads(threads);
#pragma omp parallel for schedule(static) num_threads(t)
  for (size_t j = 0; j < num_segments; j++) {
    const uint16_t *p = in + j * segment_size;
    float acc[8]      = {0, 0, 0, 0, 0, 0, 0, 0}; /* 8 lanes: vectorises, bounds error */
    for (size_t i = 0; i < segment_size; i += 8)
      for (int l = 0; l < 8; l++) acc[l] += h2f(p[i + l]);
    out[j] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
  }
  return t;
}

int tcu_cpu_segmented_scan(const uint16_t *in, void *out, int out_is_f32,
                           size_t num_segments, size_t segment_size, int threads) {
  const int t = pick_threads(threads);
#pragma omp parallel for schedule(static) num_threads(t)
  for (size_t j = 0; j < num_segments; j++) {
    const uint16_t *p = in + j * segment_size;
    float acc         = 0.f;
    if (out_is_f32) {
      float *o = (float *)out + j * segment_size;
      for (size_t i = 0; i < segment_size; i++) {
        acc += h2f(p[i]);
        o[i] = acc;
      }
    } else {
      uint16_t *o = (uint16_t *)out + j * segment_size;
      for (size_t i = 0; i < segment_size; i++) {
        acc += h2f(p[i]);
        o[i] = f2h(acc);
      }
    }
  }
  return t;
}

int tcu_cpu_full_reduce(const uint16_t *in, float *out, size_t n, int threads) {
  const int t  = pick_threads(threads);
  double total = 0.0;
  /* fixed blocks of 4096 elements, fp32 inside a block, fp64 across blocks */
  const size_t blk = 4096, nb = (n + blk - 1) / blk;
#pragma omp parallel for schedule(static) num_threads(t) reduction(+ : total)
  for (size_t b = 0; b < nb; b++) {
    const size_t lo = b * blk, hi = lo + blk < n ? lo + blk : n;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t i     = lo;
    for (; i + 8 <= hi; i += 8)
      for (int l = 0; l < 8; l++) acc[l] += h2f(in[i + l]);
    for (; i < hi; i++) acc[0] += h2f(in[i]);
    total += (double)(((acc[0] + acc[1]) + (acc[2] + acc[3])) +
                      ((acc[4] + acc[5]) + (acc[6] + acc[7])));
  }
  *out = (float)total;
  return t;
}

int tcu_cpu_full_scan(const uint16_t *in, float *out, size_t n, int threads) {
  /* Two-pass blocked scan: per-thread block totals, serial exclusive scan of
   * the totals, then a running sum seeded with the carry.  The running sum is
   * a double: an fp32 one stops growing near 2^24 for inputs in [0,1). */
  int t = pick_threads(threads);
#ifndef _OPENMP
  t = 1;
#endif
  if ((size_t)t > n / 1024 + 1) t = (int)(n / 1024 + 1);
  double totals[1024];
  if (t > 1024) t = 1024;
  const size_t per = (n + (size_t)t - 1) / (size_t)t;
#pragma omp parallel num_threads(t)
  {
#ifdef _OPENMP
    const int id = omp_get_thread_num();
#else
    const int id = 0;
#endif
    const size_t lo = (size_t)id * per < n ? (size_t)id * per : n;
    const size_t hi = lo + per < n ? lo + per : n;
    double s        = 0.0;
    for (size_t i = lo; i < hi; i++) s += (double)h2f(in[i]);
    totals[id] = s;
#pragma omp barrier
    double carry = 0.0;
    for (int k = 0; k < id; k++) carry += totals[k];
    for (size_t i = lo; i < hi; i++) {
      carry += (double)h2f(in[i]);
      out[i] = (float)carry;
    }
  }
  return t;
}
