/*
 * tcu_oracle.h -- CPU oracle for segmented / full sum-reduction and inclusive
 * prefix sum over fp16 arrays.
 *
 * TEST INFRASTRUCTURE ONLY.  This code is the checker and the timed CPU
 * baseline; it is never linked into, imported by or called from the shipped
 * CUDA library.
 *
 * PARITY UNPINNED: the reference (c3sr/tcu_scope) holds no golden vectors,
 * known-answer tests or fixtures for this path -- every validation block in
 * its drivers is compiled out (src/reduction/seg_wmma_16n.cu:82-109,
 * src/prefixsum/wmma_3kers.cu:92-129).  What this oracle restates is the
 * sequential check those blocks intended: a running sum over the inputs of
 * each segment, in double precision over the fp16-rounded inputs.
 */
#ifndef TCU_ORACLE_H_
#define TCU_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Input distributions of the seeded generator (shared, bit for bit, with the
 * device fill kernel of the library under test). */
enum {
  TCU_DIST_UNIFORM_PM1 = 0, /* (u24 - 2^23) * 2^-23  in [-1, 1)           */
  TCU_DIST_UNIFORM_01  = 1, /* u24 * 2^-24           in [0, 1)            */
  TCU_DIST_SMALL_INT   = 2, /* (u24 % 5) - 2         in {-2,...,2}: exact */
  TCU_DIST_CONST_0P001 = 3  /* half(0.001f): the reference's constant fill
                               (src/reduction/seg_wmma_16n.cu:38)          */
};

/* IEEE binary16 <-> wider formats, software, bit exact. */
uint16_t tcu_oracle_f32_to_f16(float x);     /* round to nearest even */
uint16_t tcu_oracle_f64_to_f16(double x);    /* round to nearest even */
double tcu_oracle_f16_to_f64(uint16_t h);

/* Counter-based generator: element i depends only on (seed, first_index+i). */
uint64_t tcu_oracle_hash(uint64_t seed, uint64_t index);
void tcu_oracle_fill_f16(uint16_t *out, size_t n, uint64_t seed, uint64_t first_index,
                         int dist);

/* fp64 restatement.  Segment j is in[j*S, (j+1)*S)
 * (layout: src/reduction/seg_wmma_16n.cu:14-25). */
void tcu_oracle_segmented_reduce(const uint16_t *in, double *out, size_t num_segments,
                                 size_t segment_size);
/* Inclusive scan: U has ones for i <= j (src/prefixsum/kernel.cuh:60,79-81). */
void tcu_oracle_segmented_scan(const uint16_t *in, double *out, size_t num_segments,
                               size_t segment_size);

/* Tile algebra of the reference's 256-wide scan, A.U + (L.A).1, evaluated in
 * double over one row-major 16x16 tile (src/prefixsum/kernel.cuh:316-361).
 * out[256] must equal the running sum of in[256]. */
void tcu_oracle_tile256_scan_algebra(const uint16_t *in, double *out);

/* Tolerance checks.  Both return the number of violations.
 *  f32: |got - ref| <= max(rel * |ref|, abs_floor)
 *  f16: distance in representable halves between got and half(ref) <= max_ulp */
size_t tcu_oracle_check_f32(const float *got, const double *ref, size_t n, double rel,
                            double abs_floor, double *max_abs_err, double *max_rel_err);
size_t tcu_oracle_check_f16(const uint16_t *got, const double *ref, size_t n, int max_ulp,
                            int *worst_ulp);

/* Plain CPU implementation of the same operations (fp32 accumulate, hardware
 * half conversion, OpenMP over whole segments / blocks): the timed baseline.
 * threads <= 0 means "all cores this process may run on".  Each returns the
 * thread count actually used. */
int tcu_cpu_segmented_reduce(const uint16_t *in, float *out, size_t num_segments,
                             size_t segment_size, int threads);
int tcu_cpu_segmented_scan(const uint16_t *in, void *out, int out_is_f32,
                           size_t num_segments, size_t segment_size, int threads);
int tcu_cpu_full_reduce(const uint16_t *in, float *out, size_t n, int threads);
int tcu_cpu_full_scan(const uint16_t *in, float *out, size_t n, int threads);
int tcu_cpu_available_cores(void);

#ifdef __cplusplus
}
#endif
#endif /* TCU_ORACLE_H_ */
