// Segmented reduction and scan for every segment size the tiled kernels do
// not take: multiples of 16 that are not a power of two (48, 80, 768 ...),
// which the reference's kernels accept -- its drivers only ask for "multiples
// of 16" / "multiples of 256" (src/reduction/seg_wmma_16n.cu:137-172,
// seg_wmma_256n.cu:17-27) -- and, beyond the reference, any other size from 1
// up (tails are masked).  None of the reference's registered benchmarks uses
// such a size, so this path is built for coverage, not for the roofline: data
// read straight from global memory, the same contractions and the same exact
// hi/lo parts as the tiled kernels -- one warp per segment in general, rows of
// 16 elements packed 16 to a step for the multiples of 16 up to 2048 (the
// last part of this file).  Power-of-two sizes >= 16 never come here.
//
// kVec: every segment starts on a vector boundary (segment_size % 8 == 0 for
// the 16-byte loads of the reduction, % 4 == 0 for the 8-byte loads and
// 4-element stores of the scan); otherwise elements are moved one by one.
#pragma once

#include "common.cuh"
#include "reduce_kernels.cuh"
#include "scan_kernels.cuh"

namespace TCU_NS {

constexpr int kClassGeneral   = 16;  // any segment size that is not a power of two >= 16
constexpr int kGeneralThreads = 256;

__device__ __forceinline__ uint4 ldg128(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ uint2 ldg64(const void* p) {
  return __ldg(reinterpret_cast<const uint2*>(p));
}
// halves p[0 .. count) of at most kN, zeros beyond, packed two per register
template <int kN>
__device__ __forceinline__ void ldg_halves_masked(const uint8_t* p, long long count,
                                                  uint32_t (&packed)[kN / 2]) {
  const unsigned short* h = reinterpret_cast<const unsigned short*>(p);
#pragma unroll
  for (int k = 0; k < kN / 2; ++k) {
    const uint32_t a = 2 * k < count ? __ldg(h + 2 * k) : 0u;
    const uint32_t b = 2 * k + 1 < count ? __ldg(h + 2 * k + 1) : 0u;
    packed[k] = a | (b << 16);
  }
}
template <bool OUT32>
__device__ __forceinline__ void store_masked(void* out, unsigned long long idx, long long count,
                                             float r0, float r1, float r2, float r3) {
  const float r[4] = {r0, r1, r2, r3};
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (k < count) store_seg(out, OUT32, idx + k, r[k]);
}

// Each warp walks whole segments.  Per step a lane takes 16 bytes (8 halves);
// the four registers are the A fragment of one MMA against all-ones, so every
// element lands in exactly one row sum, whichever row that is.  Row sums of
// the exact hi and lo parts are flushed into a compensated pair of floats before they can
// round (double arithmetic is slow on this part).
// kBlock: long segments, too few of them to keep the SMs busy with one warp each -- the eight
// warps of a CTA share a segment (each takes every eighth run of 128 vectors) and their sums
// meet in shared memory.
template <bool kVec, bool kBlock = false>
__global__ void __launch_bounds__(kGeneralThreads) seg_reduce_general_kernel(const ReduceParams p,
                                                             unsigned long long seg_elems) {
  pdl_prologue();
  constexpr int kWarps = kGeneralThreads / 32;
  __shared__ float2 warp_tot[kWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned long long warps = kBlock ? gridDim.x : (unsigned long long)gridDim.x * kWarps;
  const unsigned long long first = kBlock ? blockIdx.x : (unsigned long long)blockIdx.x * kWarps + warp;
  const unsigned long long vecs  = (seg_elems + 7) / 8;  // groups of 8 elements per segment
  // Vectors per lane requested before the first is used, measured at 2^28 elements with 1 / 2 /
  // 3 / 4 / 6 / 8: 0.56 / 0.75 / 0.58 / 0.56 / 0.62 / 0.82 of the copy bandwidth at 16000 elements
  // per segment, 0.64 / 0.88 / 0.63 / 0.66 / 0.62 / 0.63 at 100000.
  constexpr int kInFlight = 2;
  const unsigned long long v_first = kBlock ? 32ull * kInFlight * warp : 0ull;
  const unsigned long long v_step  = kBlock ? 32ull * kInFlight * kWarps : 32ull * kInFlight;
  const Acc zero{0.f, 0.f, 0.f, 0.f};
  constexpr int kFlushEvery = 64;  // 64 steps x 16 elements per row: sums below 2^11 stay exact

  for (unsigned long long seg = first; seg < p.num_segments; seg += warps) {
    const uint8_t* src = p.in + seg * seg_elems * 2ull;
    float tot_h = 0.f, tot_l = 0.f;
    Acc ah = zero, al = zero;
    int pending = 0;
    for (unsigned long long v0 = v_first; v0 < vecs; v0 += v_step) {
      uint4 x[kInFlight];
#pragma unroll
      for (int k = 0; k < kInFlight; ++k) {
        const unsigned long long v = v0 + 32u * k + lane;
        x[k] = make_uint4(0u, 0u, 0u, 0u);
        if (v < vecs) {
          if constexpr (kVec) {
            x[k] = ldg128(src + v * 16);
          } else {
            uint32_t w[4];
            ldg_halves_masked<8>(src + v * 16, (long long)(seg_elems - v * 8), w);
            x[k] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
#pragma unroll
      for (int k = 0; k < kInFlight; ++k) {
        uint32_t h[4], l[4];
        split_hi_lo(x[k].x, h[0], l[0]);
        split_hi_lo(x[k].y, h[1], l[1]);
        split_hi_lo(x[k].z, h[2], l[2]);
        split_hi_lo(x[k].w, h[3], l[3]);
        ah = mma_ones(h, ah);
        al = mma_ones(l, al);
      }
      pending += kInFlight;
      if (pending >= kFlushEvery) {
        pair_add(tot_h, tot_l, ah.d0, al.d0);
        pair_add(tot_h, tot_l, ah.d2, al.d2);
        ah = al = zero;
        pending = 0;
      }
    }
    pair_add(tot_h, tot_l, ah.d0, al.d0);
    pair_add(tot_h, tot_l, ah.d2, al.d2);
    // every lane of a group holds the sums of rows g and g+8: add up the 8 groups
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
      const float oh = __shfl_xor_sync(0xffffffffu, tot_h, off), ol = __shfl_xor_sync(0xffffffffu, tot_l, off);
      pair_add(tot_h, tot_l, oh, ol);
    }
    if constexpr (kBlock) {
      if (lane == 0) warp_tot[warp] = make_float2(tot_h, tot_l);
      __syncthreads();
      if (warp == 0) {
        tot_h = tot_l = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) pair_add(tot_h, tot_l, warp_tot[w].x, warp_tot[w].y);
      }
      __syncthreads();  // warp_tot is written again for the CTA's next segment
      if (warp != 0) continue;
    }
    if (lane == 0) {
      store_seg(p.out, p.out_is_f32 != 0, seg, tot_h + tot_l);
      if (p.out_f64 != nullptr) p.out_f64[seg] = (double)tot_h + (double)tot_l;
    }
  }
}

// One warp per segment, 256 elements per step as 16 rows of 16 consecutive
// elements: A.U scans every row, an all-ones MMA gives the row totals, shuffles
// turn them into row carries, and the running carry of the segment (two floats)
// joins them in the accumulator operand.  Elements past the end of the segment
// are read as zeros and not stored.
template <bool OUT32, bool kVec, int kSteps = 1>
__global__ void __launch_bounds__(kGeneralThreads) seg_scan_general_kernel(const ScanParams p,
                                                           unsigned long long seg_elems) {
  pdl_prologue();
  using Geom = ScanGeom<4>;  // linear rows: row r of a step = its elements [16r, 16r+16)
  static_assert(Geom::kLinear, "the general scan relies on the linear 16-element rows");
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const unsigned long long warps = (unsigned long long)gridDim.x * (kGeneralThreads / 32);
  const unsigned long long first =
      (unsigned long long)blockIdx.x * (kGeneralThreads / 32) + (threadIdx.x >> 5);
  const unsigned long long num_segments = p.num_elems / seg_elems;
  const ScanOperands ops = make_scan_operands(lane, p.exclusive != 0);
  const Acc zero{0.f, 0.f, 0.f, 0.f};
  const int off_lo = Geom::lo(g, t, 0);  // bytes inside the 512-byte step

  for (unsigned long long seg = first; seg < num_segments; seg += warps) {
    const unsigned long long seg_base = seg * seg_elems;
    float xh = 0.f, xl = 0.f;  // the segment so far: an exact multiple of 2^-13 plus a small rest
    // this lane's elements of step e0: four of row g, four of row g + 8 (zeros past the segment's end)
    auto load_step = [&](unsigned long long e0, uint2& lo, uint2& hi) {
      lo = hi = make_uint2(0u, 0u);
      if (e0 >= seg_elems) return;
      const uint8_t* src = p.in + (seg_base + e0) * 2ull;
      const long long n_lo = (long long)(seg_elems - e0) - off_lo / 2, n_hi = n_lo - Geom::kHiOffset / 2;
      if constexpr (kVec) {  // whole groups of four
        if (n_lo > 0) lo = ldg64(src + off_lo);
        if (n_hi > 0) hi = ldg64(src + off_lo + Geom::kHiOffset);
      } else {
        uint32_t w[2];
        ldg_halves_masked<4>(src + off_lo, n_lo, w);
        lo = make_uint2(w[0], w[1]);
        ldg_halves_masked<4>(src + off_lo + Geom::kHiOffset, n_hi, w);
        hi = make_uint2(w[0], w[1]);
      }
    };
    // The loads of the next kSteps steps are in flight while one step is worked on; measured at
    // 2^28 elements with 1 / 2 / 3 / 4 / 6 steps, fp32 / fp16 outputs: 16000 elements per segment
    // 0.81 / 0.71, 0.81 / 0.68, 0.70 / 0.59, 0.70 / 0.58, 0.63 / 0.47 of the copy bandwidth; 100000
    // elements (few warps) 0.64 / 0.43, 0.63 / 0.39, 0.65 / 0.51, 0.65 / 0.50, 0.43 / 0.32.
    uint2 nlo[kSteps], nhi[kSteps];
#pragma unroll
    for (int k = 0; k < kSteps; ++k) load_step(256ull * k, nlo[k], nhi[k]);
    for (unsigned long long e0 = 0; e0 < seg_elems; e0 += 256) {
      const long long left = (long long)(seg_elems - e0);  // elements of the segment from this step on
      // this lane's four elements of row g / row g+8: how many of them exist
      const long long n_lo = left - off_lo / 2, n_hi = n_lo - Geom::kHiOffset / 2;
      const uint2 lo = nlo[0], hi = nhi[0];
#pragma unroll
      for (int k = 0; k + 1 < kSteps; ++k) {
        nlo[k] = nlo[k + 1];
        nhi[k] = nhi[k + 1];
      }
      load_step(e0 + 256ull * kSteps, nlo[kSteps - 1], nhi[kSteps - 1]);
      uint32_t ah[4], al[4];
      split_hi_lo(lo.x, ah[0], al[0]);
      split_hi_lo(hi.x, ah[1], al[1]);
      split_hi_lo(lo.y, ah[2], al[2]);
      split_hi_lo(hi.y, ah[3], al[3]);
      const Acc th = mma_ones(ah, zero), tl = mma_ones(al, zero);
      float ch_lo, cl_lo, ch_hi, cl_hi, step_h, step_l;
      row_carries<16>(th, tl, g, ch_lo, cl_lo, ch_hi, cl_hi, step_h, step_l);
      // a large xh is held back and added last (see scan_step_independent)
      const bool fold = fabsf(xh) < 1024.f;
      const float xf = fold ? xh : 0.f, big = fold ? 0.f : xh;
      const Acc c_h{ch_lo + xf, ch_lo + xf, ch_hi + xf, ch_hi + xf};
      const Acc c_l{cl_lo + xl, cl_lo + xl, cl_hi + xl, cl_hi + xl};
      const Acc ha = mma16816(ah[0], ah[1], ah[2], ah[3], ops.ua0, ops.ua1, c_h);
      const Acc hb = mma16816(ah[0], ah[1], ah[2], ah[3], ops.ub0, ops.ub1, c_h);
      const Acc la = mma16816(al[0], al[1], al[2], al[3], ops.ua0, ops.ua1, c_l);
      const Acc lb = mma16816(al[0], al[1], al[2], al[3], ops.ub0, ops.ub1, c_l);
      const unsigned long long out_lo = seg_base + e0 + off_lo / 2;
      const unsigned long long out_hi = out_lo + Geom::kHiOffset / 2;
      const float r0 = (ha.d0 + la.d0) + big, r1 = (ha.d1 + la.d1) + big;  // row g, 4 outputs
      const float r2 = (hb.d0 + lb.d0) + big, r3 = (hb.d1 + lb.d1) + big;
      const float q0 = (ha.d2 + la.d2) + big, q1 = (ha.d3 + la.d3) + big;  // row g + 8
      const float q2 = (hb.d2 + lb.d2) + big, q3 = (hb.d3 + lb.d3) + big;
      if constexpr (kVec) {
        if (n_lo > 0) store4<OUT32>(p.out, out_lo, r0, r1, r2, r3);
        if (n_hi > 0) store4<OUT32>(p.out, out_hi, q0, q1, q2, q3);
      } else {
        store_masked<OUT32>(p.out, out_lo, n_lo, r0, r1, r2, r3);
        store_masked<OUT32>(p.out, out_hi, n_hi, q0, q1, q2, q3);
      }
      pair_add(xh, xl, step_h, step_l);
      pair_renorm(xh, xl);
    }
  }
}

// ---------------------------------------------------------------------------
// Segment sizes that are a multiple of 16 but not a power of two, up to 2048
// elements (48, 80, 240, 768 ...: what the reference's 16n kernels accept beyond
// their dispatch table).  One warp per segment would leave most lanes idle on
// the short ones, so here the array is taken as rows of 16 elements -- a
// segment is m = S / 16 whole rows -- and a warp walks a chunk of whole
// segments 16 rows (256 contiguous elements, one coalesced 512-byte read) at a
// time: an all-ones MMA gives the 16 row sums, row_carries their exclusive
// prefix inside the step, and the sums of the rows of one segment are
// differences of those prefixes (fetched from the lane that holds the
// segment's first row), plus what the segment brought from earlier steps.  All
// sums are of exact hi / lo parts, as everywhere else.
struct RowsParams {
  const uint8_t* in;
  void* out;
  double* out_f64;                 // reduction only, may be null
  unsigned long long num_segments;
  unsigned int rows_per_segment;   // m = segment_size / 16 (scan)
  unsigned int segment_bytes;      // reduction: any multiple of 16 bytes
  unsigned int segs_per_chunk;     // whole segments a warp takes at a time
  int out_is_f32;
  int exclusive;                   // scan only
};

// prefix entry of local row a (0..15) out of the per-lane values of rows g / g+8
__device__ __forceinline__ void fetch_row_prefix(int a, float eh_lo, float el_lo, float eh_hi,
                                                 float el_hi, float& h, float& l) {
  const int src = 4 * (a & 7);
  const float h0 = __shfl_sync(0xffffffffu, eh_lo, src), l0 = __shfl_sync(0xffffffffu, el_lo, src);
  const float h1 = __shfl_sync(0xffffffffu, eh_hi, src), l1 = __shfl_sync(0xffffffffu, el_hi, src);
  h = a < 8 ? h0 : h1;
  l = a < 8 ? l0 : l1;
}

template <bool OUT32>
__global__ void __launch_bounds__(kGeneralThreads) seg_rows_kernel(const RowsParams p) {
  pdl_prologue();
  using Geom = ScanGeom<4>;  // linear rows: row r of a step = its elements [16r, 16r + 16)
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const unsigned long long warps = (unsigned long long)gridDim.x * (kGeneralThreads / 32);
  const unsigned long long first =
      (unsigned long long)blockIdx.x * (kGeneralThreads / 32) + (threadIdx.x >> 5);
  const unsigned int m = p.rows_per_segment;
  const unsigned int step_q = 16u % m, step_s = 16u / m;
  const unsigned long long chunks = (p.num_segments + p.segs_per_chunk - 1) / p.segs_per_chunk;
  const ScanOperands ops = make_scan_operands(lane, p.exclusive != 0);
  const Acc zero{0.f, 0.f, 0.f, 0.f};
  const int off_lo = Geom::lo(g, t, 0);  // bytes inside the 512-byte step

  for (unsigned long long chunk = first; chunk < chunks; chunk += warps) {
    const unsigned long long seg0 = chunk * p.segs_per_chunk;
    const unsigned long long left = p.num_segments - seg0;
    const unsigned int nseg = left < p.segs_per_chunk ? (unsigned int)left : p.segs_per_chunk;
    const unsigned int rows = nseg * m;
    const unsigned long long elem0 = seg0 * m * 16ull;
    // this lane's two rows of the current step: position inside their segment, segment in the chunk
    unsigned int q_lo = (unsigned)g % m, s_lo = (unsigned)g / m;
    unsigned int q_hi = (unsigned)(g + 8) % m, s_hi = (unsigned)(g + 8) / m;
    float open_h = 0.f, open_l = 0.f;  // what the segment that is open at the start of the step has so far
    // the loads of the next two steps are in flight while one step is worked on
    constexpr int kAhead = 2;  // measured with fp32 outputs at S=48: 1 / 2 / 3 steps ahead 0.75 / 0.83 / 0.71
    uint2 nlo[kAhead], nhi[kAhead];
    auto load_step = [&](unsigned int r, uint2& lo, uint2& hi) {
      const uint8_t* src = p.in + (elem0 + 16ull * r) * 2ull;
      lo = r + g < rows ? ldg64(src + off_lo) : make_uint2(0u, 0u);
      hi = r + g + 8 < rows ? ldg64(src + off_lo + Geom::kHiOffset) : make_uint2(0u, 0u);
    };
#pragma unroll
    for (int k = 0; k < kAhead; ++k) load_step(16u * k, nlo[k], nhi[k]);
    for (unsigned int r0 = 0; r0 < rows; r0 += 16) {
      const bool ok_lo = r0 + g < rows, ok_hi = r0 + g + 8 < rows;
      const uint2 lo = nlo[0], hi = nhi[0];
#pragma unroll
      for (int k = 0; k + 1 < kAhead; ++k) {
        nlo[k] = nlo[k + 1];
        nhi[k] = nhi[k + 1];
      }
      load_step(r0 + 16u * kAhead, nlo[kAhead - 1], nhi[kAhead - 1]);
      uint32_t ah[4], al[4];
      split_hi_lo(lo.x, ah[0], al[0]);
      split_hi_lo(hi.x, ah[1], al[1]);
      split_hi_lo(lo.y, ah[2], al[2]);
      split_hi_lo(hi.y, ah[3], al[3]);
      const Acc th = mma_ones(ah, zero), tl = mma_ones(al, zero);  // d0: row g, d2: row g + 8
      float eh_lo, el_lo, eh_hi, el_hi, step_h, step_l;
      row_carries<16>(th, tl, g, eh_lo, el_lo, eh_hi, el_hi, step_h, step_l);
      // sum of the rows of this row's segment that lie before it in this step
      const bool here_lo = q_lo <= (unsigned)g, here_hi = q_hi <= (unsigned)(g + 8);
      float bh, bl;
      fetch_row_prefix(here_lo ? g - (int)q_lo : 0, eh_lo, el_lo, eh_hi, el_hi, bh, bl);
      const float xh_lo = here_lo ? eh_lo - bh : eh_lo, xl_lo = here_lo ? el_lo - bl : el_lo;
      fetch_row_prefix(here_hi ? g + 8 - (int)q_hi : 0, eh_lo, el_lo, eh_hi, el_hi, bh, bl);
      const float xh_hi = here_hi ? eh_hi - bh : eh_hi, xl_hi = here_hi ? el_hi - bl : el_hi;
      // ... plus what the segment brought along, if it began in an earlier step.  Sums are kept
      // as two floats, of the hi parts and of the lo parts: a segment is at most 2048 elements,
      // so both are exact while the sum stays below 2^11 and rounded like any float sum above.
      float ch_lo = (here_lo ? 0.f : open_h) + xh_lo, cl_lo = (here_lo ? 0.f : open_l) + xl_lo;
      float ch_hi = (here_hi ? 0.f : open_h) + xh_hi, cl_hi = (here_hi ? 0.f : open_l) + xl_hi;
      const float ih_hi = ch_hi + th.d2, il_hi = cl_hi + tl.d2;  // through the step's last row, in lane 28

      {
        // the carry of each row as an exact multiple of 2^-13 plus a small rest; a large one is
        // held back and added last (see scan_step_independent)
        const float m_lo = grid13(cl_lo), m_hi = grid13(cl_hi);
        ch_lo += m_lo;
        cl_lo -= m_lo;
        ch_hi += m_hi;
        cl_hi -= m_hi;
        float big_lo = 0.f, big_hi = 0.f;
        if (fabsf(ch_lo) >= 1024.f) { big_lo = ch_lo; ch_lo = 0.f; }
        if (fabsf(ch_hi) >= 1024.f) { big_hi = ch_hi; ch_hi = 0.f; }
        const Acc c_h{ch_lo, ch_lo, ch_hi, ch_hi}, c_l{cl_lo, cl_lo, cl_hi, cl_hi};
        const Acc ha = mma16816(ah[0], ah[1], ah[2], ah[3], ops.ua0, ops.ua1, c_h);
        const Acc hb = mma16816(ah[0], ah[1], ah[2], ah[3], ops.ub0, ops.ub1, c_h);
        const Acc la = mma16816(al[0], al[1], al[2], al[3], ops.ua0, ops.ua1, c_l);
        const Acc lb = mma16816(al[0], al[1], al[2], al[3], ops.ub0, ops.ub1, c_l);
        const unsigned long long o_lo = elem0 + 16ull * r0 + off_lo / 2;
        if (ok_lo)
          store4<OUT32>(p.out, o_lo, (ha.d0 + la.d0) + big_lo, (ha.d1 + la.d1) + big_lo,
                        (hb.d0 + lb.d0) + big_lo, (hb.d1 + lb.d1) + big_lo);
        if (ok_hi)
          store4<OUT32>(p.out, o_lo + Geom::kHiOffset / 2, (ha.d2 + la.d2) + big_hi,
                        (ha.d3 + la.d3) + big_hi, (hb.d2 + lb.d2) + big_hi, (hb.d3 + lb.d3) + big_hi);
      }
      // the segment of the step's last row stays open unless that row ends it
      const float t15_h = __shfl_sync(0xffffffffu, ih_hi, 28), t15_l = __shfl_sync(0xffffffffu, il_hi, 28);
      const unsigned int q15 = __shfl_sync(0xffffffffu, q_hi, 28);
      open_h = q15 == m - 1 ? 0.f : t15_h;
      open_l = q15 == m - 1 ? 0.f : t15_l;
      q_lo += step_q;  // 16 rows on: 16 / m segments and 16 % m rows
      s_lo += step_s;
      if (q_lo >= m) { q_lo -= m; ++s_lo; }
      q_hi += step_q;
      s_hi += step_s;
      if (q_hi >= m) { q_hi -= m; ++s_hi; }
    }
  }
}

// Reduction for the same segment sizes (and any other multiple of 8 elements up to 2048),
// without the prefixes the scan needs: a warp takes 16
// segments as the 16 rows of an MMA.  The order of the elements inside a row does not matter
// for a sum, so a lane loads 16 consecutive bytes of "its" two segments per step (four lanes
// cover 64 bytes of a segment, the warp whole 32-byte sectors of one contiguous range) and the
// four registers feed two all-ones MMAs: the row sums come out complete, no shuffles.
// kR = 64-byte steps per round (loads in flight per lane: 2 kR), the smallest that covers a
// segment, at most 4: measured at 2^28 elements with kR = 1 / 2 / 3 / 4, 48 elements per segment
// 0.66 / 0.76 / 0.62 / 0.47 of the copy bandwidth, 80 elements 0.76 / 0.73 / 0.90 / 0.73, 1000
// elements 0.68 / 0.84 / 0.85 / 0.87.
// kAny: segments of any number of elements, so a row starts at any even byte address.  A lane
// then loads the aligned 16 bytes around "its" piece and clears the halves that belong to the
// neighbouring segments (a sum does not care where in the vector an element sits).
__device__ __forceinline__ uint4 keep_halves(uint4 v, int i0, unsigned int count) {
  // halves i0 ... i0 + 7 of the row are in v: keep those with 0 <= index < count
  auto mask = [&](int i) -> uint32_t {
    return ((unsigned)i < count ? 0x0000ffffu : 0u) | ((unsigned)(i + 1) < count ? 0xffff0000u : 0u);
  };
  return make_uint4(v.x & mask(i0), v.y & mask(i0 + 2), v.z & mask(i0 + 4), v.w & mask(i0 + 6));
}

template <int kR, bool kAny = false>
__global__ void __launch_bounds__(kGeneralThreads) seg_rowsum_kernel(const RowsParams p) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const unsigned long long warps = (unsigned long long)gridDim.x * (kGeneralThreads / 32);
  const unsigned long long first =
      (unsigned long long)blockIdx.x * (kGeneralThreads / 32) + (threadIdx.x >> 5);
  const unsigned int seg_bytes    = p.segment_bytes;
  const unsigned long long groups = (p.num_segments + 15) / 16;
  const Acc zero{0.f, 0.f, 0.f, 0.f};
  const bool f32 = p.out_is_f32 != 0;

  // One round = 64 kR bytes of each of a group's segments: 2 kR loads per lane.  The loads of the
  // next round (of this group or of the warp's next group) are issued before the current round
  // is worked on.
  auto load_round = [&](unsigned long long grp, unsigned int b, uint4 (&x)[kR], uint4 (&y)[kR]) {
    const unsigned long long seg_lo = grp * 16 + g;
    const bool ok_lo = seg_lo < p.num_segments, ok_hi = seg_lo + 8 < p.num_segments;
    if constexpr (kAny) {
      const unsigned long long a_lo = seg_lo * seg_bytes, a_hi = a_lo + 8ull * seg_bytes;
      const unsigned int off_lo = (unsigned int)a_lo & 15u, off_hi = (unsigned int)a_hi & 15u;
      const uint8_t* src_lo = p.in + (a_lo - off_lo) + 16u * t + b;  // 16-byte aligned
      const uint8_t* src_hi = p.in + (a_hi - off_hi) + 16u * t + b;
      const unsigned int count = seg_bytes / 2;
#pragma unroll
      for (int k = 0; k < kR; ++k) {
        const int piece = (int)(b + 64u * k + 16u * t);  // byte offset from the aligned row start
        const int i_lo = (piece - (int)off_lo) / 2, i_hi = (piece - (int)off_hi) / 2;  // even numerators
        const bool in_lo = ok_lo && i_lo < (int)count && i_lo + 8 > 0;
        const bool in_hi = ok_hi && i_hi < (int)count && i_hi + 8 > 0;
        x[k] = in_lo ? keep_halves(ldg128(src_lo + 64u * k), i_lo, count) : make_uint4(0u, 0u, 0u, 0u);
        y[k] = in_hi ? keep_halves(ldg128(src_hi + 64u * k), i_hi, count) : make_uint4(0u, 0u, 0u, 0u);
      }
    } else {
      const uint8_t* src_lo = p.in + seg_lo * seg_bytes + 16u * t + b;
      const uint8_t* src_hi = src_lo + 8ull * seg_bytes;
#pragma unroll
      for (int k = 0; k < kR; ++k) {
        const bool in = b + 64u * k + 16u * t < seg_bytes;
        x[k] = ok_lo && in ? ldg128(src_lo + 64u * k) : make_uint4(0u, 0u, 0u, 0u);
        y[k] = ok_hi && in ? ldg128(src_hi + 64u * k) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  unsigned long long grp = first;
  unsigned int b = 0;
  if (grp >= groups) return;
  uint4 x[kR], y[kR];
  load_round(grp, b, x, y);
  Acc ah = zero, al = zero;
  for (;;) {
    unsigned long long ngrp = grp;
    unsigned int nb = b + 64u * kR;
    if (nb >= seg_bytes + (kAny ? 14u : 0u)) {  // (a row may start up to 14 bytes into its first vector)
      nb   = 0u;
      ngrp = grp + warps;
    }
    const bool more = ngrp < groups;
    uint4 nx[kR], ny[kR];
    if (more) load_round(ngrp, nb, nx, ny);
#pragma unroll
    for (int k = 0; k < kR; ++k) {
      uint4 xh, xl, yh, yl;
      split_hi_lo(x[k].x, xh.x, xl.x);
      split_hi_lo(x[k].y, xh.y, xl.y);
      split_hi_lo(x[k].z, xh.z, xl.z);
      split_hi_lo(x[k].w, xh.w, xl.w);
      split_hi_lo(y[k].x, yh.x, yl.x);
      split_hi_lo(y[k].y, yh.y, yl.y);
      split_hi_lo(y[k].z, yh.z, yl.z);
      split_hi_lo(y[k].w, yh.w, yl.w);
      ah = mma16816(xh.x, yh.x, xh.y, yh.y, kOnesH2, kOnesH2, ah);  // rows g / g + 8
      ah = mma16816(xh.z, yh.z, xh.w, yh.w, kOnesH2, kOnesH2, ah);
      al = mma16816(xl.x, yl.x, xl.y, yl.y, kOnesH2, kOnesH2, al);
      al = mma16816(xl.z, yl.z, xl.w, yl.w, kOnesH2, kOnesH2, al);
    }
    if (nb == 0u) {  // the group's last round: every column of the accumulators holds the row sums
      const unsigned long long seg_lo = grp * 16 + g, seg_hi = seg_lo + 8;
      if (t == 0) {
        if (seg_lo < p.num_segments) {
          store_seg(p.out, f32, seg_lo, ah.d0 + al.d0);
          if (p.out_f64 != nullptr) p.out_f64[seg_lo] = (double)ah.d0 + (double)al.d0;
        }
        if (seg_hi < p.num_segments) {
          store_seg(p.out, f32, seg_hi, ah.d2 + al.d2);
          if (p.out_f64 != nullptr) p.out_f64[seg_hi] = (double)ah.d2 + (double)al.d2;
        }
      }
      ah = al = zero;
    }
    if (!more) break;
#pragma unroll
    for (int k = 0; k < kR; ++k) {
      x[k] = nx[k];
      y[k] = ny[k];
    }
    grp = ngrp;
    b   = nb;
  }
}

}  // namespace TCU_NS
