// Segmented and full sum-reduction of fp16 arrays on the tensor cores.
//
// What it replaces in c3sr/tcu_scope: compute_wmma_segmented_reduction_16n
// (src/reduction/kernel.cuh:80-125), ..._256n (:301-356), ..._256n_block
// (:418-485) and the two-kernel full reduction built from them
// (src/reduction/wmma_2kers.cu:65-81).  Same contraction -- rows of the input
// times a constant matrix of ones -- but one persistent kernel for every
// segment size, fp32 accumulation, and exact partial sums (see split_hi_lo).
//
// Data flow per CTA: one producer thread streams 32 KiB tiles of the input
// into a shared-memory ring with linear TMA copies; eight consumer warps each
// own a 4 KiB slice of every tile.  Inside a slice lane-group g (4 lanes) owns
// the 512-byte "stream" [512 g, 512 g + 512): at step j every lane reads 16
// bytes of its stream (conflict-free LDS.128) and one m16n8k16 MMA adds the
// 8 x 32 halves read by the warp into rows g (first 8 bytes of each lane) and
// g + 8 (last 8 bytes) of the accumulator.  A sum is order-free, so the
// operand's k order is whatever the load produced.
#pragma once

#include "common.cuh"

namespace TCU_NS {

struct ReduceParams {
  const uint8_t* in;                     // fp16 input, 16-byte aligned
  void* out;                             // one float or half per segment
  unsigned long long num_elems;          // num_segments * segment_size
  unsigned long long num_segments;
  int out_is_f32;
  // Long segments (segment_size > kTileElems) and the full reduction only:
  unsigned long long tiles_per_segment;  // segment_size / kTileElems
  double* bound_val;                     // [2 * gridDim.x] head / tail partial of each CTA
  long long* bound_seg;                  // [2 * gridDim.x] their segment, -1 = none
  unsigned int* done_counter;            // zeroed by the host before the launch
  double* out_f64;                       // optional: segment sums in double (may be null)
  unsigned int spread_slices;            // classes 12 ... 14: slices (2048 elements) per segment
  unsigned long long test_skip_tile;     // ~0 in production; a test names a tile that is never loaded
};

// Segment classes.  4..11: segment_size = 2^class, whole segments inside one
// warp slice.  12..14: 4096/8192/16384, a segment spans 2/4/8 slices of one
// tile.  15: segment_size is a multiple of the tile (incl. the full reduction).
constexpr int kClassLong = 15;

__device__ __forceinline__ void store_seg(void* out, bool f32, unsigned long long idx, float v) {
  if (f32)
    static_cast<float*>(out)[idx] = v;
  else
    static_cast<uint16_t*>(out)[idx] = to16_rn(v);
}

// ---------------------------------------------------------------------------
// One warp reduces one 4 KiB slice.  For classes <= 11 it writes the slice's
// 2048/S segment sums; for larger classes it returns the slice total as an
// exact (hi, lo) float pair.
template <int SC>
__device__ __forceinline__ float2 reduce_slice(const uint8_t* slice, void* out, bool out_f32,
                                               unsigned long long seg_base, int valid_segs,
                                               int lane) {
  constexpr int S         = SC <= 11 ? (1 << SC) : kSliceElems;
  constexpr bool kSplit   = S >= 256;           // exact hi/lo accumulation
  constexpr int kStepsSeg = S >= 256 ? 8 : (S >= 32 ? S / 32 : 1);  // MMAs per accumulator
  const int g = lane >> 2, t = lane & 3;
  const int sw = g & 1;  // odd groups walk each pair of steps backwards: no bank conflicts
  const uint8_t* base = slice + 512 * g + 16 * t;
  const Acc zero{0.f, 0.f, 0.f, 0.f};

  // B operand.  S == 16: a 64-byte step holds two segments, X in lanes t<2 and
  // Y in lanes t>=2; k = 2t+e (+8) belongs to X iff bit 1 of t is clear, and
  // even output columns collect X, odd ones Y.  Otherwise: all ones.
  const uint32_t bsel = (S == 16) ? ((((t >> 1) & 1) == (g & 1)) ? kOnesH2 : 0u) : kOnesH2;

  float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
  Acc acc_h = zero, acc_l = zero;

#pragma unroll
  for (int j = 0; j < 8; ++j) {
    // step index j ^ sw, written so that the offset is a compile-time constant
    const uint4 w = lds128(base + 64 * j + ((j & 1) ? -64 * sw : 64 * sw));
    if constexpr (kSplit) {
      uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
      split_hi_lo(w.x, h0, l0);
      split_hi_lo(w.y, h1, l1);
      split_hi_lo(w.z, h2, l2);
      split_hi_lo(w.w, h3, l3);
      acc_h = mma16816(h0, h2, h1, h3, bsel, bsel, acc_h);
      acc_l = mma16816(l0, l2, l1, l3, bsel, bsel, acc_l);
    } else {
      const bool first = (j % kStepsSeg) == 0;
      acc_h = mma16816(w.x, w.z, w.y, w.w, bsel, bsel, first ? zero : acc_h);
      if ((j % kStepsSeg) == kStepsSeg - 1) {
        if constexpr (S == 16) {
          // this step is stream-relative step jp = j ^ sw: segments 2jp, 2jp+1
          const float x = acc_h.d0 + acc_h.d2, y = acc_h.d1 + acc_h.d3;
          if ((j >> 1) == t) {
            if (((j & 1) ^ sw) == 0) { o0 = x; o1 = y; } else { o2 = x; o3 = y; }
          }
        } else if constexpr (S == 32) {
          const float v = acc_h.d0 + acc_h.d2;
          if ((j >> 1) == t) {
            if (((j & 1) ^ sw) == 0) o0 = v; else o1 = v;
          }
        } else {  // S == 64 or 128: segment m of the stream finished
          const float v = acc_h.d0 + acc_h.d2;
          if ((j / kStepsSeg) == t) o0 = v;
        }
      }
    }
  }

  if constexpr (S == 16) {
    const int s0 = 16 * g + 4 * t;  // first of this lane's 4 consecutive segments
    if (s0 + 3 < valid_segs) {
      if (out_f32) {
        *reinterpret_cast<float4*>(static_cast<float*>(out) + seg_base + s0) =
            make_float4(o0, o1, o2, o3);
      } else {
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(out) + seg_base + s0) =
            make_uint2(pack2_rn(o0, o1), pack2_rn(o2, o3));
      }
    } else {
      const float o[4] = {o0, o1, o2, o3};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (s0 + e < valid_segs) store_seg(out, out_f32, seg_base + s0 + e, o[e]);
    }
    return make_float2(0.f, 0.f);
  } else if constexpr (S == 32) {
    const int s0 = 8 * g + 2 * t;
    if (s0 < valid_segs) store_seg(out, out_f32, seg_base + s0, o0);
    if (s0 + 1 < valid_segs) store_seg(out, out_f32, seg_base + s0 + 1, o1);
    return make_float2(0.f, 0.f);
  } else if constexpr (S == 64 || S == 128) {
    constexpr int kSegsPerStream = 256 / S;  // 4 or 2
    const int s0 = kSegsPerStream * g + t;
    if (t < kSegsPerStream && s0 < valid_segs) store_seg(out, out_f32, seg_base + s0, o0);
    return make_float2(0.f, 0.f);
  } else {
    // One accumulator pair per stream.  Rows g and g+8 together hold the
    // stream's sum in every column; both parts are exact.
    float vh = acc_h.d0 + acc_h.d2, vl = acc_l.d0 + acc_l.d2;
    constexpr int kStreamsPerSeg = S / 256;  // 1, 2, 4, 8
#pragma unroll
    for (int m = 1; m < kStreamsPerSeg; m <<= 1) {
      vh += __shfl_xor_sync(0xffffffffu, vh, 4 * m);
      vl += __shfl_xor_sync(0xffffffffu, vl, 4 * m);
    }
    if constexpr (SC <= 11) {
      const int s0 = g / kStreamsPerSeg;
      if (t == 0 && (g % kStreamsPerSeg) == 0 && s0 < valid_segs)
        store_seg(out, out_f32, seg_base + s0, vh + vl);
    }
    return make_float2(vh, vl);
  }
}

// ---------------------------------------------------------------------------
// CUDA-core ablation of reduce_slice: same loads, same outputs, but the sums
// are fp32 adds and warp shuffles instead of MMAs.  Exists so that a profile
// can show what the tensor-core formulation buys; not used by default.
__device__ __forceinline__ float sum8_halves(const uint4& w) {
  const float2 a = unpack2(w.x), b = unpack2(w.y), c = unpack2(w.z), d = unpack2(w.w);
  return ((a.x + a.y) + (b.x + b.y)) + ((c.x + c.y) + (d.x + d.y));
}

template <int SC>
__device__ __forceinline__ float2 shuffle_reduce_slice(const uint8_t* slice, void* out,
                                                       bool out_f32, unsigned long long seg_base,
                                                       int valid_segs, int lane) {
  constexpr int S         = SC <= 11 ? (1 << SC) : kSliceElems;
  constexpr int kStepsSeg = S >= 256 ? 8 : (S >= 32 ? S / 32 : 1);
  const int g = lane >> 2, t = lane & 3;
  const uint8_t* base = slice + 512 * g + 16 * t;
  float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f, acc = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float v = sum8_halves(lds128(base + 64 * j));
    if constexpr (S == 16) {
      v += __shfl_xor_sync(0xffffffffu, v, 1);  // lanes t<2: segment 2j, lanes t>=2: 2j+1
      const float other = __shfl_xor_sync(0xffffffffu, v, 2);
      const float x = t < 2 ? v : other, y = t < 2 ? other : v;
      if ((j >> 1) == t) {
        if ((j & 1) == 0) { o0 = x; o1 = y; } else { o2 = x; o3 = y; }
      }
    } else {
      acc = (j % kStepsSeg) == 0 ? v : acc + v;
      if ((j % kStepsSeg) == kStepsSeg - 1) {
        float r = acc + __shfl_xor_sync(0xffffffffu, acc, 1);
        r += __shfl_xor_sync(0xffffffffu, r, 2);
        if constexpr (S == 32) {
          if ((j >> 1) == t) { if ((j & 1) == 0) o0 = r; else o1 = r; }
        } else if constexpr (S == 64 || S == 128) {
          if ((j / kStepsSeg) == t) o0 = r;
        } else {
          o0 = r;
        }
      }
    }
  }
  if constexpr (S == 16) {
    const int s0 = 16 * g + 4 * t;
    const float o[4] = {o0, o1, o2, o3};
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (s0 + e < valid_segs) store_seg(out, out_f32, seg_base + s0 + e, o[e]);
    return make_float2(0.f, 0.f);
  } else if constexpr (S == 32) {
    const int s0 = 8 * g + 2 * t;
    if (s0 < valid_segs) store_seg(out, out_f32, seg_base + s0, o0);
    if (s0 + 1 < valid_segs) store_seg(out, out_f32, seg_base + s0 + 1, o1);
    return make_float2(0.f, 0.f);
  } else if constexpr (S == 64 || S == 128) {
    constexpr int kSegsPerStream = 256 / S;
    const int s0 = kSegsPerStream * g + t;
    if (t < kSegsPerStream && s0 < valid_segs) store_seg(out, out_f32, seg_base + s0, o0);
    return make_float2(0.f, 0.f);
  } else {
    float v = o0;
    constexpr int kStreamsPerSeg = S / 256;
#pragma unroll
    for (int m = 1; m < kStreamsPerSeg; m <<= 1) v += __shfl_xor_sync(0xffffffffu, v, 4 * m);
    if constexpr (SC <= 11) {
      const int s0 = g / kStreamsPerSeg;
      if (t == 0 && (g % kStreamsPerSeg) == 0 && s0 < valid_segs)
        store_seg(out, out_f32, seg_base + s0, v);
    }
    return make_float2(v, 0.f);
  }
}

// ---------------------------------------------------------------------------
template <int SC, bool kTensor = true>
__global__ void __launch_bounds__(kThreads, 1) seg_reduce_kernel(const ReduceParams p) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * kStages];
  __shared__ double warp_sum[2][kConsumerWarps];  // long class: per-warp running sums of a segment
  __shared__ int s_is_last;

  // 128-byte aligned ring, whatever offset the dynamic segment starts at
  uint8_t* ring = dyn_smem + ((128u - (smem_u32(dyn_smem) & 127u)) & 127u);
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Segments of 2, 4 or 8 slices: a stage of the ring does not hold 32 KiB of consecutive input
  // but one slice of each of eight consecutive segments, so that warp w meets the G slices of
  // "its" segment in G consecutive stages and adds them up in registers.  No warp ever needs
  // another warp's sum (one barrier of the consumer warps per tile measured 1.01 / 0.97 / 0.95
  // of the copy bandwidth at 4096 / 8192 / 16384 elements, a collector warp 0.93).
  constexpr bool kSpread = SC >= 12 && SC <= 14;
  // (2, 4 or 8 for segments of 4096 ... 16384 elements; longer powers of two are routed through
  // class 14 with their own count when there are enough segments to fill the SMs this way)
  const int G = kSpread ? (int)p.spread_slices : 1;
  const unsigned long long num_units = (p.num_segments + kConsumerWarps - 1) / kConsumerWarps;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_prologue();  // nothing above touched global memory

  const unsigned long long total_bytes = p.num_elems * 2ull;
  const unsigned long long num_tiles   = (total_bytes + kTileBytes - 1) / kTileBytes;
  // Short classes interleave tiles over CTAs; the long class gives each CTA a
  // contiguous run so that a segment's partial sum stays in one register.
  unsigned long long tile_begin, tile_end, tile_step;
  // One segment (the full reduction) needs no contiguity either.
  const bool single = SC == kClassLong && p.num_segments == 1;
  if (SC == kClassLong && !single) {
    tile_begin = num_tiles * blockIdx.x / gridDim.x;
    tile_end   = num_tiles * (blockIdx.x + 1ull) / gridDim.x;
    tile_step  = 1;
  } else {
    tile_begin = blockIdx.x;
    tile_end   = num_tiles;
    tile_step  = gridDim.x;
  }

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------ producer
    if (lane == 0 && kSpread) {
      uint32_t i = 0;
      bool ok = true;
      for (unsigned long long unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x) {
        const unsigned long long seg0 = unit * kConsumerWarps;
        const unsigned long long left = p.num_segments - seg0;
        const uint32_t segs = left < (unsigned long long)kConsumerWarps ? (uint32_t)left : kConsumerWarps;
        for (int j = 0; j < G; ++j, ++i) {
          const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1u)) { ok = false; break; }
          mbar_arrive_expect_tx(full0 + 8 * s, segs * kSliceBytes);
          for (uint32_t w = 0; w < segs; ++w)  // slice j of segment seg0 + w
            tma_load_1d(ring_u32 + s * kTileBytes + w * kSliceBytes,
                        p.in + ((seg0 + w) * G + j) * (unsigned long long)kSliceBytes, kSliceBytes,
                        full0 + 8 * s);
        }
      }
    } else if (lane == 0) {
      uint32_t i = 0;
      for (unsigned long long tile = tile_begin; tile < tile_end; tile += tile_step, ++i) {
        const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u)) break;
        const unsigned long long off = tile * kTileBytes;
        const unsigned long long rem = total_bytes - off;
        const uint32_t bytes = rem < (unsigned long long)kTileBytes ? (uint32_t)rem : kTileBytes;
        if (tile == p.test_skip_tile) continue;  // test hook: this stage's barrier is never armed
        mbar_arrive_expect_tx(full0 + 8 * s, bytes);
        tma_load_1d(ring_u32 + s * kTileBytes, p.in + off, bytes, full0 + 8 * s);
      }
    }
  } else {
    // ----------------------------------------------------------- consumers
    const bool out_f32 = p.out_is_f32 != 0;
    bool dead          = false;  // a wait ran out: keep the barrier protocol, skip the work
    // running state of warp 0 / lane 0 for the long class
    double run_val    = 0.0;
    long long run_seg = -1;
    bool run_is_head  = false;
    // segment of the next tile and the tile's position inside it (long class, warp 0 lane 0)
    long long next_seg = 0;
    unsigned long long tile_in_seg = 0;
    if (SC == kClassLong && !single) {
      next_seg    = (long long)(tile_begin / p.tiles_per_segment);
      tile_in_seg = tile_begin % p.tiles_per_segment;
    }
    if (SC == kClassLong && warp == 0 && lane == 0) {
      p.bound_seg[2 * blockIdx.x] = -1;
      p.bound_seg[2 * blockIdx.x + 1] = -1;
    }
    // Collective over the consumer warps: add up their running sums of segment run_seg and
    // write the result where it belongs -- the output if this CTA saw the whole segment, else
    // one of the CTA's two boundary records (head: began in an earlier CTA; tail: goes on).
    uint32_t flushes = 0;
    auto flush_segment = [&](bool segment_complete) {
      const uint32_t buf = flushes++ & 1u;
      if (lane == 0) warp_sum[buf][warp] = run_val;
      consumer_sync();
      if (warp == 0 && lane == 0) {
        double total = 0.0;
        for (int w = 0; w < kConsumerWarps; ++w) total += warp_sum[buf][w];
        if (run_is_head) {
          p.bound_val[2 * blockIdx.x] = total;
          p.bound_seg[2 * blockIdx.x] = run_seg;
        } else if (segment_complete) {
          store_seg(p.out, out_f32, run_seg, (float)total);
          if (p.out_f64) p.out_f64[run_seg] = total;
        } else {
          p.bound_val[2 * blockIdx.x + 1] = total;
          p.bound_seg[2 * blockIdx.x + 1] = run_seg;
        }
        // no fence here: this is thread 0, which fences once before it takes the completion
        // ticket below (a fence per segment costs more than the segment's tiles)
      }
    };

    if constexpr (kSpread) {
      uint32_t i = 0;
      for (unsigned long long unit = blockIdx.x; unit < num_units; unit += gridDim.x) {
        const unsigned long long seg = unit * kConsumerWarps + warp;
        const bool valid = seg < p.num_segments;  // else the stage holds nothing for this warp
        float acc_h = 0.f, acc_l = 0.f;  // compensated pair: exact hi-part sum, lo parts + round-off
#pragma unroll 1
        for (int j = 0; j < G; ++j, ++i) {
          const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
          if (!dead && !mbar_wait(full0 + 8 * s, ph)) dead = true;
          float2 tot = make_float2(0.f, 0.f);
          if (!dead && valid) {
            const uint8_t* slice = ring + s * kTileBytes + warp * kSliceBytes;
            if constexpr (kTensor)
              tot = reduce_slice<SC>(slice, p.out, out_f32, 0, 0, lane);
            else
              tot = shuffle_reduce_slice<SC>(slice, p.out, out_f32, 0, 0, lane);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + 8 * s);
          pair_add(acc_h, acc_l, tot.x, tot.y);
        }
        if (lane == 0 && valid && !dead) store_seg(p.out, out_f32, seg, acc_h + acc_l);
      }
    }

    uint32_t i = 0;
    for (unsigned long long tile = kSpread ? tile_end : tile_begin; tile < tile_end; tile += tile_step, ++i) {
      const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
      if (!dead && !mbar_wait(full0 + 8 * s, ph)) dead = true;

      uint8_t* slice = ring + s * kTileBytes + warp * kSliceBytes;
      const unsigned long long slice_off = tile * kTileBytes + (unsigned long long)warp * kSliceBytes;
      const long long left = (long long)total_bytes - (long long)slice_off;
      const int valid_bytes = left <= 0 ? 0 : (left < kSliceBytes ? (int)left : kSliceBytes);
      float2 tot = make_float2(0.f, 0.f);
      if (!dead && valid_bytes > 0) {
        if (valid_bytes < kSliceBytes) zero_slice_tail(slice, valid_bytes, lane);
        constexpr int S = SC <= 11 ? (1 << SC) : kSliceElems;
        if constexpr (kTensor)
          tot = reduce_slice<SC>(slice, p.out, out_f32, slice_off / (2ull * S),
                                 valid_bytes / (2 * S), lane);
        else
          tot = shuffle_reduce_slice<SC>(slice, p.out, out_f32, slice_off / (2ull * S),
                                         valid_bytes / (2 * S), lane);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);

      if constexpr (SC == kClassLong) {
        // Long segments: every warp keeps its own running sum of the current segment and the
        // warps only meet when the segment changes (all warps track the segment of a tile the
        // same way, so the meeting is collective).  One segment: they meet once, at the end.
        if (!single) {
          if (run_seg >= 0 && ++tile_in_seg == p.tiles_per_segment) {  // no 64-bit division per tile
            tile_in_seg = 0;
            ++next_seg;
          }
          if (next_seg != run_seg) {
            if (run_seg >= 0) flush_segment(/*segment_complete=*/true);
            run_seg     = next_seg;
            run_val     = 0.0;
            run_is_head = tile_in_seg != 0;  // began in an earlier CTA
          }
        }
        run_val += (double)tot.x + (double)tot.y;
      }
    }

    if constexpr (SC == kClassLong) {
      if (single) {
        run_seg     = 0;
        run_is_head = true;  // every CTA holds a piece of the one segment
      }
      if (run_seg >= 0 || single)
        flush_segment(/*segment_complete=*/!single && (tile_end % p.tiles_per_segment) == 0);
    }
  }

  if constexpr (SC == kClassLong) {
    // The last CTA to finish stitches together the segments that cross CTA
    // boundaries, in CTA order: deterministic, and no second launch.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      s_is_last = (atomicAdd(p.done_counter, 1u) == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_is_last) {
      __threadfence();
      // Stage the 2 * gridDim.x boundary records in the (now idle) ring with
      // all threads, then add up each segment's records in CTA order.
      double* sh_val       = reinterpret_cast<double*>(ring);
      long long* sh_seg    = reinterpret_cast<long long*>(ring + 16384);
      const unsigned int n = 2 * gridDim.x;  // the host keeps gridDim.x <= 1024
      for (unsigned int k = threadIdx.x; k < n; k += kThreads) {
        sh_seg[k] = __ldcg(&p.bound_seg[k]);
        sh_val[k] = __ldcg(&p.bound_val[k]);
      }
      __syncthreads();
      if (single) {
        // every record belongs to segment 0: fixed-shape tree sum over all threads
        double v = 0.0;
        for (unsigned int k = threadIdx.x; k < n; k += kThreads)
          if (sh_seg[k] >= 0) v += sh_val[k];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        __syncthreads();  // everyone has read its records; reuse sh_val for the warp sums
        if (lane == 0) sh_val[warp] = v;
        __syncthreads();
        if (threadIdx.x == 0) {
          double total = 0.0;
          for (int w = 0; w < kThreads / 32; ++w) total += sh_val[w];
          store_seg(p.out, p.out_is_f32 != 0, 0, (float)total);
          if (p.out_f64) p.out_f64[0] = total;
        }
      } else {
        // The records are in CTA order, so those of one segment are neighbours (with empty ones,
        // seg < 0, in between).  The first record of each segment adds up its group, in order:
        // as many threads at work as there are segments among the records, and a fixed order of
        // additions whatever that number is.
        const bool out_f32 = p.out_is_f32 != 0;
        for (unsigned int k = threadIdx.x; k < n; k += kThreads) {
          const long long seg = sh_seg[k];
          if (seg < 0) continue;
          bool first = true;  // no earlier record of this segment?
          for (unsigned int j = k; j-- > 0;) {
            if (sh_seg[j] < 0) continue;
            first = sh_seg[j] != seg;
            break;
          }
          if (!first) continue;
          double total = sh_val[k];
          for (unsigned int j = k + 1; j < n; ++j) {
            if (sh_seg[j] < 0) continue;
            if (sh_seg[j] != seg) break;
            total += sh_val[j];
          }
          store_seg(p.out, out_f32, seg, (float)total);
          if (p.out_f64) p.out_f64[seg] = total;
        }
      }
    }
  }
}

}  // namespace TCU_NS
