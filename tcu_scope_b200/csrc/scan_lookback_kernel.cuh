// Inclusive scan for segments longer than one tile, and the full scan: the
// same tensor-core slice scan as seg_scan_kernel, plus a single-pass decoupled
// look-back chain across tiles.  Takes the place of the reference's second and
// third kernels (library exclusive scan of the partial sums + add_partial_sums,
// src/prefixsum/wmma_3kers.cu:66-70, src/prefixsum/kernel.cuh:30-43), which
// re-read and re-write the whole output.
//
// Each tile owns one 64-bit status word: a double whose two lowest mantissa
// bits carry the state (0 = nothing yet, 1 = tile aggregate, 2 = inclusive
// prefix up to and including the tile), so that value and state travel in one
// atomic store.  Tiles are handed out by an atomic ticket, which guarantees
// that every predecessor of a tile already belongs to a running CTA: a wait
// can only be on work that is making progress.  Every poll loop is bounded.
#pragma once

#include "scan_kernels.cuh"

namespace tcu {

constexpr int kLookbackStages       = 3;
constexpr int kLookbackCtasPerSm    = 2;  // one CTA computes while the other looks back
constexpr int kLookbackDynSmemBytes = kLookbackStages * kTileBytes + 128;
constexpr unsigned long long kTileEnd = ~0ull;
constexpr unsigned kStateAggregate = 1u, kStateInclusive = 2u;

__device__ __forceinline__ void status_store(unsigned long long* p, double v, unsigned state) {
  const unsigned long long w =
      (static_cast<unsigned long long>(__double_as_longlong(v)) & ~3ull) | state;
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

__device__ __forceinline__ unsigned long long status_load(const unsigned long long* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}

// Run by all 32 lanes of one warp.  Returns the sum of the aggregates of the
// tiles [seg_first, tile) -- the exclusive prefix of `tile` inside its segment.
__device__ __forceinline__ double look_back(const unsigned long long* status,
                                            unsigned long long tile,
                                            unsigned long long seg_first, int lane) {
  double excl    = 0.0;
  long long base = static_cast<long long>(tile) - 1;  // lane l inspects tile base - l
  uint32_t polls = 0;
  while (true) {
    const long long idx = base - lane;
    const bool valid    = idx >= static_cast<long long>(seg_first);
    unsigned long long w = 0;
    unsigned state       = kStateAggregate;  // tiles before the segment: never used, see below
    while (true) {
      if (valid) {
        w     = status_load(status + idx);
        state = static_cast<unsigned>(w & 3ull);
      }
      if (__all_sync(0xffffffffu, state != 0u)) break;
      if (++polls > kPollAttempts) {  // give up: wrong result, flagged, but no hang
        if (lane == 0) raise_error(kErrLookbackTimeout);
        return excl;
      }
      __nanosleep(40);
    }
    // The first tile of a segment always publishes an inclusive prefix, so a
    // window that reaches below seg_first contains an inclusive lane before
    // any invalid one; invalid lanes are cut off by the mask below.
    const unsigned incl_mask = __ballot_sync(0xffffffffu, valid && state == kStateInclusive);
    double v = valid ? __longlong_as_double(static_cast<long long>(w & ~3ull)) : 0.0;
    if (incl_mask) {
      const int first = __ffs(incl_mask) - 1;
      if (lane > first) v = 0.0;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    excl += v;
    if (incl_mask) return excl;
    base -= 32;
  }
}

template <bool OUT32>
__global__ void __launch_bounds__(kThreads, kLookbackCtasPerSm)
    scan_lookback_kernel(const ScanParams p) {
  constexpr int SC = 15;  // row-stream geometry, rows always chained
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * kLookbackStages];
  __shared__ unsigned long long stage_tile[kLookbackStages];
  __shared__ float2 part[2][kConsumerWarps];
  __shared__ double tile_excl[2];

  uint8_t* ring = dyn_smem + ((128u - (smem_u32(dyn_smem) & 127u)) & 127u);
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kLookbackStages]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kLookbackStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();

  const unsigned long long total_bytes = p.num_elems * 2ull;
  const unsigned long long num_tiles   = (total_bytes + kTileBytes - 1) / kTileBytes;

  if (warp == kConsumerWarps) {
    if (lane == 0) {
      for (uint32_t i = 0;; ++i) {
        const uint32_t s = i % kLookbackStages, ph = (i / kLookbackStages) & 1u;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u)) break;
        const unsigned long long tile = atomicAdd(p.ticket, 1u);
        if (tile >= num_tiles) {
          stage_tile[s] = kTileEnd;
          mbar_arrive(full0 + 8 * s);  // release: the consumers see the end marker
          break;
        }
        stage_tile[s] = tile;
        const unsigned long long off = tile * kTileBytes;
        const unsigned long long rem = total_bytes - off;
        const uint32_t bytes = rem < (unsigned long long)kTileBytes ? (uint32_t)rem : kTileBytes;
        mbar_arrive_expect_tx(full0 + 8 * s, bytes);
        tma_load_1d(ring_u32 + s * kTileBytes, p.in + off, bytes, full0 + 8 * s);
      }
    }
    return;
  }

  using Geom = ScanGeom<SC>;
  const int g = lane >> 2, t = lane & 3;
  const ScanOperands ops = make_scan_operands(lane);
  const Acc zero{0.f, 0.f, 0.f, 0.f};

  for (uint32_t i = 0;; ++i) {
    const uint32_t s = i % kLookbackStages, ph = (i / kLookbackStages) & 1u;
    // All eight warps wait on the same phase, so they give up together.
    if (!mbar_wait(full0 + 8 * s, ph)) break;
    const unsigned long long tile = stage_tile[s];
    if (tile == kTileEnd) break;

    uint8_t* slice = ring + s * kTileBytes + warp * kSliceBytes;
    const unsigned long long slice_off = tile * kTileBytes + (unsigned long long)warp * kSliceBytes;
    const long long left  = (long long)total_bytes - (long long)slice_off;
    const int valid_bytes = left <= 0 ? 0 : (left < kSliceBytes ? (int)left : kSliceBytes);
    const bool active     = valid_bytes > 0;
    if (active && valid_bytes < kSliceBytes) zero_slice_tail(slice, valid_bytes, lane);

    // ---- pass 1 over the slice: row totals
    Acc tot_h = zero, tot_l = zero;
    if (active) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t ah[4], al[4];
        load_split<Geom>(slice, g, t, j, ah, al);
        tot_h = mma_ones(ah, tot_h);
        tot_l = mma_ones(al, tot_l);
      }
    }
    float ch_lo, cl_lo, ch_hi, cl_hi, slice_h, slice_l;
    row_carries<16>(tot_h, tot_l, g, ch_lo, cl_lo, ch_hi, cl_hi, slice_h, slice_l);
    if (lane == 0) part[i & 1][warp] = make_float2(active ? slice_h : 0.f, active ? slice_l : 0.f);
    consumer_sync();

    // ---- warp 0: publish this tile, find its exclusive prefix
    if (warp == 0) {
      double agg = 0.0;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w)
        agg += (double)part[i & 1][w].x + (double)part[i & 1][w].y;
      const unsigned long long seg_first = (tile / p.tiles_per_segment) * p.tiles_per_segment;
      double excl = 0.0;
      if (tile == seg_first) {
        if (tile == 0 && p.shard_totals != nullptr)  // earlier shards of a multi-GPU scan
          for (int k = 0; k < p.shard_index; ++k) excl += p.shard_totals[k];
        if (lane == 0) status_store(p.tile_status + tile, excl + agg, kStateInclusive);
      } else {
        if (lane == 0) status_store(p.tile_status + tile, agg, kStateAggregate);
        excl = look_back(p.tile_status, tile, seg_first, lane);
        if (lane == 0) status_store(p.tile_status + tile, excl + agg, kStateInclusive);
      }
      if (lane == 0) tile_excl[i & 1] = excl;
    }
    consumer_sync();

    // ---- carry into this slice: tile prefix + earlier slices of the tile, as two floats
    double carry = tile_excl[i & 1];
    for (int w = 0; w < warp; ++w) carry += (double)part[i & 1][w].x + (double)part[i & 1][w].y;
    const float xh = (float)carry;
    const float xl = (float)(carry - (double)xh);

    // ---- pass 2: the scans proper
    if (active) {
      const unsigned long long elem_base = slice_off / 2;
      const int valid_elems = valid_bytes / 2;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t ah[4], al[4];
        load_split<Geom>(slice, g, t, j, ah, al);
        scan_step<SC, OUT32, true>(j, ah, al, ops, ch_lo, cl_lo, ch_hi, cl_hi, xh, xl, p.out,
                                   elem_base, valid_elems, g, t);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);
  }
}

}  // namespace tcu
