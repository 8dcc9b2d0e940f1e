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
//
// A tile's prefix is known only when every earlier tile of the machine has
// been loaded and summed, several microseconds after its own load -- more
// data than shared memory can hold at full bandwidth.  So a tile is not kept
// on chip while it waits: it is loaded twice, the second time out of L2.
//   producer A: ticket, TMA load (L2 evict-last)       -> fullA[a]
//   pass-1 warps: slice totals, row carries (kept in a small queue slot q)
//                                                      -> p1done[q], emptyA[a]
//   one of the look-back warps: publish aggregate, walk back, publish prefix
//                                                      -> resolved[q]
//   producer B: waits for resolved[q], loads the tile again (L2 evict-first)
//                                                      -> fullB[b]
//   pass-2 warps: the scan, seeded; stores             -> emptyB[b], qfree[q]
// Ring A only ever holds tiles in flight or being summed, ring B only tiles
// whose prefix is already known; what waits for a look-back is a 4 KiB queue
// slot, not a 32 KiB tile.
#pragma once

#include "scan_kernels.cuh"

namespace TCU_NS {

// Ring and queue depths are measured optima (sweep at 2^30 elements): rings of
// 2 + 3 stages and 10 queue slots; 6 look-back warps keep up with the tiles.
constexpr int kRingA = 2;   // stages of the first-read ring
constexpr int kRingB = 3;   // stages of the second-read ring
constexpr int kQueue = 10;  // tiles between their first and second read, per CTA
constexpr int kLookbackWarps = 6;
// A look-back warp's first tile must be in the first pass over the queue: a
// wait for a later phase on a fresh barrier would fall through.
static_assert(kLookbackWarps <= kQueue, "at most one look-back warp per queue slot");
constexpr int kLookbackCtasPerSm    = 1;
// Warp roles: [0,8) pass 1, [8,16) pass 2, 16 producer A, 17 producer B, 18.. look-back.
constexpr int kPass2Warp0           = kConsumerWarps;
constexpr int kProducerAWarp        = 2 * kConsumerWarps;
constexpr int kProducerBWarp        = kProducerAWarp + 1;
constexpr int kLookbackWarp0        = kProducerBWarp + 1;
constexpr int kLookbackThreads      = (2 * kConsumerWarps + 2 + kLookbackWarps) * 32;
// one float4 (row carries) per pass-1 lane, kept from pass 1 to pass 2 (summing
// the rows of the slice again in pass 2 instead measured 0.55 against 0.88)
constexpr bool kSaveCarries         = true;
constexpr int kCarryBytesPerSlot    = kSaveCarries ? kConsumerWarps * 32 * 16 : 0;
constexpr int kLookbackDynSmemBytes =
    (kRingA + kRingB) * kTileBytes + kQueue * kCarryBytesPerSlot + 1024;
constexpr uint32_t kNoEnd = 0xffffffffu;

constexpr unsigned long long kTileEnd = ~0ull;
constexpr unsigned kStateAggregate = 1u, kStateInclusive = 2u;
constexpr unsigned long long kBlockTiles = 32;  // tiles per second-level status word

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

// Run by all 32 lanes of one warp.  Walks the status words from index `last`
// downwards, adding aggregates, until it meets an inclusive prefix (returns
// with found_inclusive = true: the sum is a complete prefix) or has passed
// index `first` (found_inclusive = false: the sum covers [first, last] only).
// Each poll reads one word per lane (256 bytes per warp); words already summed
// are never read again, and a poll that makes no progress backs off.
//
// `prefetched` (with use_prefetched) is the word this lane would read in the
// first window, loaded earlier by the caller -- the block-level window is
// fetched in the same round trip as the tile-level one.
__device__ __forceinline__ double look_back(const unsigned long long* status, long long last,
                                            long long first, int lane, bool& found_inclusive,
                                            bool use_prefetched = false,
                                            unsigned long long prefetched = 0ull) {
  double sum     = 0.0;
  uint32_t polls = 0;
  found_inclusive = false;
  while (last >= first) {
    const long long idx = last - lane;
    const bool valid    = idx >= first;
    const unsigned long long w =
        use_prefetched ? prefetched : (valid ? status_load(status + idx) : 0ull);
    use_prefetched = false;
    const unsigned state = static_cast<unsigned>(w & 3ull);
    const unsigned not_ready = __ballot_sync(0xffffffffu, valid && state == 0u);
    const unsigned stops     = __ballot_sync(0xffffffffu, !valid || state == kStateInclusive);
    const int z = not_ready ? __ffs(not_ready) - 1 : 32;  // first word nothing is published in
    const int t = stops ? __ffs(stops) - 1 : 32;          // first inclusive word / end of range
    const int take = z < t ? z : t;                       // lanes [0, take) hold aggregates
    double v = 0.0;
    if (lane < take || (lane == t && t < z && valid))
      v = __longlong_as_double(static_cast<long long>(w & ~3ull));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    sum += v;
    if (t < z) {  // reached an inclusive prefix, or walked past `first`
      found_inclusive = __shfl_sync(0xffffffffu, valid ? 1 : 0, t) != 0;
      return sum;
    }
    last -= take;
    if (take == 0) {  // the nearest word is still empty: wait for its tile, but not forever
      if (++polls > wait_limit(&g_wait_limits.status)) {
        if (lane == 0) raise_error(kErrLookbackTimeout);
        return sum;  // wrong result, flagged, but no hang
      }
      __nanosleep(polls < 8 ? 64 : 256);
    }
  }
  return sum;
}

// try_wait loop that also gives up when the CTA-wide abort flag is raised or,
// for the look-back warps, when the tile stream has ended before index `idx`.
__device__ __forceinline__ bool mbar_wait_or_stop(uint32_t bar, uint32_t parity,
                                                  volatile uint32_t* abort_flag,
                                                  volatile uint32_t* end_index, uint32_t idx) {
  uint32_t limit = kFastAttempts;  // the real bound is fetched once these have failed
  for (uint32_t attempt = 0; attempt < limit; ++attempt) {
    if (mbar_try_wait(bar, parity)) return true;
    if (attempt + 1 == kFastAttempts) limit = wait_limit(&g_wait_limits.barrier);
    if (*abort_flag) return false;
    if (end_index != nullptr && *end_index <= idx) return false;
  }
  raise_error(kErrBarrierTimeout);
  *abort_flag = 1u;
  return false;
}

// kSwz: tiles arrive through the tensor map `tmap` (2-D view {64, num_elems/64},
// 128-byte swizzle; needs num_elems % 64 == 0), which makes the row-strided
// 8-byte loads of both passes conflict-free; otherwise through linear copies.
template <bool OUT32, bool kSwz>
__global__ void __launch_bounds__(kLookbackThreads, kLookbackCtasPerSm)
    scan_lookback_kernel(const ScanParams p, const __grid_constant__ CUtensorMap tmap) {
  constexpr int SC = 15;  // row-stream geometry, rows always chained
  constexpr int NA = kRingA, NB = kRingB, NQ = kQueue;
  extern __shared__ uint8_t dyn_smem[];
  // fullA | emptyA | fullB | emptyB | p1done | resolved | qfree
  __shared__ __align__(8) uint64_t bars[2 * NA + 2 * NB + 3 * NQ];
  __shared__ unsigned long long slot_tile[NQ];
  __shared__ float2 part[NQ][kConsumerWarps];      // slice totals (exact hi, lo)
  __shared__ float2 xcarry[NQ][kConsumerWarps];    // everything before a slice in its segment: (coarse, rest)
  __shared__ uint32_t s_abort, s_end_index;

  // 1 KiB-aligned rings: the swizzle pattern repeats every 1024 bytes
  uint8_t* ring_a = dyn_smem + ((1024u - (smem_u32(dyn_smem) & 1023u)) & 1023u);
  uint8_t* ring_b = ring_a + NA * kTileBytes;
  float4* carries = reinterpret_cast<float4*>(ring_b + NB * kTileBytes);  // [NQ][8][32]
  const uint32_t ring_a_u32 = smem_u32(ring_a), ring_b_u32 = smem_u32(ring_b);
  const uint32_t full_a0 = smem_u32(&bars[0]), empty_a0 = full_a0 + 8 * NA;
  const uint32_t full_b0 = empty_a0 + 8 * NA, empty_b0 = full_b0 + 8 * NB;
  const uint32_t p1done0 = empty_b0 + 8 * NB, resolved0 = p1done0 + 8 * NQ,
                 qfree0 = resolved0 + 8 * NQ;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &s_abort;
  volatile uint32_t* end_index  = &s_end_index;

  if (threadIdx.x == 0) {
    for (int a = 0; a < NA; ++a) {
      mbar_init(full_a0 + 8 * a, 1);
      mbar_init(empty_a0 + 8 * a, kConsumerWarps);
    }
    for (int b = 0; b < NB; ++b) {
      mbar_init(full_b0 + 8 * b, 1);
      mbar_init(empty_b0 + 8 * b, kConsumerWarps);
    }
    for (int q = 0; q < NQ; ++q) {
      mbar_init(p1done0 + 8 * q, kConsumerWarps);
      mbar_init(resolved0 + 8 * q, 1);
      mbar_init(qfree0 + 8 * q, kConsumerWarps);
    }
    s_abort     = 0u;
    s_end_index = kNoEnd;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_prologue();  // nothing above touched global memory

  const unsigned long long total_bytes = p.num_elems * 2ull;
  const unsigned long long num_tiles   = (total_bytes + kTileBytes - 1) / kTileBytes;

  // one tile into one ring stage, by either kind of copy
  auto load_tile = [&](uint32_t dst, unsigned long long tile, uint32_t bar, uint64_t policy) {
    const unsigned long long off = tile * kTileBytes;
    const unsigned long long rem = total_bytes - off;
    const uint32_t bytes = rem < (unsigned long long)kTileBytes ? (uint32_t)rem : kTileBytes;
    if constexpr (kSwz) {
      // the whole box always arrives: rows past the end of the array come as zeros
      mbar_arrive_expect_tx(bar, kTileBytes);
      tma_load_2d_hint(dst, &tmap, 0, (int)(tile * kTileRows), bar, policy);
    } else {
      mbar_arrive_expect_tx(bar, bytes);
      tma_load_1d_hint(dst, p.in + off, bytes, bar, policy);
    }
  };

  if (warp == kProducerAWarp) {
    // ---------------------------------------------------------- producer A
    if (lane == 0) {
      const uint64_t keep = l2_policy_evict_last();  // the tile is read again within microseconds
      for (uint32_t i = 0;; ++i) {
        const uint32_t a = i % NA, q = i % NQ;
        if (!mbar_wait_or_stop(qfree0 + 8 * q, ((i / NQ) & 1u) ^ 1u, abort_flag, nullptr, 0)) break;
        if (!mbar_wait_or_stop(empty_a0 + 8 * a, ((i / NA) & 1u) ^ 1u, abort_flag, nullptr, 0)) break;
        const unsigned long long tile = atomicAdd(p.ticket, 1u);
        if (tile >= num_tiles) {
          slot_tile[q] = kTileEnd;
          mbar_arrive(full_a0 + 8 * a);  // release: the pass-1 warps see the end marker
          break;
        }
        slot_tile[q] = tile;
        load_tile(ring_a_u32 + a * kTileBytes, tile, full_a0 + 8 * a, keep);
      }
    }
    return;
  }

  if (warp == kProducerBWarp) {
    // ---------------------------------------------------------- producer B
    if (lane == 0) {
      const uint64_t drop = l2_policy_evict_first();  // last use of these lines
      for (uint32_t k = 0;; ++k) {
        const uint32_t b = k % NB, q = k % NQ;
        if (!mbar_wait_or_stop(resolved0 + 8 * q, (k / NQ) & 1u, abort_flag, end_index, k)) break;
        if (!mbar_wait_or_stop(empty_b0 + 8 * b, ((k / NB) & 1u) ^ 1u, abort_flag, nullptr, 0)) break;
        load_tile(ring_b_u32 + b * kTileBytes, slot_tile[q], full_b0 + 8 * b, drop);
      }
    }
    return;
  }

  if (warp >= kLookbackWarp0) {
    // ------------------------------------------------------ look-back warps
    for (uint32_t i = warp - kLookbackWarp0;; i += kLookbackWarps) {
      const uint32_t q = i % NQ, ph = (i / NQ) & 1u;
      if (!mbar_wait_or_stop(p1done0 + 8 * q, ph, abort_flag, end_index, i)) break;
      const unsigned long long tile = slot_tile[q];
      // the tile's total, and in lane w what the tile holds before slice w (double arithmetic is
      // slow on this part: it is done here, once per tile, not in the eight pass-2 warps)
      double agg = 0.0, pre = 0.0;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const double v = (double)part[q][w].x + (double)part[q][w].y;
        if (w < lane) pre += v;
        agg += v;
      }
      // Two levels: tiles inside a block of kBlockTiles tiles, then whole blocks
      // (block b of a segment = tiles [seg_first + b*32, +32)).  A walk is at
      // most one window inside the block plus about one window over blocks,
      // however many tiles are in flight on the machine.
      const unsigned long long tps       = p.tiles_per_segment;
      const unsigned long long seg_first = (tile / tps) * tps;
      const unsigned long long rel       = tile - seg_first;
      const unsigned long long blk       = rel / kBlockTiles;            // block inside the segment
      const unsigned long long blk_first = seg_first + blk * kBlockTiles;
      // block status words of all segments, one run of words per segment
      const unsigned long long blk_base = (seg_first / tps) * ((tps + kBlockTiles - 1) / kBlockTiles);
      const bool closes_block = (rel % kBlockTiles) == kBlockTiles - 1 && rel + 1 < tps;
      double excl = 0.0;
      if (rel == 0) {
        if (tile == 0 && p.shard_totals != nullptr)  // earlier shards of a multi-GPU scan
          for (int k = 0; k < p.shard_index; ++k) excl += p.shard_totals[k];
        if (lane == 0) status_store(p.tile_status + tile, excl + agg, kStateInclusive);
      } else {
        if (lane == 0) status_store(p.tile_status + tile, agg, kStateAggregate);
        // first window of the block-level walk, in flight together with the tile-level one
        const long long blk_last = (long long)(blk_base + blk) - 1;
        const long long blk_idx  = blk_last - lane;
        const unsigned long long blk_word =
            blk_idx >= (long long)blk_base ? status_load(p.block_status + blk_idx) : 0ull;
        bool complete = false;
        const double in_block = look_back(p.tile_status, (long long)tile - 1,
                                          (long long)blk_first, lane, complete);
        double before_block = 0.0;
        if (!complete) {  // blk > 0 here: block 0 starts with the segment's inclusive first tile
          if (closes_block && lane == 0)
            status_store(p.block_status + blk_base + blk, in_block + agg, kStateAggregate);
          bool dummy;
          before_block = look_back(p.block_status, blk_last, (long long)blk_base, lane, dummy,
                                   /*use_prefetched=*/true, blk_word);
        }
        excl = before_block + in_block;
        if (lane == 0) status_store(p.tile_status + tile, excl + agg, kStateInclusive);
      }
      // the last tile of a block publishes the prefix through the block
      if (closes_block && lane == 0)
        status_store(p.block_status + blk_base + blk, excl + agg, kStateInclusive);
      // Everything before slice w, as two floats: xh a multiple of 2^-13 (what the hi parts are
      // made of), xl the small rest.
      if (lane < kConsumerWarps) {
        const double carry    = excl + pre;
        const double carry_hi = rint(carry * 8192.0) * (1.0 / 8192.0);
        const float xh = (float)carry_hi;
        xcarry[q][lane] = make_float2(xh, (float)(carry - (double)xh));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(resolved0 + 8 * q);  // release: xcarry is visible to the waiters
    }
    return;
  }

  // --------------------------------------------------------------- consumers
  using Geom = ScanGeom<SC>;
  const int cw = warp & (kConsumerWarps - 1);  // the slice this warp owns, in either pass
  const int g = lane >> 2, t = lane & 3;
  const ScanOperands ops = make_scan_operands(lane, p.exclusive != 0);
  const Acc zero{0.f, 0.f, 0.f, 0.f};

  struct SliceView {
    uint8_t* slice;
    unsigned long long slice_off;
    int valid_bytes;
  };
  auto slice_view = [&](uint8_t* stage, unsigned long long tile) {
    SliceView v;
    v.slice     = stage + cw * kSliceBytes;
    v.slice_off = tile * kTileBytes + (unsigned long long)cw * kSliceBytes;
    const long long left = (long long)total_bytes - (long long)v.slice_off;
    v.valid_bytes = left <= 0 ? 0 : (left < kSliceBytes ? (int)left : kSliceBytes);
    return v;
  };

  // pass 1 of local tile i: slice total and row carries.  false = no such tile.
  auto pass1 = [&](uint32_t i) -> bool {
    const uint32_t a = i % NA, q = i % NQ;
    if (!mbar_wait_or_stop(full_a0 + 8 * a, (i / NA) & 1u, abort_flag, nullptr, 0)) return false;
    const unsigned long long tile = slot_tile[q];
    if (tile == kTileEnd) {
      if (lane == 0) *end_index = i;  // lets producer B, the look-back and the pass-2 warps leave
      return false;
    }
    const SliceView v = slice_view(ring_a + a * kTileBytes, tile);
    const bool active = v.valid_bytes > 0;
    if constexpr (!kSwz)
      if (active && v.valid_bytes < kSliceBytes) zero_slice_tail(v.slice, v.valid_bytes, lane);
    Acc tot_h = zero, tot_l = zero;
    if (active) {
      const SliceAddr<Geom, kSwz> addr(v.slice, g, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t ah[4], al[4];
        load_split(addr, j, ah, al);
        tot_h = mma_ones(ah, tot_h);
        tot_l = mma_ones(al, tot_l);
      }
    }
    float ch_lo, cl_lo, ch_hi, cl_hi, slice_h, slice_l;
    row_carries<16>(tot_h, tot_l, g, ch_lo, cl_lo, ch_hi, cl_hi, slice_h, slice_l);
    if constexpr (kSaveCarries)
      carries[(q * kConsumerWarps + cw) * 32 + lane] = make_float4(ch_lo, cl_lo, ch_hi, cl_hi);
    if (lane == 0) part[q][cw] = make_float2(active ? slice_h : 0.f, active ? slice_l : 0.f);
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(p1done0 + 8 * q);
      mbar_arrive(empty_a0 + 8 * a);  // the stage can take the next first read
    }
    return true;
  };

  // pass 2 of local tile k: the scan proper, seeded with everything before the slice
  auto pass2 = [&](uint32_t k) -> bool {
    const uint32_t b = k % NB, q = k % NQ;
    // producer B loads the tile only after its look-back; the second wait returns at once
    // and makes xcarry visible to this warp as well
    if (!mbar_wait_or_stop(full_b0 + 8 * b, (k / NB) & 1u, abort_flag, end_index, k)) return false;
    if (!mbar_wait_or_stop(resolved0 + 8 * q, (k / NQ) & 1u, abort_flag, end_index, k)) return false;
    const unsigned long long tile = slot_tile[q];
    const SliceView v = slice_view(ring_b + b * kTileBytes, tile);
    // Everything before this slice, as the look-back warp left it.  While xh is below 2^10 it
    // rides through the MMAs' accumulator operand with the row carries and every sum stays
    // exact; a larger one would push the row sums out of the accumulator's 24 bits, so it is
    // held back and added to each output last.
    const float xh = xcarry[q][cw].x, xl = xcarry[q][cw].y;
    const bool fold = fabsf(xh) < 1024.f;
    const float xf = fold ? xh : 0.f, big = fold ? 0.f : xh;
    if (v.valid_bytes > 0) {
      if constexpr (!kSwz)
        if (v.valid_bytes < kSliceBytes) zero_slice_tail(v.slice, v.valid_bytes, lane);
      const SliceAddr<Geom, kSwz> addr(v.slice, g, t);
      float4 c;
      if constexpr (kSaveCarries) {
        c = carries[(q * kConsumerWarps + cw) * 32 + lane];
      } else {
        Acc tot_h = zero, tot_l = zero;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t ah[4], al[4];
          load_split(addr, j, ah, al);
          tot_h = mma_ones(ah, tot_h);
          tot_l = mma_ones(al, tot_l);
        }
        float slice_h, slice_l;
        row_carries<16>(tot_h, tot_l, g, c.x, c.y, c.z, c.w, slice_h, slice_l);
      }
      RowCarry rc{c.x + xf, c.y + xl, c.z + xf, c.w + xl};
      const unsigned long long elem_base = v.slice_off / 2;
      const int valid_elems = v.valid_bytes / 2;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t ah[4], al[4];
        load_split(addr, j, ah, al);
        scan_step_independent<SC, OUT32, /*kStream=*/true>(j, ah, al, ops, rc, p.out, elem_base,
                                                           valid_elems, g, t, big);
      }
    }
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(empty_b0 + 8 * b);
      mbar_arrive(qfree0 + 8 * q);  // slot_tile, part, carries and xcarry of the slot are free
    }
    return true;
  };

  if (warp < kPass2Warp0) {
    for (uint32_t i = 0; pass1(i); ++i) {}
  } else {
    for (uint32_t k = 0; pass2(k); ++k) {}
  }
}

}  // namespace TCU_NS
