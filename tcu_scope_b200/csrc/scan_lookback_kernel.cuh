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
// Inside a CTA the look-back is taken off the critical path.  Tile i goes
//   producer:  TMA load                               -> full[s]
//   consumers: pass 1 (slice totals, row carries)     -> p1done[s]
//   one of 4 look-back warps: publish aggregate, walk back, publish prefix
//                                                     -> resolved[s]
//   consumers: pass 2 (the scan, seeded), stores      -> empty[s]
// and the consumers run pass 1 kLookahead tiles ahead of pass 2, so that a
// tile's aggregate is public long before its successors need it and several
// look-backs per CTA are in flight while the tensor cores stay busy.
#pragma once

#include "scan_kernels.cuh"

namespace tcu {

#ifndef TCU_LB_STAGES
#define TCU_LB_STAGES 6
#endif
#ifndef TCU_LB_SAVE_CARRIES
#define TCU_LB_SAVE_CARRIES 1
#endif
constexpr int kLookbackStages       = TCU_LB_STAGES;
constexpr bool kSaveCarries         = TCU_LB_SAVE_CARRIES != 0;
#ifndef TCU_LOOKAHEAD
#define TCU_LOOKAHEAD 4
#endif
constexpr int kLookahead            = TCU_LOOKAHEAD;  // pass 1 runs this many tiles ahead of pass 2
#ifndef TCU_LB_WARPS
#define TCU_LB_WARPS 6
#endif
constexpr int kLookbackWarps        = TCU_LB_WARPS;
// A look-back warp's first tile must be in the first pass over the ring: a
// wait for a later phase on a fresh barrier would fall through.
static_assert(kLookbackWarps <= kLookbackStages, "at most one look-back warp per ring stage");
constexpr int kLookbackCtasPerSm    = 1;
// Warp roles: [0,8) pass-1 warps, [8,16) pass-2 warps, 16 producer, 17.. look-back.
// Pass 1 and pass 2 of different tiles run at the same time on different warps:
// twice the warps to interleave on each scheduler, which is what the dependent
// MMA / shuffle chains of the two passes need to keep the issue slots busy.
constexpr int kPass2Warp0           = kConsumerWarps;
constexpr int kProducerWarp         = 2 * kConsumerWarps;
constexpr int kLookbackWarp0        = kProducerWarp + 1;
constexpr int kLookbackThreads      = (2 * kConsumerWarps + 1 + kLookbackWarps) * 32;
// one float4 (row carries) per consumer lane, kept from pass 1 to pass 2
constexpr int kCarryBytesPerStage   = kSaveCarries ? kConsumerWarps * 32 * 16 : 0;
constexpr int kLookbackDynSmemBytes =
    kLookbackStages * (kTileBytes + kCarryBytesPerStage) + 1024;
constexpr uint32_t kNoEnd = 0xffffffffu;

#ifdef TCU_LB_PROFILE
// debug counters (ns): [0] look-back time sum [1] tiles [2] look-back max
// [3] pass-2 warp 8 wait for resolved  [4] pass-1 warp 0 wait for full  [5] pass-1 compute
// [6] pass-2 compute  [7] producer wait for empty
// [8] in-block walk ns [9] block walk ns [10] in-block empty polls [11] block empty polls
// [12] ns from the tile's ticket to the start of its look-back
__device__ unsigned long long g_lb_stats[16];
__device__ unsigned long long g_lb_polls_scratch;
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define LB_T0() const unsigned long long lb_t0 = gtime()
#define LB_ADD(slot, cond) do { if (cond) atomicAdd(&g_lb_stats[slot], gtime() - lb_t0); } while (0)
#else
#define LB_T0()
#define LB_ADD(slot, cond)
#endif
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
#ifdef TCU_LB_PROFILE
  const bool use_prefetched_slot = use_prefetched;  // block-level walks are the prefetched ones
#endif
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
#ifdef TCU_LB_PROFILE
      if (lane == 0) atomicAdd(&g_lb_stats[status == nullptr ? 10 : 10 + (int)use_prefetched_slot], 1ull);
#endif
      if (++polls > kPollAttempts) {
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
  for (uint32_t attempt = 0; attempt < kWaitAttempts; ++attempt) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    if (done) return true;
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
  constexpr int NS = kLookbackStages;
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[4 * NS];  // full | p1done | resolved | empty
  __shared__ unsigned long long stage_tile[NS];
  __shared__ float2 part[NS][kConsumerWarps];      // slice totals (exact hi, lo)
  __shared__ double tile_excl[NS];                 // exclusive prefix of the tile in its segment
  __shared__ uint32_t s_abort, s_end_index;

  // 1 KiB-aligned ring: the swizzle pattern repeats every 1024 bytes
  uint8_t* ring = dyn_smem + ((1024u - (smem_u32(dyn_smem) & 1023u)) & 1023u);
  float4* carries = reinterpret_cast<float4*>(ring + NS * kTileBytes);  // [NS][8][32]
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t full0 = smem_u32(&bars[0]), p1done0 = smem_u32(&bars[NS]),
                 resolved0 = smem_u32(&bars[2 * NS]), empty0 = smem_u32(&bars[3 * NS]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &s_abort;
  volatile uint32_t* end_index  = &s_end_index;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(p1done0 + 8 * s, kConsumerWarps);
      mbar_init(resolved0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kConsumerWarps);
    }
    s_abort     = 0u;
    s_end_index = kNoEnd;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_prologue();  // nothing above touched global memory

  const unsigned long long total_bytes = p.num_elems * 2ull;
  const unsigned long long num_tiles   = (total_bytes + kTileBytes - 1) / kTileBytes;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      for (uint32_t i = 0;; ++i) {
        const uint32_t s = i % NS, ph = (i / NS) & 1u;
        {
          LB_T0();
          if (!mbar_wait_or_stop(empty0 + 8 * s, ph ^ 1u, abort_flag, nullptr, 0)) break;
          LB_ADD(7, true);
        }
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
        if constexpr (kSwz) {
          // the whole box always arrives: rows past the end of the array come as zeros
          mbar_arrive_expect_tx(full0 + 8 * s, kTileBytes);
          tma_load_2d(ring_u32 + s * kTileBytes, &tmap, 0, (int)(tile * kTileRows), full0 + 8 * s);
        } else {
          mbar_arrive_expect_tx(full0 + 8 * s, bytes);
          tma_load_1d(ring_u32 + s * kTileBytes, p.in + off, bytes, full0 + 8 * s);
        }
      }
    }
    return;
  }

  if (warp >= kLookbackWarp0) {
    // ------------------------------------------------------ look-back warps
    for (uint32_t i = warp - kLookbackWarp0;; i += kLookbackWarps) {
      const uint32_t s = i % NS, ph = (i / NS) & 1u;
      if (!mbar_wait_or_stop(p1done0 + 8 * s, ph, abort_flag, end_index, i)) break;
      const unsigned long long tile = stage_tile[s];
      LB_T0();
      double agg = 0.0;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) agg += (double)part[s][w].x + (double)part[s][w].y;
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
#ifdef TCU_LB_PROFILE
        const unsigned long long lb_t1 = gtime();
        if (lane == 0) atomicAdd(&g_lb_stats[8], lb_t1 - lb_t0);
#endif
        double before_block = 0.0;
        if (!complete) {  // blk > 0 here: block 0 starts with the segment's inclusive first tile
          if (closes_block && lane == 0)
            status_store(p.block_status + blk_base + blk, in_block + agg, kStateAggregate);
          bool dummy;
          before_block = look_back(p.block_status, blk_last, (long long)blk_base, lane, dummy,
                                   /*use_prefetched=*/true, blk_word);
        }
        excl = before_block + in_block;
#ifdef TCU_LB_PROFILE
        if (lane == 0) atomicAdd(&g_lb_stats[9], gtime() - lb_t1);
#endif
        if (lane == 0) status_store(p.tile_status + tile, excl + agg, kStateInclusive);
      }
      // the last tile of a block publishes the prefix through the block
      if (closes_block && lane == 0)
        status_store(p.block_status + blk_base + blk, excl + agg, kStateInclusive);
      if (lane == 0) {
        tile_excl[s] = excl;
        mbar_arrive(resolved0 + 8 * s);  // release: tile_excl is visible to the waiters
#ifdef TCU_LB_PROFILE
        const unsigned long long dt = gtime() - lb_t0;
        atomicAdd(&g_lb_stats[0], dt);
        atomicAdd(&g_lb_stats[1], 1ull);
        atomicMax(&g_lb_stats[2], dt);
#endif
      }
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
  auto slice_view = [&](uint32_t s, unsigned long long tile) {
    SliceView v;
    v.slice     = ring + s * kTileBytes + cw * kSliceBytes;
    v.slice_off = tile * kTileBytes + (unsigned long long)cw * kSliceBytes;
    const long long left = (long long)total_bytes - (long long)v.slice_off;
    v.valid_bytes = left <= 0 ? 0 : (left < kSliceBytes ? (int)left : kSliceBytes);
    return v;
  };

  // pass 1 of local tile i: slice total and row carries.  false = no such tile.
  auto pass1 = [&](uint32_t i) -> bool {
    const uint32_t s = i % NS, ph = (i / NS) & 1u;
    {
      LB_T0();
      if (!mbar_wait_or_stop(full0 + 8 * s, ph, abort_flag, nullptr, 0)) return false;
      LB_ADD(4, threadIdx.x == 0);
    }
    LB_T0();
    const unsigned long long tile = stage_tile[s];
    if (tile == kTileEnd) {
      if (lane == 0) *end_index = i;  // lets the look-back warps leave
      return false;
    }
    const SliceView v = slice_view(s, tile);
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
      carries[(s * kConsumerWarps + cw) * 32 + lane] = make_float4(ch_lo, cl_lo, ch_hi, cl_hi);
    if (lane == 0) part[s][cw] = make_float2(active ? slice_h : 0.f, active ? slice_l : 0.f);
    __syncwarp();
    if (lane == 0) mbar_arrive(p1done0 + 8 * s);
    LB_ADD(5, threadIdx.x == 0);
    return true;
  };

  // pass 2 of local tile k: the scan proper, seeded with everything before the slice
  auto pass2 = [&](uint32_t k) -> bool {
    const uint32_t s = k % NS, ph = (k / NS) & 1u;
    // the tile landed long ago (pass 1 has read it); this wait returns at once and makes the
    // copy's bytes visible to this warp as well
    {
      LB_T0();
      if (!mbar_wait_or_stop(full0 + 8 * s, ph, abort_flag, end_index, k)) return false;
      if (!mbar_wait_or_stop(resolved0 + 8 * s, ph, abort_flag, end_index, k)) return false;
      LB_ADD(3, threadIdx.x == kPass2Warp0 * 32);
    }
    LB_T0();
    const unsigned long long tile = stage_tile[s];
    const SliceView v = slice_view(s, tile);
    double carry = tile_excl[s];
    for (int w = 0; w < cw; ++w) carry += (double)part[s][w].x + (double)part[s][w].y;
    // Everything before this slice, as two floats that ride through the MMAs'
    // accumulator operand with the row carries: xh a multiple of 2^-13 (what the
    // hi parts are made of, so sums below 2^11 stay exact), xl the small rest.
    const double carry_hi = rint(carry * 8192.0) * (1.0 / 8192.0);
    const float xh = (float)carry_hi;
    const float xl = (float)(carry - (double)xh);
    if (v.valid_bytes > 0) {
      float ch_lo, cl_lo, ch_hi, cl_hi;
      const SliceAddr<Geom, kSwz> addr(v.slice, g, t);
      if constexpr (kSaveCarries) {
        const float4 c = carries[(s * kConsumerWarps + cw) * 32 + lane];
        ch_lo = c.x, cl_lo = c.y, ch_hi = c.z, cl_hi = c.w;
      } else {  // no room to keep them: redo the row totals
        Acc tot_h = zero, tot_l = zero;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t ah[4], al[4];
          load_split(addr, j, ah, al);
          tot_h = mma_ones(ah, tot_h);
          tot_l = mma_ones(al, tot_l);
        }
        float slice_h, slice_l;
        row_carries<16>(tot_h, tot_l, g, ch_lo, cl_lo, ch_hi, cl_hi, slice_h, slice_l);
      }
      RowCarry rc{ch_lo + xh, cl_lo + xl, ch_hi + xh, cl_hi + xl};
      const unsigned long long elem_base = v.slice_off / 2;
      const int valid_elems = v.valid_bytes / 2;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t ah[4], al[4];
        load_split(addr, j, ah, al);
        scan_step_independent<SC, OUT32>(j, ah, al, ops, rc, p.out, elem_base, valid_elems, g, t);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);
    LB_ADD(6, threadIdx.x == kPass2Warp0 * 32);
    return true;
  };

  if (warp < kPass2Warp0) {
    for (uint32_t i = 0; pass1(i); ++i) {}
  } else {
    for (uint32_t k = 0; pass2(k); ++k) {}
  }
}

}  // namespace tcu
