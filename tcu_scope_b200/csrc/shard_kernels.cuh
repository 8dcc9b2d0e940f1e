// Full reduction and full inclusive scan of an array that is sharded
// contiguously over several GPUs, one shard per GPU.
//
// The reference is single-GPU (src/init/cuda.cpp:45 selects one device; its
// full scan is three kernels over one array, src/prefixsum/wmma_3kers.cu:63-70),
// so this layer has no counterpart there.  What crosses NVLink is one double per
// GPU -- the shard totals -- and it is stored by the producing kernel itself:
//
//   pass 1, shard_reduce_kernel: every CTA sums a contiguous run of tiles and
//     leaves one total per CTA; the last CTA to finish adds them up and stores
//     {shard total, sequence number} into a slot in EVERY rank's memory (plain
//     st.global over the peer mapping; the slot arrays are a few hundred bytes).
//     For the full reduction the same CTA then waits (bounded) until all ranks'
//     totals have arrived in its own memory and writes their sum.
//   pass 2, shard_scan_kernel: every CTA waits (bounded) for the totals of the
//     EARLIER ranks in its own GPU's memory, adds the totals of the earlier CTAs
//     of pass 1, and scans its run of tiles with the carry kept in a register.
//     No look-back, no status words: the order inside a CTA is the only order.
//
// A shard is therefore read twice (2 + 6 bytes per element for fp32 outputs).
// To get part of the second read out of L2 instead of HBM, pass 1 walks each
// run BACKWARDS (a sum does not care) and loads the tiles it reads last -- the
// head of the run, which pass 2 reads first -- with the evict-last priority;
// pass 2 loads with evict-first and stores with st.global.cs.
//
// Only local memory is ever the source of a TMA copy; remote memory is written
// with ordinary stores and never read.
#pragma once

#include "reduce_kernels.cuh"
#include "scan_kernels.cuh"

namespace TCU_NS {

constexpr int kMaxRanks   = 16;  // ranks of one exchange group
constexpr int kSlotEpochs = 4;   // slots rotate with the call's sequence number

// One rank's total as it lies in every rank's slot array: [kSlotEpochs][kMaxRanks].
struct PeerSlot {
  double total;
  unsigned long long seq;  // the call this total belongs to; written after the total (release)
};

// The sequence number of a call is kept in device memory and advanced by pass 1
// itself (every rank makes the same calls, so the counters agree): a call's
// launches carry no per-call value and can be replayed from a CUDA graph.
struct ExchangeParams {
  PeerSlot* slots[kMaxRanks];       // slot array of every rank; [rank] is this GPU's own
  int rank, world;
  unsigned long long* seq_counter;  // calls made so far on this rank
};

struct ShardParams {
  const uint8_t* in;               // this GPU's shard, fp16, 16-byte aligned
  void* out;                       // pass 2: one float or half per element
  unsigned long long num_elems;    // elements of the shard (a multiple of 16)
  int out_is_f32;
  int keep_tiles;                  // pass 1: tiles per CTA loaded with the evict-last priority
  double* cta_total;               // [gridDim.x]: pass 1 writes, pass 2 reads
  unsigned int* done_counter;      // wraps back to zero by itself (atomicInc)
  float* total_f32;                // pass 1, optional: the total (of all ranks if wait_all)
  double* total_f64;               // likewise, in double
  int wait_all;                    // pass 1: 1 = full reduction, the result is the sum over ranks
  ExchangeParams x;
};

__device__ __forceinline__ void publish_total(const ExchangeParams& x, unsigned long long seq,
                                              int peer, double total) {
  PeerSlot* dst = x.slots[peer] + (seq % kSlotEpochs) * kMaxRanks + x.rank;
  asm volatile("st.relaxed.sys.global.f64 [%0], %1;" ::"l"(&dst->total), "d"(total) : "memory");
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(&dst->seq), "l"(seq) : "memory");
}

// Run by all 32 lanes of a warp: lane k < count waits until rank k's total of
// this call has arrived in this GPU's slot array.  Returns the sum of the
// totals of ranks [0, count) added in rank order (the same value in every lane
// and in every warp that asks).  The wait is bounded: when it runs out the
// error word is raised and the missing totals count as zero.
__device__ __forceinline__ double wait_totals(const ExchangeParams& x, unsigned long long seq,
                                              int count, int lane) {
  const PeerSlot* mine = x.slots[x.rank] + (seq % kSlotEpochs) * kMaxRanks;
  bool ready     = lane >= count;
  uint32_t polls = 0, limit = 1;
  while (!__all_sync(0xffffffffu, ready)) {
    if (!ready) {
      unsigned long long s;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(s) : "l"(&mine[lane].seq) : "memory");
      ready = s == seq;
    }
    if (polls == 0) limit = wait_limit(&g_wait_limits.peer);
    if (++polls > limit) {
      if (lane == 0) raise_error(kErrPeerTimeout);
      break;
    }
    __nanosleep(polls < 64 ? 32 : 400);
  }
  double v = 0.0;
  if (lane < count && ready)
    asm volatile("ld.relaxed.sys.global.f64 %0, [%1];" : "=d"(v) : "l"(&mine[lane].total) : "memory");
  double sum = 0.0;
  for (int k = 0; k < count; ++k) sum += __shfl_sync(0xffffffffu, v, k);
  return sum;
}

// The tiles of CTA b: [run_begin(b), run_begin(b + 1)).  Both passes use it.
__device__ __forceinline__ unsigned long long run_begin(unsigned long long num_tiles,
                                                        unsigned long long cta) {
  return num_tiles * cta / gridDim.x;
}

// Sum of cta_total[0 .. count) in a fixed order, by one warp; same value in every lane.
__device__ __forceinline__ double sum_cta_totals(const double* cta_total, unsigned count, int lane) {
  double v = 0.0;
  for (unsigned k = lane; k < count; k += 32) v += __ldcg(cta_total + k);
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// ---------------------------------------------------------------------------
// Pass 1.  Same ring, slices and contraction as seg_reduce_kernel's long class;
// the differences are the contiguous, backwards run per CTA with its L2
// priorities, one total per CTA kept for pass 2, and the exchange at the end.
__global__ void __launch_bounds__(kThreads, 1) shard_reduce_kernel(const ShardParams p) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * kStages];
  __shared__ double warp_sum[kConsumerWarps];
  __shared__ int s_is_last;

  uint8_t* ring = dyn_smem + ((128u - (smem_u32(dyn_smem) & 127u)) & 127u);
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

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
  const unsigned long long tile_begin  = run_begin(num_tiles, blockIdx.x);
  const unsigned long long tile_end    = run_begin(num_tiles, blockIdx.x + 1ull);
  const unsigned long long run_tiles   = tile_end - tile_begin;

  if (warp == kConsumerWarps) {
    if (lane == 0) {
      const uint64_t keep = l2_policy_evict_last(), drop = l2_policy_evict_first();
      for (unsigned long long i = 0; i < run_tiles; ++i) {  // tile_end - 1 down to tile_begin
        const uint32_t s = (uint32_t)(i % kStages), ph = (uint32_t)(i / kStages) & 1u;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u)) break;
        const unsigned long long tile = tile_end - 1 - i;
        const unsigned long long off  = tile * kTileBytes;
        const unsigned long long rem  = total_bytes - off;
        const uint32_t bytes = rem < (unsigned long long)kTileBytes ? (uint32_t)rem : kTileBytes;
        mbar_arrive_expect_tx(full0 + 8 * s, bytes);
        // the head of the run is what pass 2 reads first: ask L2 to hold on to it
        const bool head = tile - tile_begin < (unsigned long long)p.keep_tiles;
        tma_load_1d_hint(ring_u32 + s * kTileBytes, p.in + off, bytes, full0 + 8 * s,
                         head ? keep : drop);
      }
    }
  } else {
    bool dead      = false;
    double run_val = 0.0;  // this warp's slices of the run
    for (unsigned long long i = 0; i < run_tiles; ++i) {
      const uint32_t s = (uint32_t)(i % kStages), ph = (uint32_t)(i / kStages) & 1u;
      if (!dead && !mbar_wait(full0 + 8 * s, ph)) dead = true;
      const unsigned long long tile = tile_end - 1 - i;
      uint8_t* slice = ring + s * kTileBytes + warp * kSliceBytes;
      const unsigned long long slice_off = tile * kTileBytes + (unsigned long long)warp * kSliceBytes;
      const long long left  = (long long)total_bytes - (long long)slice_off;
      const int valid_bytes = left <= 0 ? 0 : (left < kSliceBytes ? (int)left : kSliceBytes);
      if (!dead && valid_bytes > 0) {
        if (valid_bytes < kSliceBytes) zero_slice_tail(slice, valid_bytes, lane);
        const float2 tot = reduce_slice<kClassLong>(slice, nullptr, true, 0, 0, lane);
        run_val += (double)tot.x + (double)tot.y;  // exact parts, added in a fixed order
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
    if (lane == 0) warp_sum[warp] = run_val;
  }

  __syncthreads();
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int w = 0; w < kConsumerWarps; ++w) total += warp_sum[w];
    p.cta_total[blockIdx.x] = total;
    __threadfence();
    s_is_last = (atomicInc(p.done_counter, gridDim.x - 1) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_is_last || warp != 0) return;

  // ---- the last CTA: shard total, exchange, optional sum over ranks
  __threadfence();
  double total = sum_cta_totals(p.cta_total, gridDim.x, lane);
  unsigned long long seq = 0;
  if (lane == 0) {
    seq = *p.x.seq_counter + 1;  // this call's number; pass 2 reads it back
    *p.x.seq_counter = seq;
  }
  seq = __shfl_sync(0xffffffffu, seq, 0);
  if (lane < p.x.world) publish_total(p.x, seq, lane, total);
  if (p.wait_all) total = wait_totals(p.x, seq, p.x.world, lane);
  if (lane == 0) {
    if (p.total_f32) *p.total_f32 = (float)total;
    if (p.total_f64) *p.total_f64 = total;
  }
}

// ---------------------------------------------------------------------------
// Pass 2.  The slice scan is seg_scan_kernel's for segments of a whole tile
// (the slice is read and split once into registers, row carries from the row
// totals, slice totals meet in shared memory once per tile); the carry from
// everything earlier rides through the accumulators while it is small and is
// added last once it is not (scan_step_independent).  The carry across tiles
// is a compensated pair of floats every warp keeps for itself.  The consumer warps meet at one
// barrier per tile: with fp32 outputs, two thirds of the traffic are writes,
// and they reach HBM in better order when a CTA's warps store the same tile
// together (point-to-point hand-offs measured 3 % slower, 16 warps on half
// slices 5 % slower, swizzled tensor-map loads 8 % slower than linear ones).
template <bool OUT32>
__global__ void __launch_bounds__(kThreads, 1) shard_scan_kernel(const ShardParams p) {
  constexpr int SC = 15;  // row-stream geometry, rows always chained
  using Geom = ScanGeom<SC>;
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * kStages];
  __shared__ float2 part[2][kConsumerWarps];  // slice totals (exact hi, lo) of the tile in flight

  uint8_t* ring = dyn_smem + ((128u - (smem_u32(dyn_smem) & 127u)) & 127u);
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_prologue();  // nothing above touched global memory; pass 1 of this GPU is complete

  const unsigned long long total_bytes = p.num_elems * 2ull;
  const unsigned long long num_tiles   = (total_bytes + kTileBytes - 1) / kTileBytes;
  const unsigned long long tile_begin  = run_begin(num_tiles, blockIdx.x);
  const unsigned long long tile_end    = run_begin(num_tiles, blockIdx.x + 1ull);

  if (warp == kConsumerWarps) {
    if (lane == 0) {
      const uint64_t drop = l2_policy_evict_first();  // last use of these lines
      uint32_t i = 0;
      for (unsigned long long tile = tile_begin; tile < tile_end; ++tile, ++i) {
        const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u)) break;
        const unsigned long long off = tile * kTileBytes;
        const unsigned long long rem = total_bytes - off;
        const uint32_t bytes = rem < (unsigned long long)kTileBytes ? (uint32_t)rem : kTileBytes;
        mbar_arrive_expect_tx(full0 + 8 * s, bytes);
        tma_load_1d_hint(ring_u32 + s * kTileBytes, p.in + off, bytes, full0 + 8 * s, drop);
      }
    }
    return;
  }

  // ------------------------------------------------------------- consumers
  const int g = lane >> 2, t = lane & 3;
  const ScanOperands ops = make_scan_operands(lane, false);
  const Acc zero{0.f, 0.f, 0.f, 0.f};
  bool dead = false;

  // everything before this CTA's run: the earlier ranks' shards, the earlier CTAs' runs
  double run = 0.0;
  if (tile_begin < tile_end) {
    if (p.x.rank > 0) run = wait_totals(p.x, __ldcg(p.x.seq_counter), p.x.rank, lane);
    run += sum_cta_totals(p.cta_total, blockIdx.x, lane);
  }
  // ... kept from here on as two floats (double arithmetic measured slow on this part): rh a
  // multiple of 2^-13 like the hi parts, rl the rest
  float rh = (float)(rint(run * 8192.0) * (1.0 / 8192.0));
  float rl = (float)(run - (double)rh);

  uint32_t i = 0;
  for (unsigned long long tile = tile_begin; tile < tile_end; ++tile, ++i) {
    const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
    if (!dead && !mbar_wait(full0 + 8 * s, ph)) dead = true;

    uint8_t* slice = ring + s * kTileBytes + warp * kSliceBytes;
    const unsigned long long slice_off = tile * kTileBytes + (unsigned long long)warp * kSliceBytes;
    const long long left  = (long long)total_bytes - (long long)slice_off;
    const int valid_bytes = left <= 0 ? 0 : (left < kSliceBytes ? (int)left : kSliceBytes);
    const bool active     = !dead && valid_bytes > 0;
    if (active && valid_bytes < kSliceBytes) zero_slice_tail(slice, valid_bytes, lane);

    // the whole slice into registers, split into exact parts; row totals on the way
    const SliceAddr<Geom, false> addr(slice, g, t);
    uint32_t ah[8][4], al[8][4];
    Acc tot_h = zero, tot_l = zero;
    if (active) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        load_split(addr, j, ah[j], al[j]);
        tot_h = mma_ones(ah[j], tot_h);
        tot_l = mma_ones(al[j], tot_l);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);  // everything needed is in registers

    float ch_lo, cl_lo, ch_hi, cl_hi, slice_h, slice_l;
    row_carries<16>(tot_h, tot_l, g, ch_lo, cl_lo, ch_hi, cl_hi, slice_h, slice_l);
    if (lane == 0) part[i & 1][warp] = make_float2(active ? slice_h : 0.f, active ? slice_l : 0.f);
    consumer_sync();  // one meeting per tile; part[] is double-buffered across it
    // One chain of exact additions over the tile's slices: this warp's carry on the way, the
    // run's new total at the end.  (ch, cl) is a compensated pair: ch the sum of the hi parts,
    // cl the lo parts plus whatever an addition to ch rounded off (nothing below 2^11).
    float ch = rh, cl = rl, wh = rh, wl = rl;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
      if (w == warp) {
        wh = ch;
        wl = cl;
      }
      const float2 pr = part[i & 1][w];
      pair_add(ch, cl, pr.x, pr.y);
    }
    rh = ch;
    rl = cl;
    pair_renorm(rh, rl);  // multiples of 2^-13 that the lo parts have added up to move over
    if (!active) continue;

    // everything before this slice as two floats: xh a multiple of 2^-13, xl the
    // rest.  Below 2^10, xh rides through the accumulators with the row carries
    // (every sum stays exact); above, it is added to each output last.
    float xh = wh, xl = wl;
    pair_renorm(xh, xl);
    const bool fold = fabsf(xh) < 1024.f;
    const float xf = fold ? xh : 0.f, big = fold ? 0.f : xh;
    RowCarry rc{ch_lo + xf, cl_lo + xl, ch_hi + xf, cl_hi + xl};
    const unsigned long long elem_base = slice_off / 2;
    const int valid_elems = valid_bytes / 2;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      scan_step_independent<SC, OUT32, true>(j, ah[j], al[j], ops, rc, p.out, elem_base,
                                             valid_elems, g, t, big);
  }
}

}  // namespace TCU_NS
