// Segmented and full inclusive prefix sum of fp16 arrays on the tensor cores.
//
// What it replaces in c3sr/tcu_scope: compute_wmma_segmented_prefixsum_16n
// (src/prefixsum/kernel.cuh:86-150), ..._256n (:441-506), ..._256n_block
// (:586-678) and the three-kernel full scan built on ..._256n_ps + a library
// exclusive scan + add_partial_sums (src/prefixsum/wmma_3kers.cu:63-70).  The
// contraction is the paper's: a 16 x 16 block of input rows times the
// upper-triangular ones matrix U gives 16 independent 16-wide inclusive scans
// (kernel.cuh:60,79-81).  Differences: one persistent single-pass kernel per
// segment class, fp32 accumulation of exact hi/lo parts, the running carry fed
// through the accumulator operand of the next MMA instead of a shared-memory
// round trip, and a decoupled look-back chain across tiles in place of the
// second and third kernel.
//
// Layout inside one warp's 4 KiB slice (2048 halves): 16 "rows" of 128
// consecutive halves.  MMA row r walks row r of the slice 16 halves per step,
// so the carry of a row flows from step to step inside that row (the C operand
// of the next MMA), and only once per slice do the 16 row totals have to be
// scanned across lanes with shuffles.  For 16-element segments there is no
// carry at all and the rows are simply consecutive 16-element segments.
#pragma once

#include "common.cuh"

namespace TCU_NS {

struct ScanParams {
  const uint8_t* in;             // fp16 input, 16-byte aligned
  void* out;                     // half or float per element, 16-byte aligned
  unsigned long long num_elems;
  int out_is_f32;
  // look-back class only
  unsigned long long tiles_per_segment;  // segment_size / kTileElems
  unsigned long long* tile_status;       // [num_tiles], zeroed by the host before the launch
  unsigned long long* block_status;      // [~num_tiles/32 + segments], zeroed likewise
  unsigned int* ticket;                  // dynamic tile counter, zeroed by the host
  const double* shard_totals;            // optional: totals of all shards of a multi-GPU scan
  int shard_index;                       // this GPU's position in shard_totals
  int exclusive;                         // 1: out[i] excludes in[i] (strictly triangular operand)
};

// B operands for "A times U" with the k order that the 8-byte row loads give:
// lane (g,t) holds row elements 4t..4t+3 as k = 2t, 2t+1, 2t+8, 2t+9.  Column
// n of the first MMA is output position 4(n>>1) + (n&1), of the second one
// that plus 2, so each lane ends up with the 4 consecutive outputs 4t..4t+3 of
// its rows -- the same positions it loaded.
struct ScanOperands {
  uint32_t ua0, ua1, ub0, ub1;
};

// exclusive: position p contributes to output q only if p < q, i.e. U without
// its diagonal; row totals and carries do not change.
__device__ __forceinline__ ScanOperands make_scan_operands(int lane, bool exclusive) {
  const int g = lane >> 2, t = lane & 3;
  const int qa = 4 * (g >> 1) + (g & 1) - (exclusive ? 1 : 0), qb = qa + 2;
  auto pack = [](bool e0, bool e1) -> uint32_t {
    return (e0 ? kOne16 : 0u) | (e1 ? (kOne16 << 16) : 0u);
  };
  ScanOperands o;
  o.ua0 = pack(4 * t + 0 <= qa, 4 * t + 1 <= qa);
  o.ua1 = pack(4 * t + 2 <= qa, 4 * t + 3 <= qa);
  o.ub0 = pack(4 * t + 0 <= qb, 4 * t + 1 <= qb);
  o.ub1 = pack(4 * t + 2 <= qb, 4 * t + 3 <= qb);
  return o;
}

// kStream: the lines are not read again by this kernel -- mark them as the
// first to leave L2 (st.global.cs), so that they do not displace data that is.
template <bool OUT32, bool kStream = false>
__device__ __forceinline__ void store4(void* out, unsigned long long idx, float r0, float r1,
                                       float r2, float r3) {
  if constexpr (OUT32) {
    float* dst = static_cast<float*>(out) + idx;
    if constexpr (kStream)
      asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};"
                   ::"l"(dst), "f"(r0), "f"(r1), "f"(r2), "f"(r3) : "memory");
    else
      *reinterpret_cast<float4*>(dst) = make_float4(r0, r1, r2, r3);
  } else {
    const uint32_t ua = pack2_rn(r0, r1), ub = pack2_rn(r2, r3);
    uint16_t* dst = static_cast<uint16_t*>(out) + idx;
    if constexpr (kStream)
      asm volatile("st.global.cs.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(ua), "r"(ub) : "memory");
    else
      *reinterpret_cast<uint2*>(dst) = make_uint2(ua, ub);
  }
}

// Shape of one consumer warp's slice: a 32 KiB tile divided among W consumer
// warps, each slice 16 rows (the 16 rows of the MMA's A operand) walked 16
// elements per step.  W = 8: 4 KiB slices, rows of 128 elements, 8 steps.
// W = 16: 2 KiB slices, rows of 64 elements, 4 steps -- twice the warps per
// scheduler to hide the latencies of the split / MMA / add / convert chains,
// half the registers per warp for the slice it keeps, carry chains half as long.
template <int W>
struct SliceShape {
  static_assert(W == 8 || W == 16, "8 or 16 consumer warps per tile");
  static constexpr int kWarps        = W;
  static constexpr int kBytes        = kTileBytes / W;
  static constexpr int kRowBytes     = kBytes / 16;
  static constexpr int kRowElemsLog2 = W == 8 ? 7 : 6;
  static constexpr int kSteps        = kRowBytes / 32;
  static constexpr int kThreads      = (W + 1) * 32;  // + 1 producer warp
};

// Byte offset inside the slice of the 8 bytes lane (g,t) loads for MMA row g
// at step j (row g+8 is kHiOffset further).
template <int SC, int W = 8>
struct ScanGeom {
  using Shape = SliceShape<W>;
  static constexpr bool kLinear   = SC == 4;  // rows = consecutive 16-element segments
  static constexpr int kSteps     = Shape::kSteps;
  static constexpr int kHiOffset  = kLinear ? 256 : Shape::kBytes / 2;
  __device__ static __forceinline__ int lo(int g, int t, int j) {
    return kLinear ? 512 * j + 32 * g + 8 * t : Shape::kRowBytes * g + 32 * j + 8 * t;
  }
};

// Where lane (g,t) finds its 8 bytes of MMA row g at step j (row g+8 is
// kHiOffset further).  kSwz: the tile was written by a swizzled tensor-map copy
// (slices start on 4 KiB boundaries of a 1 KiB-aligned tile, so the swizzle
// only depends on the offset inside the slice).  The swizzled offset of
// 256g + 32j + 8t has the closed form
//   256g + 128(j>>2) + 8(t&1) + 16((t>>1) ^ (j>>2)) + 32((j&3) ^ (g&3)),
// i.e. one of two lane-constant bases plus one of four lane-constant terms:
// one add per load instead of a shift-mask-xor sequence.
template <class Geom, bool kSwz>
struct SliceAddr {
  const uint8_t* base[2];
  int term[4];
  __device__ __forceinline__ SliceAddr(const uint8_t* slice, int g, int t) {
    static_assert(!kSwz || Geom::Shape::kRowBytes == 256, "the closed form is for 256-byte rows");
    if constexpr (kSwz) {
      base[0] = slice + 256 * g + 8 * (t & 1) + 16 * (t >> 1);
      base[1] = slice + 256 * g + 128 + 8 * (t & 1) + 16 * ((t >> 1) ^ 1);
#pragma unroll
      for (int c = 0; c < 4; ++c) term[c] = 32 * (c ^ (g & 3));
    } else {
      base[0] = base[1] = slice + Geom::lo(g, t, 0);
      term[0] = term[1] = term[2] = term[3] = 0;
    }
  }
  __device__ __forceinline__ const uint8_t* lo(int j) const {
    if constexpr (kSwz)
      return base[j >> 2] + term[j & 3];
    else
      return base[0] + (Geom::lo(0, 0, j) - Geom::lo(0, 0, 0));  // compile-time offset
  }
};

// Load the 2 x 8 bytes lane (g,t) owns at step j and split them into exact
// hi / lo A operands: [0] row g k 2t,2t+1  [1] row g+8 k 2t,2t+1
//                     [2] row g k 2t+8,+9  [3] row g+8 k 2t+8,+9.
template <class Geom, bool kSwz>
__device__ __forceinline__ void load_split(const SliceAddr<Geom, kSwz>& addr, int j,
                                           uint32_t (&ah)[4], uint32_t (&al)[4]) {
  const uint8_t* p = addr.lo(j);
  const uint2 lo = lds64(p);
  const uint2 hi = lds64(p + Geom::kHiOffset);
  split_hi_lo(lo.x, ah[0], al[0]);
  split_hi_lo(hi.x, ah[1], al[1]);
  split_hi_lo(lo.y, ah[2], al[2]);
  split_hi_lo(hi.y, ah[3], al[3]);
}

__device__ __forceinline__ Acc mma_ones(const uint32_t (&a)[4], Acc c) {
  return mma16816(a[0], a[1], a[2], a[3], kOnesH2, kOnesH2, c);
}

// Carry into each MMA row = sum of the totals of the earlier rows of the same
// segment.  tot.d0 / tot.d2 hold the totals of rows g / g+8 (in every lane of
// the group); slice rows are ordered 0..7 = "lo" rows of g = 0..7, 8..15 =
// "hi" rows.  kRowsPerSeg in {2,4,8,16}.  Also returns the slice total (only
// meaningful when all 16 rows form one segment).
template <int kRowsPerSeg>
__device__ __forceinline__ void row_carries(const Acc& tot_h, const Acc& tot_l, int g,
                                            float& ch_lo, float& cl_lo, float& ch_hi,
                                            float& cl_hi, float& slice_h, float& slice_l) {
  constexpr int kRG = kRowsPerSeg >= 8 ? 8 : kRowsPerSeg;
  float ih_lo = tot_h.d0, il_lo = tot_l.d0, ih_hi = tot_h.d2, il_hi = tot_l.d2;
#pragma unroll
  for (int d = 1; d < kRG; d <<= 1) {
    const float a = __shfl_up_sync(0xffffffffu, ih_lo, 4 * d);
    const float b = __shfl_up_sync(0xffffffffu, il_lo, 4 * d);
    const float c = __shfl_up_sync(0xffffffffu, ih_hi, 4 * d);
    const float e = __shfl_up_sync(0xffffffffu, il_hi, 4 * d);
    if ((g & (kRG - 1)) >= d) {
      ih_lo += a;
      il_lo += b;
      ih_hi += c;
      il_hi += e;
    }
  }
  ch_lo = __shfl_up_sync(0xffffffffu, ih_lo, 4);
  cl_lo = __shfl_up_sync(0xffffffffu, il_lo, 4);
  ch_hi = __shfl_up_sync(0xffffffffu, ih_hi, 4);
  cl_hi = __shfl_up_sync(0xffffffffu, il_hi, 4);
  if ((g & (kRG - 1)) == 0) ch_lo = cl_lo = ch_hi = cl_hi = 0.f;
  slice_h = slice_l = 0.f;
  if constexpr (kRowsPerSeg == 16) {
    const float th = __shfl_sync(0xffffffffu, ih_lo, 28);  // total of rows 0..7
    const float tl = __shfl_sync(0xffffffffu, il_lo, 28);
    ch_hi += th;
    cl_hi += tl;
    slice_h = __shfl_sync(0xffffffffu, ih_hi, 28) + th;
    slice_l = __shfl_sync(0xffffffffu, il_hi, 28) + tl;
  }
}

// One step of one slice: 16 rows x 16 elements.  D = A.U + carry for the hi
// and the lo parts (4 MMAs), the carry for the next step (2 more, only when a
// segment continues), then out = hi + lo.  The carry from earlier slices of the
// segment is not added here per output: the caller adds it once to the row
// carries, and it rides through the accumulator operand with them.
template <int SC, bool OUT32, int W = 8>
__device__ __forceinline__ void scan_step(int j, const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                          const ScanOperands& ops, float& ch_lo, float& cl_lo,
                                          float& ch_hi, float& cl_hi, void* out,
                                          unsigned long long elem_base, int valid_elems, int g,
                                          int t, uint8_t* staged = nullptr) {
  using Geom = ScanGeom<SC, W>;
  // segments no longer than a row: kStepsPerSeg steps each, the carry starts over with each
  constexpr bool kInRow      = SC <= Geom::Shape::kRowElemsLog2;
  constexpr int kStepsPerSeg = kInRow ? (1 << SC) / 16 : Geom::kSteps;
  if (kInRow && (j % kStepsPerSeg) == 0) ch_lo = cl_lo = ch_hi = cl_hi = 0.f;
  const Acc c_h{ch_lo, ch_lo, ch_hi, ch_hi}, c_l{cl_lo, cl_lo, cl_hi, cl_hi};
  const Acc ha = mma16816(ah[0], ah[1], ah[2], ah[3], ops.ua0, ops.ua1, c_h);
  const Acc hb = mma16816(ah[0], ah[1], ah[2], ah[3], ops.ub0, ops.ub1, c_h);
  const Acc la = mma16816(al[0], al[1], al[2], al[3], ops.ua0, ops.ua1, c_l);
  const Acc lb = mma16816(al[0], al[1], al[2], al[3], ops.ub0, ops.ub1, c_l);
  const bool carry_on = ((j + 1) % kStepsPerSeg) != 0;
  if (carry_on) {
    const Acc nh = mma_ones(ah, c_h), nl = mma_ones(al, c_l);
    ch_lo = nh.d0;
    ch_hi = nh.d2;
    cl_lo = nl.d0;
    cl_hi = nl.d2;
  }
  const int e_lo = Geom::lo(g, t, j) / 2, e_hi = e_lo + Geom::kHiOffset / 2;
  if constexpr (!OUT32) {
    if (staged != nullptr) {  // results replace the inputs in the ring stage; a bulk copy stores them
      store4<false>(staged, e_lo, ha.d0 + la.d0, ha.d1 + la.d1, hb.d0 + lb.d0, hb.d1 + lb.d1);
      store4<false>(staged, e_hi, ha.d2 + la.d2, ha.d3 + la.d3, hb.d2 + lb.d2, hb.d3 + lb.d3);
      return;
    }
  }
  if (e_lo < valid_elems)
    store4<OUT32>(out, elem_base + e_lo, ha.d0 + la.d0, ha.d1 + la.d1, hb.d0 + lb.d0,
                  hb.d1 + lb.d1);
  if (e_hi < valid_elems)
    store4<OUT32>(out, elem_base + e_hi, ha.d2 + la.d2, ha.d3 + la.d3, hb.d2 + lb.d2,
                  hb.d3 + lb.d3);
}

// Variant of scan_step for rows that are chained over all eight steps, with
// the running carry kept by fp32 adds instead of a dependent MMA: the totals of
// this step come from MMAs with a zero accumulator, independent of every other
// step, so consecutive steps overlap even with few warps per scheduler.
// `big`: the part of the prefix before this slice that is too large to ride
// through the accumulators without costing them their low bits (0 when there
// is none); it is added once, last, so each output is rounded once at its own
// magnitude.
struct RowCarry {
  float h_lo, l_lo, h_hi, l_hi;  // (exact hi part, lo part) x (row g, row g+8)
};

template <int SC, bool OUT32, bool kStream = false, int W = 8>
__device__ __forceinline__ void scan_step_independent(int j, const uint32_t (&ah)[4],
                                                      const uint32_t (&al)[4],
                                                      const ScanOperands& ops, RowCarry& c,
                                                      void* out, unsigned long long elem_base,
                                                      int valid_elems, int g, int t, float big) {
  using Geom = ScanGeom<SC, W>;
  const Acc zero{0.f, 0.f, 0.f, 0.f};
  const Acc c_h{c.h_lo, c.h_lo, c.h_hi, c.h_hi}, c_l{c.l_lo, c.l_lo, c.l_hi, c.l_hi};
  const Acc ha = mma16816(ah[0], ah[1], ah[2], ah[3], ops.ua0, ops.ua1, c_h);
  const Acc hb = mma16816(ah[0], ah[1], ah[2], ah[3], ops.ub0, ops.ub1, c_h);
  const Acc la = mma16816(al[0], al[1], al[2], al[3], ops.ua0, ops.ua1, c_l);
  const Acc lb = mma16816(al[0], al[1], al[2], al[3], ops.ub0, ops.ub1, c_l);
  if (j != Geom::kSteps - 1) {
    const Acc th = mma_ones(ah, zero), tl = mma_ones(al, zero);
    c.h_lo += th.d0;
    c.h_hi += th.d2;
    c.l_lo += tl.d0;
    c.l_hi += tl.d2;
  }
  const int e_lo = Geom::lo(g, t, j) / 2, e_hi = e_lo + Geom::kHiOffset / 2;
  if (e_lo < valid_elems)
    store4<OUT32, kStream>(out, elem_base + e_lo, (ha.d0 + la.d0) + big, (ha.d1 + la.d1) + big,
                           (hb.d0 + lb.d0) + big, (hb.d1 + lb.d1) + big);
  if (e_hi < valid_elems)
    store4<OUT32, kStream>(out, elem_base + e_hi, (ha.d2 + la.d2) + big, (ha.d3 + la.d3) + big,
                           (hb.d2 + lb.d2) + big, (hb.d3 + lb.d3) + big);
}

// Segment classes as for the reduction: class = log2(segment size), 4..14.
// Launch shape per class.  16-element segments have no carry and need few
// registers: two CTAs per SM with 8 consumer warps each (3-stage rings).  From
// 32 elements on the slice is read and split once into registers (which frees
// the ring stage early and takes the loads off the carry chain), one CTA per
// SM; these classes are bound by the latency of their dependent instruction
// chains, not by issue slots or the tensor pipe, so they run 16 consumer warps
// on half-size slices (see SliceShape) where that measured faster: 16-bit
// outputs of 64- and 256...1024-element segments (+3-5 %).
__host__ __device__ constexpr int scan_warps(int sc, bool out32) {
  return !out32 && (sc == 6 || (sc >= 8 && sc <= 10)) ? 16 : 8;
}
constexpr int kScanBulkMaxClass = 6;  // largest class whose fp16 outputs leave through shared memory
// Two CTAs per SM (3-stage rings) only for 16-bit outputs of 16-element segments; everything else
// reads and splits the slice once into registers, one CTA per SM.  Ring depth, measured at 2^28
// elements: the classes whose fp16 outputs leave through the ring stage hold a stage one tile
// longer (5 stages); fp32 outputs of 16 ... 64-element segments run faster on a SHALLOW ring of 2
// stages, and the 16-element ones on one CTA per SM at that (0.91 / 0.96 / 0.96 of the copy
// bandwidth against 0.87 / 0.93 / 0.89 with 2 x 3 and 5 stages: reads that run far ahead get in
// the way of twice as many bytes of writes); the others measured best with 4 (2 stages: fp32
// outputs of 4096 and 8192 elements -2 %, fp16 outputs from 256 elements on between -3 and +5 %
// from box to box).
__host__ __device__ constexpr int scan_ctas_per_sm(int sc, bool out32) { return sc == 4 && !out32 ? 2 : 1; }
__host__ __device__ constexpr int scan_stages(int sc, bool out32) {
  if (scan_ctas_per_sm(sc, out32) == 2) return 3;
  if (out32) return sc <= 6 ? 2 : kStages;
  return sc <= kScanBulkMaxClass ? 5 : kStages;
}
__host__ __device__ constexpr int scan_dyn_smem_bytes(int sc, bool out32) {
  return scan_stages(sc, out32) * kTileBytes + 128;
}

template <int kWarps>
__device__ __forceinline__ void consumer_sync_n() {
  asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
}

template <int SC, bool OUT32, int W = scan_warps(SC, OUT32)>
__global__ void __launch_bounds__(SliceShape<W>::kThreads, scan_ctas_per_sm(SC, OUT32))
    seg_scan_kernel(const ScanParams p) {
  static_assert(SC >= 4 && SC <= 14, "the look-back class has its own kernel");
  using Shape = SliceShape<W>;
  using Geom  = ScanGeom<SC, W>;
  constexpr int kStages = scan_stages(SC, OUT32);  // shadows the library-wide ring depth
  constexpr int kSteps  = Shape::kSteps;
  constexpr int LR      = Shape::kRowElemsLog2;
  constexpr bool kScanCache = scan_ctas_per_sm(SC, OUT32) == 1;  // slice kept in registers between passes
  // segments longer than a row: rows per segment inside the slice, warps per segment beyond
  constexpr bool kRows      = SC > LR;
  constexpr int kRowsPerSeg = SC >= LR + 4 ? 16 : (kRows ? 1 << (SC - LR) : 1);
  constexpr bool kCross     = SC > LR + 4;
  constexpr int kWarpsPerSeg = kCross ? 1 << (SC - LR - 4) : 1;
  // fp16 outputs of a slice overwrite its inputs in the ring stage and leave
  // through one bulk copy per warp; the stage is released one tile later, once
  // that copy has read it.
  constexpr bool kBulkStore = !OUT32 && kScanCache && SC <= kScanBulkMaxClass;
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * kStages];
  // Slice totals cross warps either under a barrier of all consumer warps, or
  // point to point: a warp publishes its total with a sequence number and only
  // the later warps of the same segment wait for it, so the warps do not fall
  // into lock step.  A warp cannot be more than kStages tiles ahead of the
  // slowest one (stages are released by all of them), so 2 * kStages slots are
  // never overwritten while still being read.
  constexpr bool kP2P = kCross && (!OUT32 || W == 16);
  constexpr int kPartSlots = kP2P ? 2 * kStages : 2;
  __shared__ float2 part[kPartSlots][W];
  __shared__ uint32_t part_seq[kPartSlots][W];

  uint8_t* ring = dyn_smem + ((128u - (smem_u32(dyn_smem) & 127u)) & 127u);
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, W);
    }
    mbar_fence_init();
  }
  if (threadIdx.x < kPartSlots * W) (&part_seq[0][0])[threadIdx.x] = 0u;
  __syncthreads();
  pdl_prologue();  // nothing above touched global memory

  const unsigned long long total_bytes = p.num_elems * 2ull;
  const unsigned long long num_tiles   = (total_bytes + kTileBytes - 1) / kTileBytes;

  if (warp == W) {
    if (lane == 0) {
      uint32_t i = 0;
      for (unsigned long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++i) {
        const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u)) break;
        const unsigned long long off = tile * kTileBytes;
        const unsigned long long rem = total_bytes - off;
        const uint32_t bytes = rem < (unsigned long long)kTileBytes ? (uint32_t)rem : kTileBytes;
        mbar_arrive_expect_tx(full0 + 8 * s, bytes);
        tma_load_1d(ring_u32 + s * kTileBytes, p.in + off, bytes, full0 + 8 * s);
      }
    }
    return;
  }

  // ------------------------------------------------------------- consumers
  const int g = lane >> 2, t = lane & 3;
  const ScanOperands ops = make_scan_operands(lane, p.exclusive != 0);
  const Acc zero{0.f, 0.f, 0.f, 0.f};
  bool dead = false;

  uint32_t i = 0;
  for (unsigned long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++i) {
    const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
    if (!dead && !mbar_wait(full0 + 8 * s, ph)) dead = true;

    uint8_t* slice = ring + s * kTileBytes + warp * Shape::kBytes;
    const unsigned long long slice_off = tile * kTileBytes + (unsigned long long)warp * Shape::kBytes;
    const long long left  = (long long)total_bytes - (long long)slice_off;
    const int valid_bytes = left <= 0 ? 0 : (left < Shape::kBytes ? (int)left : Shape::kBytes);
    const bool active     = !dead && valid_bytes > 0;
    if (active && valid_bytes < Shape::kBytes) zero_slice_tail<Shape::kBytes>(slice, valid_bytes, lane);

    // ---- load + split the whole slice; row totals for classes that chain rows
    // (two accumulator pairs, even and odd steps: half the dependent MMA chain)
    const SliceAddr<Geom, false> addr(slice, g, t);
    constexpr int kKeep = kScanCache ? kSteps : 1;
    uint32_t ah[kKeep][4], al[kKeep][4];
    Acc tot_h = zero, tot_l = zero, tot_h2 = zero, tot_l2 = zero;
    if (active && (kScanCache || kRows)) {
#pragma unroll
      for (int j = 0; j < kSteps; ++j) {
        load_split(addr, j, ah[kScanCache ? j : 0], al[kScanCache ? j : 0]);
        if constexpr (kRows) {
          if (j & 1) {
            tot_h2 = mma_ones(ah[kScanCache ? j : 0], tot_h2);
            tot_l2 = mma_ones(al[kScanCache ? j : 0], tot_l2);
          } else {
            tot_h = mma_ones(ah[kScanCache ? j : 0], tot_h);
            tot_l = mma_ones(al[kScanCache ? j : 0], tot_l);
          }
        }
      }
      if constexpr (kRows) {  // exact parts: the sums are exact whatever the order
        tot_h.d0 += tot_h2.d0;
        tot_h.d2 += tot_h2.d2;
        tot_l.d0 += tot_l2.d0;
        tot_l.d2 += tot_l2.d2;
      }
    }
    if constexpr (kScanCache && !kBulkStore) {
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);  // everything needed is in registers
    }
    // fp32 outputs: two of every three bytes of traffic are writes, and they reach HBM in
    // better order when the warps of a CTA work on the same tile at the same time (measured
    // 0.87-0.90 -> 0.96-1.03 of the copy bandwidth for 32...2048-element segments); with
    // 16-bit outputs the warps' own instruction streams are the limit and a meeting per tile
    // costs 10 %.  The classes that span warps meet anyway.
    if constexpr (OUT32 && kScanCache && !kCross) consumer_sync_n<W>();

    // ---- carries into each MMA row, and from the earlier slices of the segment
    float ch_lo = 0.f, cl_lo = 0.f, ch_hi = 0.f, cl_hi = 0.f;
    float xh = 0.f, xl = 0.f;
    if constexpr (kRows) {
      float slice_h, slice_l;
      row_carries<kRowsPerSeg>(tot_h, tot_l, g, ch_lo, cl_lo, ch_hi, cl_hi, slice_h, slice_l);
      if constexpr (kCross) {
        const int w0 = warp & ~(kWarpsPerSeg - 1);
        const uint32_t slot = i % kPartSlots;
        if (lane == 0)
          part[slot][warp] = make_float2(active ? slice_h : 0.f, active ? slice_l : 0.f);
        if constexpr (kP2P) {
          if (lane == 0) st_release_cta(&part_seq[slot][warp], i + 1u);
          // lane k waits for the k-th earlier warp of the segment
          bool ready = w0 + lane >= warp;
          for (uint32_t spin = 0; !__all_sync(0xffffffffu, ready); ++spin) {
            if (!ready) ready = ld_acquire_cta(&part_seq[slot][w0 + lane]) == i + 1u;
            if ((spin & 1023u) == 1023u && spin > wait_limit(&g_wait_limits.flag)) {
              if (lane == 0) raise_error(kErrBarrierTimeout);  // a warp of this CTA died
              dead = true;
              break;
            }
          }
        } else {
          consumer_sync_n<W>();
        }
        for (int w = w0; w < warp; ++w) {
          const float2 pr = part[slot][w];
          xh += pr.x;
          xl += pr.y;
        }
        // everything before this slice in its segment rides along with the row carries
        ch_lo += xh;
        ch_hi += xh;
        cl_lo += xl;
        cl_hi += xl;
      }
    }
    if (active) {
      const unsigned long long elem_base = slice_off / 2;
      const int valid_elems = valid_bytes / 2;
#pragma unroll
      for (int j = 0; j < kSteps; ++j) {
        if constexpr (!kScanCache) load_split(addr, j, ah[0], al[0]);  // second read
        scan_step<SC, OUT32, W>(j, ah[kScanCache ? j : 0], al[kScanCache ? j : 0], ops, ch_lo, cl_lo,
                                ch_hi, cl_hi, p.out, elem_base, valid_elems, g, t,
                                kBulkStore ? slice : nullptr);
      }
    }
    if constexpr (kBulkStore) {
      fence_proxy_async_smem();  // the generic-proxy writes above, before the bulk copy reads them
      __syncwarp();
      if (lane == 0) {
        if (active)
          tma_store_1d(static_cast<uint8_t*>(p.out) + slice_off, smem_u32(slice),
                       static_cast<uint32_t>(valid_bytes));
        bulk_commit_group();
        bulk_wait_group_read<1>();  // the previous tile's copy has read its stage
        if (i > 0) mbar_arrive(empty0 + 8 * ((i - 1) % kStages));
      }
    }
    if constexpr (!kScanCache) {
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
  }
  if constexpr (kBulkStore) {
    if (lane == 0) bulk_wait_group_read<0>();  // shared memory must outlive the copies that read it
  }
}

}  // namespace TCU_NS
