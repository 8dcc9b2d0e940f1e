// Segmented inclusive scan on the fifth-generation tensor cores: tcgen05.mma
// with the accumulators in tensor memory, for segments of 16 ... 16384 elements
// (16-bit outputs: up to 2^20).
//
// The contraction is the one of compute_wmma_segmented_prefixsum_16n / _256n
// (src/prefixsum/kernel.cuh:86-150,441-506) -- rows of the input times the
// upper-triangular ones matrix U -- at the shape Blackwell's tensor core wants:
// one tile is 128 rows of 64 consecutive halves, D[128 x 64] = A[128 x 64] .
// U[64 x 64] gives 128 independent 64-wide inclusive scans per instruction
// group (four K = 16 steps), issued by one thread, both operands read from
// shared memory, the fp32 result in tensor memory.  A row's total is the last
// column of its scan; the carries between the rows of a segment are a
// shuffle scan over those totals (exact hi / lo float pairs), added while the
// results are on their way from tensor memory to global memory.  A warp reads
// 32 rows (2048 elements) of a tile; longer segments are spread over several
// tiles, one quarter of each, so that one warp still meets all rows of "its"
// segment in order and carries the running total in registers.
//
// Exactness is kept the way the mma.sync kernels keep it (split_hi_lo): four
// warps split every tile into an exact "hi" tile and an exact "lo" tile in
// shared memory (written in the 128-byte-swizzled K-major layout the tensor
// core reads), the tensor core scans both, and every output is
// (hi + carry_hi) + (lo + carry_lo): both sums exact, one rounding.
//
// Warps: 0 TMA producer | 1 MMA issuer, owner of the tensor memory | 2-5 split
// | 6-13 epilogue, two sets of four taking alternate tiles (tcgen05.ld 32x32b:
// one row of 64 outputs per thread).  A
// thread's row is 128 or 256 contiguous bytes of the output and its neighbours'
// rows lie that far apart, so storing from registers would touch 32 lines per
// instruction (measured: 0.60 of the copy bandwidth whatever the output type);
// the rows go to a swizzled staging buffer instead and leave as one tensor-map
// bulk store per warp and tile, which also clips the rows past the end of the
// array.  Every wait is bounded; tensor memory is freed on every exit path.
#pragma once

#include "scan_kernels.cuh"
#include "tcgen05_reduce_kernel.cuh"

namespace TCU_NS {

constexpr int kUscanRawStages   = 4;                   // 16 KiB tiles as the TMA copies deliver them (at most)
constexpr int kUscanSplitStages = 2;                   // (hi, lo) tile pairs, 32 KiB each
constexpr int kUscanAccStages   = 2;                   // accumulator pairs in tensor memory
constexpr int kUscanMaxLog2     = 20;                  // longest segment (spread over 2^9 tiles)
constexpr int kUscanN           = 64;                  // columns of U = outputs per row
constexpr int kUscanBBytes      = kUscanN * 128;       // U, K-major: 64 rows of 64 halves
constexpr int kUscanTmemCols    = kUscanAccStages * 2 * kUscanN;  // 256
constexpr int kUscanThreads     = 14 * 32;             // producer, MMA issuer, 4 split, 2 x 4 epilogue warps
// staging: two buffers of 32 box rows x 128 bytes for each of the eight epilogue warps
constexpr int kUscanStageBytes   = 32 * 128;
constexpr int kUscanDynSmemBytes = kUscanRawStages * kUmmaTileBytes +
                                   kUscanSplitStages * 2 * kUmmaTileBytes + kUscanBBytes +
                                   8 * 2 * kUscanStageBytes + 1024;
constexpr uint32_t kUscanInstrDesc = (1u << 4) | (kUmmaAB << 7) | (kUmmaAB << 10) |
                                     ((kUscanN >> 3) << 17) | ((kUmmaRows >> 4) << 24);

__device__ __forceinline__ void umma_f16_desc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 16 consecutive accumulator columns of this thread's row
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
  uint32_t r;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
  return r;
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Packed fp32 add (two lanes of a 64-bit register pair per instruction; new with sm_100).
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// One box of a 2-D tensor map, shared memory -> global, tracked by the issuing
// thread's bulk async-group.  Rows of the box that lie past the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, int c0, int c1, uint32_t src_smem) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(src_smem)
               : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tmap, int c0, int c1, int c2, uint32_t src_smem) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(src_smem)
               : "memory");
}

// Registers are per SM sub-partition (16 K): 14 warps put four on one, so a thread may use 128
// at most.  A bound of 512 threads makes the compiler keep to exactly that.
// kExcl: exclusive scan.  Segments shorter than a row: U is strictly triangular; longer ones: U
// stays inclusive (its last column is the row total the carries need) and every thread shifts its
// row by one column on the way out -- column 0 is the carry alone.
template <int LOG2S, bool OUT32, bool kExcl = false>
__global__ void __launch_bounds__(512, 1)
    tcgen05_scan_kernel(const ScanParams p, const __grid_constant__ CUtensorMap omap) {
  static_assert(LOG2S >= 4 && LOG2S <= kUscanMaxLog2, "16 ... 2^20 elements per segment");
  static_assert(LOG2S <= 14 || !OUT32, "segments longer than 16384 elements: 16-bit outputs only");
  constexpr int S = 1 << LOG2S;
  // Segments of more than 2048 elements (32 rows, what one epilogue warp reads of a tile) are
  // spread over G tiles so that one warp still sees a whole segment: a group is four consecutive
  // segments, and tile j of a group holds rows 32 j ... 32 j + 31 of each of them, one segment
  // per quarter of the tile.  The warp of a quarter then meets its segment's rows in order, tile
  // after tile, and carries the running total in a register: no warp waits for another.
  constexpr int G            = LOG2S > 11 ? 1 << (LOG2S - 11) : 1;
  constexpr int kPer         = G == 1 ? 1 : 2 * G;  // tiles of one work unit (a tile, or two groups)
  constexpr int kRowsPerSeg  = S <= 64 ? 1 : (G > 1 ? 32 : S / 64);  // rows of a segment in a tile
  constexpr int kLanesPerSeg = kRowsPerSeg;
  // Depth of the input ring, measured at 2^28 elements (2 / 3 / 4 / 5 stages): fp32 outputs 0.90 /
  // 0.95 / 0.88 / -- of the copy bandwidth at every segment size (reads that run far ahead get in
  // the way of twice as many bytes of writes); 16-bit outputs -- / 0.93 / 1.00 / 0.89 at 256
  // elements per segment, 0.88 / 0.98 / 0.88 at 4096, 0.93 / 0.95 / 0.87 at 16.
  constexpr int NR = OUT32 ? 3 : kUscanRawStages;
  constexpr int NH = kUscanSplitStages, NA = kUscanAccStages;
  extern __shared__ uint8_t dyn_smem[];
  // raw_full | raw_empty | hl_full | hl_empty | acc_full | acc_empty
  __shared__ __align__(8) uint64_t bars[2 * NR + 2 * NH + 2 * NA];
  __shared__ uint32_t s_tmem_base;
  __shared__ uint32_t s_failed;

  uint8_t* raw   = dyn_smem + ((1024u - (smem_u32(dyn_smem) & 1023u)) & 1023u);
  uint8_t* split = raw + NR * kUmmaTileBytes;            // [NH][hi | lo]
  uint8_t* bmat  = split + NH * 2 * kUmmaTileBytes;      // all 1 KiB aligned
  uint8_t* stage = bmat + kUscanBBytes;                  // [2 sets][4 warps][2 buffers]
  const uint32_t raw_u32 = smem_u32(raw), split_u32 = smem_u32(split), bmat_u32 = smem_u32(bmat);
  const uint32_t raw_full0 = smem_u32(&bars[0]), raw_empty0 = raw_full0 + 8 * NR;
  const uint32_t hl_full0 = raw_empty0 + 8 * NR, hl_empty0 = hl_full0 + 8 * NH;
  const uint32_t acc_full0 = hl_empty0 + 8 * NH, acc_empty0 = acc_full0 + 8 * NA;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const unsigned long long num_rows = p.num_elems / kSwizzleRowElems;
  // Work units are interleaved over the CTAs.  A unit is one tile, or, for spread segments, two
  // groups whose tiles alternate (tile i of the unit belongs to group i % 2): the two sets of
  // epilogue warps, which take alternate tiles, then own one group each.
  const unsigned long long num_units =
      G == 1 ? (num_rows + kPer * kUmmaRows - 1) / (kPer * kUmmaRows)
             : (num_rows + 2ull * G * kUmmaRows - 1) / (2ull * G * kUmmaRows);
  auto unit_of = [&](uint32_t i) -> unsigned long long {
    return blockIdx.x + (unsigned long long)(i / kPer) * gridDim.x;
  };
  // First of the 32 rows that quarter q of this CTA's i-th tile holds.
  auto quarter_row = [&](uint32_t i, int q) -> unsigned long long {
    if constexpr (G == 1) {
      return (unit_of(i) * kPer + i % kPer) * kUmmaRows + 32ull * q;
    } else {
      const uint32_t r = i % kPer;
      const unsigned long long group = 2ull * unit_of(i) + (r & 1u);
      return (group * 4ull + q) * (32ull * G) + 32ull * (r >> 1);
    }
  };

  // Requests the CTA's i-th tile into its ring stage (one thread).
  auto issue_tile = [&](uint32_t i) {
    const uint32_t s = i % NR;
    // Linear copies (measured faster than a tensor-map copy; the split warps put the tile into
    // the layout the tensor core wants): 16 KiB of consecutive input, or one piece of 4 KiB
    // per quarter.  Behind the end of the array the stage keeps stale data: those rows only
    // feed rows after them, and none of these is stored.
    const uint32_t dst = raw_u32 + s * kUmmaTileBytes, bar = raw_full0 + 8 * s;
    if constexpr (G == 1) {
      const unsigned long long row = quarter_row(i, 0);
      if (row >= num_rows) {
        mbar_arrive(bar);
      } else {
        const unsigned long long rem = (num_rows - row) * 128ull;
        const uint32_t bytes = rem < (unsigned long long)kUmmaTileBytes ? (uint32_t)rem : kUmmaTileBytes;
        mbar_arrive_expect_tx(bar, bytes);
        tma_load_1d(dst, p.in + row * 128ull, bytes, bar);
      }
    } else {
      // whole segments only: a quarter's 32 rows are all inside the array or all outside
      uint32_t pieces = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) pieces += quarter_row(i, q) < num_rows ? 1u : 0u;
      if (pieces == 0) {
        mbar_arrive(bar);
      } else {
        mbar_arrive_expect_tx(bar, pieces * 4096u);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const unsigned long long row = quarter_row(i, q);
          if (row < num_rows) tma_load_1d(dst + q * 4096u, p.in + row * 128ull, 4096u, bar);
        }
      }
    }
  };

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&omap)) : "memory");
    for (int s = 0; s < NR; ++s) {
      mbar_init(raw_full0 + 8 * s, 1);
      mbar_init(raw_empty0 + 8 * s, 4);  // one arrival per split warp
    }
    for (int h = 0; h < NH; ++h) {
      mbar_init(hl_full0 + 8 * h, 4);    // one arrival per split warp
      mbar_init(hl_empty0 + 8 * h, 1);   // tcgen05.commit
    }
    for (int a = 0; a < NA; ++a) {
      mbar_init(acc_full0 + 8 * a, 1);   // tcgen05.commit
      mbar_init(acc_empty0 + 8 * a, 4);  // one arrival per epilogue warp
    }
    s_failed = 0u;
    mbar_fence_init();
    // This thread is also the producer: it fills the ring right away, so that the first tiles are
    // in flight while the others build U and allocate tensor memory.
    pdl_prologue();
    for (uint32_t i = 0; i < (uint32_t)NR && unit_of(i) < num_units; ++i) issue_tile(i);
  }
  // U restricted to the segments inside a row: B[n][k] = 1 iff k <= n and both in one segment.
  for (int idx = threadIdx.x; idx < kUscanN * kSwizzleRowElems; idx += kUscanThreads) {
    const int n = idx / kSwizzleRowElems, k = idx % kSwizzleRowElems;
    const bool one = (kExcl && S < 64 ? k < n : k <= n) && (S >= 64 || (k >> LOG2S) == (n >> LOG2S));
    *reinterpret_cast<uint16_t*>(bmat + swizzle128(n * 128 + k * 2)) =
        one ? static_cast<uint16_t>(kOne16) : uint16_t(0);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // B: generic writes -> async reads
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&s_tmem_base)), "r"(static_cast<uint32_t>(kUscanTmemCols)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  pdl_prologue();  // nothing above touched global memory
  const uint32_t tmem_base = s_tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      // the first NR tiles were requested before the CTA-wide set-up (see above)
      for (uint32_t i = NR; unit_of(i) < num_units; ++i) {
        const uint32_t s = i % NR, ph = (i / NR) & 1u;
        // 16-element segments with 16-bit outputs measured best with a producer that does not
        // refill a stage the instant it is free: 0.98 of the copy bandwidth at 2^28 elements with a
        // pause of 500 ns or 1 us after a failed look, 0.94 with none or 250 ns, 0.91 with 2 us
        const bool got = (LOG2S == 4 && !OUT32) ? mbar_wait_paced(raw_empty0 + 8 * s, ph ^ 1u, 500u)
                                                : mbar_wait(raw_empty0 + 8 * s, ph ^ 1u);
        if (!got) { s_failed = 1u; break; }
        issue_tile(i);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      for (uint32_t i = 0; unit_of(i) < num_units; ++i) {
        const uint32_t h = i % NH, hph = (i / NH) & 1u;
        const uint32_t a = i % NA, aph = (i / NA) & 1u;
        if (!mbar_wait(acc_empty0 + 8 * a, aph ^ 1u)) { s_failed = 1u; break; }  // accumulators drained
        if (!mbar_wait(hl_full0 + 8 * h, hph)) { s_failed = 1u; break; }         // hi and lo written
        tcgen05_fence_after_sync();
        const uint32_t hi_addr = split_u32 + h * 2 * kUmmaTileBytes, lo_addr = hi_addr + kUmmaTileBytes;
        const uint32_t d_hi = tmem_base + a * 2 * kUscanN, d_lo = d_hi + kUscanN;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)  // K = 64 halves in four steps of 16 (32 bytes)
          umma_f16_desc(d_hi, umma_smem_desc(hi_addr + 32 * kb), umma_smem_desc(bmat_u32 + 32 * kb),
                        kUscanInstrDesc, kb > 0 ? 1u : 0u);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
          umma_f16_desc(d_lo, umma_smem_desc(lo_addr + 32 * kb), umma_smem_desc(bmat_u32 + 32 * kb),
                        kUscanInstrDesc, kb > 0 ? 1u : 0u);
        umma_commit(hl_empty0 + 8 * h);  // the pair may be overwritten once these MMAs have read it
        umma_commit(acc_full0 + 8 * a);  // ... and the epilogue may read the accumulators
      }
    }
  } else if (warp < 6) {
    // --------------------------------------------------------------- split
    const int tid = threadIdx.x - 64;  // 0 .. 127
    for (uint32_t i = 0; unit_of(i) < num_units; ++i) {
      const uint32_t s = i % NR, ph = (i / NR) & 1u;
      const uint32_t h = i % NH, hph = (i / NH) & 1u;
      if (!mbar_wait(raw_full0 + 8 * s, ph)) { s_failed = 1u; break; }
      if (!mbar_wait(hl_empty0 + 8 * h, hph ^ 1u)) { s_failed = 1u; break; }
      // 16-byte chunk tid + 128 c of the tile: row 16 c + tid / 8, chunk tid % 8 of that row; in
      // the hi / lo tiles it goes where the 128-byte swizzle puts it (chunk index XOR row mod 8)
      const uint8_t* src = raw + s * kUmmaTileBytes + 16 * tid;
      uint8_t* hi = split + h * 2 * kUmmaTileBytes + 128 * (tid >> 3) + (((tid & 7) ^ ((tid >> 3) & 7)) << 4);
      uint8_t* lo = hi + kUmmaTileBytes;
      uint4 w[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) w[c] = lds128(src + 2048 * c);
      __syncwarp();
      if (lane == 0) mbar_arrive(raw_empty0 + 8 * s);  // the tile is in registers
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 vh, vl;
        split_hi_lo(w[c].x, vh.x, vl.x);
        split_hi_lo(w[c].y, vh.y, vl.y);
        split_hi_lo(w[c].z, vh.z, vl.z);
        split_hi_lo(w[c].w, vh.w, vl.w);
        *reinterpret_cast<uint4*>(hi + 2048 * c) = vh;
        *reinterpret_cast<uint4*>(lo + 2048 * c) = vl;
      }
      fence_proxy_async_smem();  // generic writes of hi / lo, before the tensor core reads them
      __syncwarp();
      if (lane == 0) mbar_arrive(hl_full0 + 8 * h);
    }
  } else {
    // ------------------------------------------------------------ epilogue
    // Two sets of four warps take alternate tiles (set e: tiles e, e + 2, ... of this CTA, which
    // are the tiles of accumulator stage e), so that one set's trip through tensor memory, the
    // carry shuffles and the staging overlaps the other's.
    const int quarter = warp & 3;  // a warp may only touch TMEM lanes 32*(warp%4) .. +31
    const uint32_t set = warp >= 10 ? 1u : 0u;
    float rh = 0.f, rl = 0.f;  // spread segments: the total of the segment's rows in the group's earlier tiles
    for (uint32_t i = set; unit_of(i) < num_units; i += 2) {
      const uint32_t a = i % NA, aph = (i / NA) & 1u;
      if (!mbar_wait(acc_full0 + 8 * a, aph)) { s_failed = 1u; break; }
      tcgen05_fence_after_sync();
      const uint32_t t_hi = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * 2 * kUscanN;
      const uint32_t t_lo = t_hi + kUscanN;

      // first half of the row, and the row totals (the last column), in one trip
      uint32_t vh[2][16], vl[2][16];
      uint32_t uh = 0, ul = 0;
      tmem_ld16(t_hi, vh[0]);
      tmem_ld16(t_hi + 16, vh[1]);
      tmem_ld16(t_lo, vl[0]);
      tmem_ld16(t_lo + 16, vl[1]);
      if constexpr (kRowsPerSeg > 1) {
        uh = tmem_ld1(t_hi + 63);
        ul = tmem_ld1(t_lo + 63);
      }
      tmem_wait_ld();

      // carry into this row: the totals of the earlier rows of its segment
      float cb = 0.f, cs = 0.f, big = 0.f;
      if constexpr (kRowsPerSeg > 1) {
        // Rows of one warp: an exclusive shuffle scan of their totals.  A warp holds at most 2048
        // elements, so the sums of exact hi parts and of exact lo parts stay exact in fp32.
        float ih = __uint_as_float(uh), il = __uint_as_float(ul);
#pragma unroll
        for (int d = 1; d < kLanesPerSeg; d <<= 1) {
          const float x = __shfl_up_sync(0xffffffffu, ih, d), y = __shfl_up_sync(0xffffffffu, il, d);
          if ((lane & (kLanesPerSeg - 1)) >= d) {
            ih += x;
            il += y;
          }
        }
        cb = __shfl_up_sync(0xffffffffu, ih, 1);
        cs = __shfl_up_sync(0xffffffffu, il, 1);
        if ((lane & (kLanesPerSeg - 1)) == 0) cb = cs = 0.f;
        if constexpr (G > 1) {
          // The segment goes on over the group's tiles.  What this warp met of it so far is kept
          // as two floats (double arithmetic measured 7 % of the kernel's time here): rh, a sum of
          // hi parts and so a multiple of 2^-13, exact below 2^11, and rl, the sum of the lo parts
          // less its multiples of 2^-13, which move over to rh; beyond 2^11 rl also takes what
          // the additions to rh round off, so that rh + rl keeps 48 bits.
          const float th = __shfl_sync(0xffffffffu, ih, 31), tl = __shfl_sync(0xffffffffu, il, 31);
          if ((i % kPer) < 2u) {  // the group's first tile: the segment begins here
            rh = 0.f;
            rl = 0.f;
          } else {
            const float ns = rl + cs;
            const float m  = grid13(ns);
            cs = ns - m;
            float nb, e;
            two_sum(rh, cb + m, nb, e);
            if (fabsf(nb) >= 2048.f) {  // no longer adds exactly: held back and added last
              cs += e;
              big = nb;
              cb  = 0.f;
            } else {
              cb = nb;
            }
          }
          pair_add(rh, rl, th, tl);
          pair_renorm(rh, rl);
        }
      }

      const float2 cb2 = make_float2(cb, cb), cs2 = make_float2(cs, cs);
      const bool any_big = S > 2048 && __any_sync(0xffffffffu, big != 0.f);
      // This thread's outputs go to the warp's staging buffers as box rows of 128 bytes with the
      // 128-byte swizzle the tensor map expects (16-byte chunk index XOR box row mod 8) and leave
      // through bulk tensor stores.  16-bit outputs: a row is one box row, the warp's two
      // buffers take alternate tiles, so the copy of one overlaps the filling of the other.
      // fp32 outputs: a row is two box rows of one 8 KiB box (view {32 floats, 2 halves, rows}),
      // stored whole -- 8 KiB contiguous in global memory per copy; two copies of alternate
      // 128-byte pieces measured 0.86 of the copy bandwidth where the mma.sync kernels reach 0.97.
      const unsigned long long row0 = quarter_row(i, quarter);  // first row of this warp
      uint8_t* const bufs = stage + (set * 4 + quarter) * 2 * kUscanStageBytes;
      constexpr bool kShift = kExcl && S >= 64;
      uint32_t ph = 0u, pl = 0u;  // exclusive: the column before the one being written (bits of 0.f at first)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (half == 1) {
          tmem_ld16(t_hi + 32, vh[0]);
          tmem_ld16(t_hi + 48, vh[1]);
          tmem_ld16(t_lo + 32, vl[0]);
          tmem_ld16(t_lo + 48, vl[1]);
          tmem_wait_ld();
          tcgen05_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty0 + 8 * a);  // the accumulators are in registers now
        }
        uint8_t* const buf = bufs + (OUT32 ? 0 : (int)((i >> 1) & 1u)) * kUscanStageBytes;
        if (half == 0) {
          if (lane == 0) bulk_wait_group_read<OUT32 ? 0 : 1>();  // the store that last read this buffer is done
          __syncwarp();
        }
        uint8_t* const my_row = buf + (OUT32 ? lane * 256 + half * 128 : lane * 128);
        const int key = OUT32 ? (2 * lane + half) & 7 : lane & 7;  // box row mod 8
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          float o[16];
#pragma unroll
          for (int e = 0; e < 16; e += 2) {  // two outputs per packed fp32x2 instruction
            const uint32_t h0 = kShift ? (e == 0 ? ph : vh[cc][e == 0 ? 0 : e - 1]) : vh[cc][e];
            const uint32_t l0 = kShift ? (e == 0 ? pl : vl[cc][e == 0 ? 0 : e - 1]) : vl[cc][e];
            const uint32_t h1 = kShift ? vh[cc][e] : vh[cc][e + 1];
            const uint32_t l1 = kShift ? vl[cc][e] : vl[cc][e + 1];
            const float2 t = add2(add2(make_float2(__uint_as_float(h0), __uint_as_float(h1)), cb2),
                                  add2(make_float2(__uint_as_float(l0), __uint_as_float(l1)), cs2));
            o[e]     = t.x;  // (hi + cb) + (lo + cs): two exact sums, one rounding
            o[e + 1] = t.y;
          }
          if constexpr (kShift) {
            ph = vh[cc][15];
            pl = vl[cc][15];
          }
          if constexpr (S > 2048) {
            if (any_big) {  // warp-uniform: only carries of 2^11 and more are held back
#pragma unroll
              for (int e = 0; e < 16; ++e) o[e] += big;
            }
          }
          if constexpr (OUT32) {  // this half row is one box row of 32 floats
#pragma unroll
            for (int e = 0; e < 16; e += 4) {
              const int j = cc * 4 + e / 4;
              *reinterpret_cast<float4*>(my_row + ((j ^ key) << 4)) =
                  make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
            }
          } else {  // the whole row is one box row of 64 halves
#pragma unroll
            for (int e = 0; e < 16; e += 8) {
              const int j = 2 * (2 * half + cc) + e / 8;
              *reinterpret_cast<uint4*>(my_row + ((j ^ key) << 4)) =
                  make_uint4(pack2_rn(o[e], o[e + 1]), pack2_rn(o[e + 2], o[e + 3]),
                             pack2_rn(o[e + 4], o[e + 5]), pack2_rn(o[e + 6], o[e + 7]));
            }
          }
        }
        if (half == 1) {
          fence_proxy_async_smem();  // generic writes of the buffer, before the bulk store reads it
          __syncwarp();
          if (lane == 0) {
            if (row0 < num_rows) {
              if constexpr (OUT32)
                tma_store_3d(&omap, 0, 0, (int)row0, smem_u32(buf));
              else
                tma_store_2d(&omap, 0, (int)row0, smem_u32(buf));
            }
            bulk_commit_group();
          }
        }
      }
    }
    if (lane == 0) bulk_wait_group_read<0>();  // shared memory must outlive the stores that read it
  }

  // ------------------------------------------------------------------ exit
  tcgen05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && s_failed) raise_error(kErrBarrierTimeout);
  if (warp == 1) {
    tcgen05_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"(static_cast<uint32_t>(kUscanTmemCols)) : "memory");
  }
}

}  // namespace TCU_NS
