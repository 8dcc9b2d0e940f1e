// Segmented reduction of segments of 16 ... 2048 elements on the
// fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor
// memory.  Same contraction as reduce_kernels.cuh -- rows of the input times a
// constant 0/1 matrix -- but issued the Blackwell way: one thread launches
// M=128 x N=16 x K=16 MMAs that read both operands straight from shared memory
// (no register fragments), four MMAs cover a 128 x 64 tile (16 KiB), and four
// epilogue warps read the sums back with tcgen05.ld, one output row per thread
// (segments of 128 elements and more are 2 ... 32 rows: the epilogue adds the
// row sums of neighbouring lanes with shuffles).
//
//   A (128 x 64 halves, K-major): tile rows = 64 consecutive input halves,
//       loaded by a swizzled tensor-map TMA copy (SWIZZLE_128B).
//   B (16 x 64, K-major, same swizzle): B[n][k] = 1 iff k / S == n, built once
//       in shared memory; column n of D is the sum of the n-th segment of a row.
//   D (128 lanes x 16 fp32 columns of TMEM), a ring of accumulators deep enough
//       to hide the MMA -> commit -> tcgen05.ld -> release round trip.
//
// Warps: 0 TMA producer, 1 MMA issuer (and TMEM owner), 2..9 epilogue (two sets).  Every
// mbarrier wait is bounded; TMEM is released on every path out of the kernel.
#pragma once

#include "common.cuh"
#include "reduce_kernels.cuh"

namespace TCU_NS {

constexpr int kUmmaRows       = 128;                               // rows (TMEM lanes) per tile
constexpr int kUmmaTileElems  = kUmmaRows * kSwizzleRowElems;      // 8192 halves
constexpr int kUmmaTileBytes  = kUmmaTileElems * 2;                // 16 KiB
// Ring: stages of TWO tiles (32 KiB, one tensor-map copy, one round of barrier operations for
// the producer and the issuer thread), 3 of them.  With stages of one tile this variant stayed at
// 0.90 of the copy bandwidth whatever the depth (3 ... 12 stages), the form of the copy (linear
// or tensor map) or the number of epilogue warps: a kernel that only reads turns tiles over
// twice as fast as a scan, and the single-thread chains of barrier operations set the pace.
// Measured at 2^28 elements with 2 / 3 / 4 / 6 stages of two tiles: 0.87-0.93 / 0.96-1.02 /
// 0.95-1.00 / 0.88-0.92 (segment sizes 64 ... 2048; 16-element segments 0.81 / 0.89 / 0.89 / 0.83,
// bound by their 4 bytes written per 32 read like the mma.sync kernel's 0.92 in the same run).
constexpr int kUmmaStages     = 3;
constexpr int kUmmaPerStage   = 2;                                 // tiles a ring stage holds
constexpr int kUmmaStageBytes = kUmmaPerStage * kUmmaTileBytes;    // 32 KiB, one tensor-map copy
constexpr int kUmmaN          = 16;                                // accumulator columns per tile
constexpr int kUmmaBBytes     = kUmmaN * kSwizzleRowElems * 2;     // 2 KiB
constexpr int kUmmaEpiSets    = 2;  // sets of four epilogue warps that take alternate stages
constexpr int kUmmaThreads    = (2 + 4 * kUmmaEpiSets) * 32;
constexpr int kUmmaAccStages  = 4;              // accumulators in flight (power of two)
constexpr int kUmmaAccCols    = kUmmaPerStage * kUmmaN;            // accumulator columns of one stage
constexpr int kUmmaTmemCols   = kUmmaAccStages * kUmmaAccCols < 32 ? 32 : kUmmaAccStages * kUmmaAccCols;
static_assert((kUmmaAccStages & (kUmmaAccStages - 1)) == 0 && kUmmaTmemCols <= 512 &&
              (kUmmaTmemCols & (kUmmaTmemCols - 1)) == 0, "TMEM columns: a power of two, 32..512");
constexpr int kUmmaDynSmemBytes = kUmmaStages * kUmmaStageBytes + kUmmaBBytes + 1024;

// 64-bit shared-memory matrix descriptor, K-major, 128-byte swizzle: start
// address and offsets in 16-byte units; rows of one 8-row group are 128 bytes
// apart, groups 1024 bytes apart (stride byte offset); descriptor version 1;
// layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) |
         (1ull << 46) | (2ull << 61);
}

// 32-bit instruction descriptor: fp32 accumulator (bit 4), A and B formats
// (bits 7-9 and 10-12: 0 = f16, 1 = bf16), both K-major, N = 16 (field
// N >> 3), M = 128 (field M >> 4).
constexpr uint32_t kUmmaAB        = TCU_BF16 ? 1u : 0u;
constexpr uint32_t kUmmaInstrDesc = (1u << 4) | (kUmmaAB << 7) | (kUmmaAB << 10) |
                                    ((kUmmaN >> 3) << 17) | ((kUmmaRows >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kUmmaInstrDesc), "r"(accumulate)
      : "memory");
}

// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

template <int LOG2S>
__global__ void __launch_bounds__(kUmmaThreads, 1)
    tcgen05_reduce_kernel(const ReduceParams p, const __grid_constant__ CUtensorMap tmap) {
  static_assert(LOG2S >= 4 && LOG2S <= 11, "16 ... 2048 elements per segment");
  // 4, 2 or 1 sums per 64-element row; from 128 elements on a segment is 2 ... 32 whole rows
  constexpr int kSegsPerRow = LOG2S <= 6 ? (kSwizzleRowElems >> LOG2S) : 1;
  constexpr int kRowsPerSeg = LOG2S <= 6 ? 1 : (1 << (LOG2S - 6));
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * kUmmaStages + 2 * kUmmaAccStages];
  __shared__ uint32_t s_tmem_base;
  __shared__ uint32_t s_failed;

  uint8_t* tiles = dyn_smem + ((1024u - (smem_u32(dyn_smem) & 1023u)) & 1023u);
  uint8_t* bmat  = tiles + kUmmaStages * kUmmaStageBytes;  // 1 KiB aligned as well
  const uint32_t tiles_u32 = smem_u32(tiles), bmat_u32 = smem_u32(bmat);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kUmmaStages]);
  const uint32_t tfull0 = smem_u32(&bars[2 * kUmmaStages]), tempty0 = tfull0 + 8 * kUmmaAccStages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap)) : "memory");
    for (int s = 0; s < kUmmaStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < kUmmaAccStages; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 4);  // one arrival per epilogue warp
    }
    s_failed = 0u;
    mbar_fence_init();
    {
      // This thread is also the producer: it fills the ring right away, so the first tiles are
      // in flight while the others build B and allocate tensor memory.
      pdl_prologue();
      const unsigned long long rows  = p.num_elems / kSwizzleRowElems;
      const unsigned long long tiles = (rows + kUmmaPerStage * kUmmaRows - 1) / (kUmmaPerStage * kUmmaRows);
      unsigned long long tile = blockIdx.x;
      for (int s = 0; s < kUmmaStages && tile < tiles; ++s, tile += gridDim.x) {
        mbar_arrive_expect_tx(full0 + 8 * s, kUmmaStageBytes);
        tma_load_2d(tiles_u32 + s * kUmmaStageBytes, &tmap, 0, (int)(tile * kUmmaPerStage * kUmmaRows),
                    full0 + 8 * s);
      }
    }
  }
  // B operand, written through the same 128-byte swizzle the MMA expects.
  for (int idx = threadIdx.x; idx < kUmmaN * kSwizzleRowElems; idx += kUmmaThreads) {
    const int n = idx / kSwizzleRowElems, k = idx % kSwizzleRowElems;
    const bool one = n < kSegsPerRow && (k >> LOG2S) == n;
    *reinterpret_cast<uint16_t*>(bmat + swizzle128(n * 128 + k * 2)) =
        one ? static_cast<uint16_t>(kOne16) : uint16_t(0);
  }
  // make the generic-proxy writes of B visible to the tensor core's async reads
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {  // TMEM allocation is a whole-warp operation; the base address lands in smem
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&s_tmem_base)), "r"(static_cast<uint32_t>(kUmmaTmemCols)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  pdl_prologue();  // nothing above touched global memory
  const uint32_t tmem_base = s_tmem_base;

  const unsigned long long num_rows  = p.num_elems / kSwizzleRowElems;
  // A ring stage, and a step of every role, is kUmmaPerStage tiles: with single tiles the chains
  // of barrier operations of the producer and issuer threads, not HBM, set the pace of a kernel
  // that only reads (0.90 of the copy bandwidth whatever the ring depth or the copy's form).
  const unsigned long long num_tiles =
      (num_rows + kUmmaPerStage * kUmmaRows - 1) / (kUmmaPerStage * kUmmaRows);

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      // the first kUmmaStages tiles were requested before the CTA-wide set-up (see above)
      uint32_t i = kUmmaStages;
      for (unsigned long long tile = blockIdx.x + (unsigned long long)i * gridDim.x; tile < num_tiles;
           tile += gridDim.x, ++i) {
        const uint32_t s = i % kUmmaStages, ph = (i / kUmmaStages) & 1u;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u)) { s_failed = 1u; break; }
        mbar_arrive_expect_tx(full0 + 8 * s, kUmmaStageBytes);  // rows past the end arrive as zeros
        tma_load_2d(tiles_u32 + s * kUmmaStageBytes, &tmap, 0, (int)(tile * kUmmaPerStage * kUmmaRows),
                    full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t i = 0;
      for (unsigned long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++i) {
        const uint32_t s = i % kUmmaStages, ph = (i / kUmmaStages) & 1u;
        const uint32_t a = i % kUmmaAccStages, aph = (i / kUmmaAccStages) & 1u;
        if (!mbar_wait(tempty0 + 8 * a, aph ^ 1u)) { s_failed = 1u; break; }  // accumulator drained
        if (!mbar_wait(full0 + 8 * s, ph)) { s_failed = 1u; break; }          // tile landed
        tcgen05_fence_after_sync();
        const uint32_t a_addr = tiles_u32 + s * kUmmaStageBytes;
#pragma unroll
        for (int h = 0; h < kUmmaPerStage; ++h)
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)  // K = 64 halves in four steps of 16 (32 bytes)
            umma_f16(tmem_base + a * kUmmaAccCols + h * kUmmaN,
                     umma_smem_desc(a_addr + h * kUmmaTileBytes + 32 * kb),
                     umma_smem_desc(bmat_u32 + 32 * kb), kb > 0 ? 1u : 0u);
        umma_commit(empty0 + 8 * s);   // the stage may be refilled once these MMAs have read it
        umma_commit(tfull0 + 8 * a);   // ... and the epilogue may read the accumulator
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // a warp may only touch TMEM lanes 32*(warp%4) .. +31
    const bool out_f32 = p.out_is_f32 != 0;
    uint32_t i = (warp - 2) / 4;  // this warp's set: tiles i, i + kUmmaEpiSets, ... of the CTA
    for (unsigned long long tile = blockIdx.x + (unsigned long long)i * gridDim.x; tile < num_tiles;
         tile += (unsigned long long)kUmmaEpiSets * gridDim.x, i += kUmmaEpiSets) {
      const uint32_t a = i % kUmmaAccStages, aph = (i / kUmmaAccStages) & 1u;
      if (!mbar_wait(tfull0 + 8 * a, aph)) { s_failed = 1u; break; }
      tcgen05_fence_after_sync();
      uint32_t r[kUmmaPerStage][4];
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * kUmmaAccCols;
#pragma unroll
      for (int h = 0; h < kUmmaPerStage; ++h)
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r[h][0]), "=r"(r[h][1]), "=r"(r[h][2]), "=r"(r[h][3])
                     : "r"(taddr + h * kUmmaN) : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * a);  // values are in registers now
#pragma unroll
      for (int h = 0; h < kUmmaPerStage; ++h) {
        const unsigned long long row = (tile * kUmmaPerStage + h) * kUmmaRows + quarter * 32 + lane;
        if constexpr (kRowsPerSeg > 1) {
          // a segment is kRowsPerSeg consecutive rows = consecutive lanes of this warp: add the row
          // sums up (rows past the end of the array are zeros and join harmlessly)
          float v = __uint_as_float(r[h][0]);
#pragma unroll
          for (int m = 1; m < kRowsPerSeg; m <<= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
          const unsigned long long seg = row / kRowsPerSeg;
          if ((lane & (kRowsPerSeg - 1)) == 0 && seg < p.num_segments) store_seg(p.out, out_f32, seg, v);
        } else {
          const unsigned long long seg = row * kSegsPerRow;
          if (seg < p.num_segments) {  // rows past the end of the array hold zeros: not stored
            const float v0 = __uint_as_float(r[h][0]), v1 = __uint_as_float(r[h][1]);
            const float v2 = __uint_as_float(r[h][2]), v3 = __uint_as_float(r[h][3]);
            if constexpr (kSegsPerRow == 4) {
              if (out_f32) {
                *reinterpret_cast<float4*>(static_cast<float*>(p.out) + seg) = make_float4(v0, v1, v2, v3);
              } else {
                *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.out) + seg) =
                    make_uint2(pack2_rn(v0, v1), pack2_rn(v2, v3));
              }
            } else if constexpr (kSegsPerRow == 2) {
              store_seg(p.out, out_f32, seg, v0);
              store_seg(p.out, out_f32, seg + 1, v1);
            } else {
              store_seg(p.out, out_f32, seg, v0);
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ exit
  tcgen05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && s_failed) raise_error(kErrBarrierTimeout);
  if (warp == 1) {
    tcgen05_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"(static_cast<uint32_t>(kUmmaTmemCols)) : "memory");
  }
}

}  // namespace TCU_NS
