// CUDA-core ablation of the segmented scan: the same TMA ring and the same
// outputs as seg_scan_kernel, but every sum is an fp32 add or a warp shuffle.
// It exists so that a profile can show what the tensor-core formulation buys;
// it does not split inputs into exact parts, so its results carry ordinary
// fp32 rounding.  Not used by default.
#pragma once

#include "scan_kernels.cuh"

namespace TCU_NS {

template <int SC, bool OUT32>
__global__ void __launch_bounds__(kThreads, 1) shuffle_scan_kernel(const ScanParams p) {
  static_assert(SC >= 4 && SC <= 14, "segment classes up to one tile");
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) uint64_t bars[2 * kStages];
  __shared__ float part[2][kConsumerWarps];

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

  if (warp == kConsumerWarps) {
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

  constexpr int S = SC <= 11 ? (1 << SC) : kSliceElems;  // segment extent inside one slice
  constexpr int kLanesPerSeg = S / 8 < 32 ? S / 8 : 32;  // lanes of one 512-byte block per segment
  bool dead = false;

  uint32_t i = 0;
  for (unsigned long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++i) {
    const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
    if (!dead && !mbar_wait(full0 + 8 * s, ph)) dead = true;

    uint8_t* slice = ring + s * kTileBytes + warp * kSliceBytes;
    const unsigned long long slice_off = tile * kTileBytes + (unsigned long long)warp * kSliceBytes;
    const long long left  = (long long)total_bytes - (long long)slice_off;
    const int valid_bytes = left <= 0 ? 0 : (left < kSliceBytes ? (int)left : kSliceBytes);
    const bool active     = !dead && valid_bytes > 0;
    if (active && valid_bytes < kSliceBytes) zero_slice_tail(slice, valid_bytes, lane);

    float run = 0.f;  // carry across the 512-byte blocks of one segment
    if constexpr (SC >= 12) {
      float tot = 0.f;
      if (active) {
#pragma unroll
        for (int j = 0; j < 8; ++j) tot += sum8_halves(lds128(slice + 512 * j + 16 * lane));
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, off);
      if (lane == 0) part[i & 1][warp] = tot;
      consumer_sync();
      constexpr int kWarpsPerSeg = 1 << (SC - 11);
      for (int w = warp & ~(kWarpsPerSeg - 1); w < warp; ++w) run += part[i & 1][w];
    }

    if (active) {
      const unsigned long long elem_base = slice_off / 2;
      const int valid_elems = valid_bytes / 2;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 w = lds128(slice + 512 * j + 16 * lane);
        float f[8];
        {
          const float2 a = unpack2(w.x), b = unpack2(w.y), c = unpack2(w.z), d = unpack2(w.w);
          f[0] = a.x; f[1] = f[0] + a.y; f[2] = f[1] + b.x; f[3] = f[2] + b.y;
          f[4] = f[3] + c.x; f[5] = f[4] + c.y; f[6] = f[5] + d.x; f[7] = f[6] + d.y;
        }
        // inclusive scan of the lane totals across the lanes of one segment
        float inc = f[7];
#pragma unroll
        for (int d = 1; d < kLanesPerSeg; d <<= 1) {
          const float v = __shfl_up_sync(0xffffffffu, inc, d);
          if ((lane & (kLanesPerSeg - 1)) >= d) inc += v;
        }
        float excl = __shfl_up_sync(0xffffffffu, inc, 1);
        if ((lane & (kLanesPerSeg - 1)) == 0) excl = 0.f;
        float base = excl;
        if constexpr (S > 256) {
          base += run;
          const float block_total = __shfl_sync(0xffffffffu, inc, 31);
          run = (((j + 1) * 256) % S == 0) ? 0.f : run + block_total;
        }
        const int e0 = 256 * j + 8 * lane;
        if (e0 < valid_elems) {
          store4<OUT32>(p.out, elem_base + e0, f[0] + base, f[1] + base, f[2] + base, f[3] + base);
          store4<OUT32>(p.out, elem_base + e0 + 4, f[4] + base, f[5] + base, f[6] + base,
                        f[7] + base);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);
  }
}

}  // namespace TCU_NS
