// Seeded input fill.  Element i of a logical array is a pure function of
// (seed, i), so every GPU shard and the CPU oracle produce the same bits with
// no transfers.  Stands in for the reference's constant fill
// (cuda_memory_set / setFP16, src/utils/cuda_helpers.cuh:123-181).
#pragma once

#include "common.cuh"

namespace TCU_NS {

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Every value below is exact in fp32 before the one rounding to half, so the
// host and the device cannot disagree.
__device__ __forceinline__ float dist_value(uint64_t h, int dist) {
  const uint32_t u24 = static_cast<uint32_t>(h >> 40);
  switch (dist) {
    case 0: return static_cast<float>(static_cast<int32_t>(u24) - (1 << 23)) * 0x1p-23f;
    case 1: return static_cast<float>(u24) * 0x1p-24f;
    case 2: return static_cast<float>(static_cast<int32_t>(u24 % 5u) - 2);
    default: return 0.001f;
  }
}

// One thread writes 8 consecutive halves (16 bytes).
__global__ void fill_f16_kernel(uint4* out, size_t groups, uint64_t seed, uint64_t first_index,
                                int dist) {
  const uint64_t key = splitmix64(seed);
  for (size_t grp = blockIdx.x * size_t(blockDim.x) + threadIdx.x; grp < groups;
       grp += size_t(gridDim.x) * blockDim.x) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint64_t i0 = key + first_index + grp * 8 + 2 * e;
      w[e] = pack2_rn(dist_value(splitmix64(i0), dist), dist_value(splitmix64(i0 + 1), dist));
    }
    out[grp] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace TCU_NS
