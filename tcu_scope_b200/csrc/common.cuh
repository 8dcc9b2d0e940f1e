// Shared device-side building blocks for the sm_100a reduce / scan kernels:
// tile geometry, mbarrier + TMA bulk-copy wrappers with bounded waits, the
// m16n8k16 tensor-core contraction and the constant operands it is fed.
#pragma once

#include <cuda.h>  // CUtensorMap (the type only; the encoder is looked up at run time)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// The library is compiled twice from the same sources: once for fp16 inputs
// (TCU_BF16 = 0, namespace tcu) and once for bf16 inputs (TCU_BF16 = 1,
// namespace tcu_bf16).  Everything that depends on the 16-bit element type is
// in the few helpers below: the MMA instruction, the constant 1.0, the exact
// hi/lo split and the conversions of the 16-bit outputs.
#ifndef TCU_BF16
#define TCU_BF16 0
#endif
#if TCU_BF16
#define TCU_NS tcu_bf16
#define TCU_MMA_TYPES "f32.bf16.bf16.f32"
#define TCU_X2 "bf16x2"
#else
#define TCU_NS tcu
#define TCU_MMA_TYPES "f32.f16.f16.f32"
#define TCU_X2 "f16x2"
#endif

namespace TCU_NS {

// ---------------------------------------------------------------- geometry
// One CTA tile is what a single TMA bulk copy brings into one ring stage.  A
// tile is cut into one contiguous slice per consumer warp.
constexpr int kConsumerWarps = 8;
constexpr int kSliceElems    = 2048;                         // halves per warp slice
constexpr int kSliceBytes    = kSliceElems * 2;              // 4 KiB
constexpr int kTileElems     = kSliceElems * kConsumerWarps; // 16384 halves per tile
constexpr int kTileBytes     = kTileElems * 2;               // 32 KiB
constexpr int kStages        = 4;                            // 4 stages = 128 KiB in flight per SM
constexpr int kThreads       = (kConsumerWarps + 1) * 32;    // + 1 producer warp
constexpr int kRingBytes     = kStages * kTileBytes;

// Device-side error word bits (read back by tcu_device_error()).
constexpr unsigned kErrBarrierTimeout  = 1u;  // an mbarrier wait ran out
constexpr unsigned kErrLookbackTimeout = 2u;  // a tile-status poll ran out
constexpr unsigned kErrPeerTimeout     = 4u;  // a wait for another GPU's total ran out

// Wait bounds.  try_wait suspends for at most kWaitHintNs per attempt, so a
// wait gives up after roughly barrier * kWaitHintNs (about 2 s) instead of
// hanging the device.  The limits live in device memory so that a test can
// shorten them and make a wait run out within a millisecond; a kernel reads
// them only after a few dozen attempts have failed, never on its fast path.
constexpr uint32_t kWaitHintNs = 1000;
struct WaitLimits {
  uint32_t barrier;  // mbarrier try_wait attempts
  uint32_t status;   // tile-status polls of the look-back (each ~0.5 us)
  uint32_t flag;     // shared-memory flag polls between warps of a CTA
  uint32_t peer;     // polls of a total another GPU stores into this one's memory (each ~0.5 us)
};
constexpr WaitLimits kDefaultWaitLimits = {1u << 21, 1u << 22, 1u << 24, 1u << 23};
__device__ WaitLimits g_wait_limits = kDefaultWaitLimits;

__device__ __forceinline__ uint32_t wait_limit(const uint32_t* field) {
  return *reinterpret_cast<const volatile uint32_t*>(field);
}

__device__ unsigned int g_error_word;  // sticky until cleared by the host

__device__ __forceinline__ void raise_error(unsigned bits) { atomicOr(&g_error_word, bits); }

// ------------------------------------------------------------------ smem / mbarrier
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(kWaitHintNs)
      : "memory");
  return done != 0;
}

// Bounded wait on a phase parity.  Returns false (after raising the error
// word) when the phase never completed.  The bound lives in global memory
// and is fetched only after kFastAttempts attempts have failed: a fetch after
// the first failed attempt put an L2 round trip between a barrier's
// completion and the waiter noticing it, which cost the single-thread chains
// of the tcgen05 reduction a fifth of their throughput.
constexpr uint32_t kFastAttempts = 32;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
#pragma unroll 1
  for (uint32_t attempt = 0; attempt < kFastAttempts; ++attempt)
    if (mbar_try_wait(bar, parity)) return true;
  const uint32_t limit = wait_limit(&g_wait_limits.barrier);
#pragma unroll 1
  for (uint32_t attempt = kFastAttempts; attempt < limit; ++attempt)
    if (mbar_try_wait(bar, parity)) return true;
  raise_error(kErrBarrierTimeout);
  return false;
}

// The same wait for a thread that should not be too quick: after a first failed attempt it
// sleeps `pace_ns` before it looks again.  A producer paced like this runs a little less far
// ahead of the consumers than its ring would let it.
__device__ __forceinline__ bool mbar_wait_paced(uint32_t bar, uint32_t parity, uint32_t pace_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  __nanosleep(pace_ns);
  return mbar_wait(bar, parity);
}

// Linear TMA: global -> this CTA's shared memory, completion counted in bytes
// on an mbarrier.  Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void tma_load_1d(uint32_t dst_smem, const void* src_gmem,
                                            uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst_smem), "l"(src_gmem), "r"(bytes), "r"(bar)
      : "memory");
}

// Flag hand-off between warps of one CTA through shared memory.
__device__ __forceinline__ void st_release_cta(uint32_t* p, uint32_t v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_cta(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}

// Linear TMA the other way: this CTA's shared memory -> global, tracked by the
// issuing thread's bulk async-group.  Same alignment rules.
__device__ __forceinline__ void tma_store_1d(void* dst_gmem, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(dst_gmem), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Returns once all but the newest kPending groups of this thread have finished
// READING shared memory (their global writes may still be in flight).
template <int kPending>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
// Orders this thread's generic-proxy shared-memory writes before later
// async-proxy (TMA, tensor core) reads of the same locations.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Tiled TMA through a tensor map: one box of the 2-D view {64 halves, rows} of
// the input lands in shared memory with the 128-byte swizzle applied (16-byte
// chunk index XOR row index mod 8), which is what makes the scan kernels'
// row-strided 8-byte loads conflict-free.  c0 is an element coordinate (a
// multiple of 8 elements = 16 bytes), c1 a row coordinate; rows past the end
// of the tensor arrive as zeros and still count towards the byte total.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tmap, int c0,
                                            int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// L2 eviction-priority policies for the hinted copies below.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_1d_hint(uint32_t dst_smem, const void* src_gmem,
                                                 uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;"
      ::"r"(dst_smem), "l"(src_gmem), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst_smem, const CUtensorMap* tmap, int c0,
                                                 int c1, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(bar),
        "l"(policy)
      : "memory");
}

constexpr int kSwizzleRowElems = 64;                  // 128-byte rows of the tensor view
constexpr int kTileRows = kTileElems / kSwizzleRowElems;  // 256 rows per tile (the box height)

// Byte offset inside a 1024-byte-aligned tile after the 128-byte swizzle.
__device__ __forceinline__ int swizzle128(int off) { return off ^ (((off >> 7) & 7) << 4); }

// Programmatic dependent launch.  Every kernel of the library lets the next
// kernel in the stream be scheduled early (its CTAs start as SMs drain, and do
// their barrier set-up) and itself touches global memory only after everything
// launched before it has completed and is visible.  Both are no-ops for
// launches made without the programmatic-serialization attribute.
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Named barrier over the consumer warps only (the producer warp never joins).
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}

// ------------------------------------------------------------------ shared loads
__device__ __forceinline__ uint4 lds128(const uint8_t* p) {
  return *reinterpret_cast<const uint4*>(p);
}

__device__ __forceinline__ uint2 lds64(const uint8_t* p) {
  return *reinterpret_cast<const uint2*>(p);
}

// Zero the tail [valid_bytes, kSliceBytes) of one warp's slice.  Only the last
// tile of an array can be short; stale shared memory behind it may hold NaN or
// Inf bit patterns, and 0 * NaN inside the contraction would poison valid rows.
template <int kBytes = kSliceBytes>
__device__ __forceinline__ void zero_slice_tail(uint8_t* slice, int valid_bytes, int lane) {
  for (int b = valid_bytes + lane * 16; b < kBytes; b += 32 * 16)
    *reinterpret_cast<uint4*>(slice + b) = make_uint4(0u, 0u, 0u, 0u);
  __syncwarp();
}

// ------------------------------------------------------------------ tensor core
// D(16x8,f32) = A(16x16,f16,row) * B(16x8,f16,col) + C.  Lane = 4*g + t holds
//   A: a0={row g,  k 2t,2t+1}  a1={row g+8, k 2t,2t+1}
//      a2={row g,  k 2t+8,+9}  a3={row g+8, k 2t+8,+9}
//   B: b0={k 2t,2t+1; n g}     b1={k 2t+8,2t+9; n g}
//   D: d0,d1={row g;   n 2t,2t+1}   d2,d3={row g+8; n 2t,2t+1}
struct Acc {
  float d0, d1, d2, d3;
};

__device__ __forceinline__ Acc mma16816(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1, Acc c) {
  Acc d;
  asm(
      "mma.sync.aligned.m16n8k16.row.col." TCU_MMA_TYPES " "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d.d0), "=f"(d.d1), "=f"(d.d2), "=f"(d.d3)
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c.d0), "f"(c.d1), "f"(c.d2),
        "f"(c.d3));
  return d;
}

constexpr uint32_t kOne16  = TCU_BF16 ? 0x3F80u : 0x3C00u;  // 1.0 in the element type
constexpr uint32_t kOnesH2 = kOne16 | (kOne16 << 16);       // (1, 1)

// Conversions of 16-bit outputs and (for the CUDA-core ablation) inputs.
__device__ __forceinline__ uint32_t pack2_rn(float a, float b) {
#if TCU_BF16
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
#else
  const __half2 v = __floats2half2_rn(a, b);
#endif
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint16_t to16_rn(float a) {
#if TCU_BF16
  const __nv_bfloat16 v = __float2bfloat16_rn(a);
#else
  const __half v = __float2half_rn(a);
#endif
  return *reinterpret_cast<const uint16_t*>(&v);
}
__device__ __forceinline__ float2 unpack2(uint32_t w) {
#if TCU_BF16
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
#else
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
#endif
}

// x = hi + lo exactly, for every finite half x.  hi is x rounded to a multiple
// of 2^-13 or coarser (the ulp of half in [0.25, 0.5) after adding 0.375), so
// sums of up to 2^11 hi parts of inputs in [-1, 1] are exact in fp32; |lo| <=
// 2^-11 and a multiple of 2^-24, so the same holds for the lo parts.  Feeding
// the two parts to separate tensor-core accumulators makes every partial sum
// exact, whatever order and rounding the hardware adder uses.
__device__ __forceinline__ void split_hi_lo(uint32_t x, uint32_t& hi, uint32_t& lo) {
  constexpr uint32_t kMagic = TCU_BF16 ? 0x3EC03EC0u : 0x36003600u;  // (0.375, 0.375)
  uint32_t t;
  asm("add.rn." TCU_X2 " %0, %1, %2;" : "=r"(t) : "r"(x), "r"(kMagic));
  asm("sub.rn." TCU_X2 " %0, %1, %2;" : "=r"(hi) : "r"(t), "r"(kMagic));
  asm("sub.rn." TCU_X2 " %0, %1, %2;" : "=r"(lo) : "r"(x), "r"(hi));
}

// s + e = a + b exactly (Knuth's two-sum).
__device__ __forceinline__ void two_sum(float a, float b, float& s, float& e) {
  const float t  = __fadd_rn(a, b);
  const float bb = __fsub_rn(t, a);
  e = __fadd_rn(__fsub_rn(a, __fsub_rn(t, bb)), __fsub_rn(b, bb));
  s = t;
}

// (h, l) += (bh, bl) for compensated pairs: l also takes what the addition to h rounds off.
__device__ __forceinline__ void pair_add(float& h, float& l, float bh, float bl) {
  float e;
  two_sum(h, bh, h, e);
  l += bl + e;
}

// The multiple of 2^-13 nearest to x, |x| < 512: floats between 1024 and 2048 are 2^-13 apart.
__device__ __forceinline__ float grid13(float x) { return __fsub_rn(__fadd_rn(x, 1536.f), 1536.f); }

// Moves the multiples of 2^-13 that l has added up to over to h; h + l stays what it was (for
// a large l the move is no longer to the grid, but still exact).
__device__ __forceinline__ void pair_renorm(float& h, float& l) {
  const float m = grid13(l);
  float e;
  two_sum(h, m, h, e);
  l = __fsub_rn(l, m) + e;
}

}  // namespace TCU_NS
