// C ABI of the library (see include/tcu_scope.h): argument validation, the
// runtime -> compile-time dispatch on segment size that the reference does
// with a switch over template instantiations
// (src/reduction/seg_wmma_16n.cu:137-172), workspace layout and launches.
// Nothing in this file allocates device memory.
#include "../../include/tcu_scope.h"

#include <cuda_runtime.h>

#include <cstring>
#include <new>

#include "common.cuh"
#include "fill_kernels.cuh"
#include "general_kernels.cuh"
#include "reduce_kernels.cuh"
#include "scan_kernels.cuh"
#include "scan_lookback_kernel.cuh"
#include "shuffle_kernels.cuh"
#include "tcgen05_reduce_kernel.cuh"
#include "tcgen05_scan_kernel.cuh"
#if !TCU_BF16
#include "shard_kernels.cuh"
#endif

#if TCU_BF16
// Second compilation of this file (capi_bf16.cu): the same entry points for
// bf16 inputs, under their _bf16 names; 16-bit outputs are bf16 as well.  The
// entry points that are not about an element type exist once, in the fp16 build.
#define tcu_segmented_reduce_f16 tcu_segmented_reduce_bf16
#define tcu_segmented_scan_f16 tcu_segmented_scan_bf16
#define tcu_segmented_exclusive_scan_f16 tcu_segmented_exclusive_scan_bf16
#define tcu_full_exclusive_scan_f16 tcu_full_exclusive_scan_bf16
#define tcu_full_reduce_f16 tcu_full_reduce_bf16
#define tcu_full_scan_f16 tcu_full_scan_bf16
#define tcu_fill_f16 tcu_fill_bf16
#endif

namespace {

using namespace TCU_NS;

constexpr int kMaxDevices    = 64;
constexpr size_t kWsHeader   = 256;   // counters live in the first 256 bytes
constexpr int kMaxLongGrid   = 1024;  // boundary records must fit the idle ring
constexpr int kDynSmemBytes  = kRingBytes + 128;

int g_sm_count[kMaxDevices];

// Scratch of tcu_full_scan_f16_static: tile-status words of the look-back scan
// for up to 2^30 elements (header + a word per tile + the block-level words,
// about 0.8 MiB).  It
// lives in every GPU's memory from the moment the library is loaded there.
// In host code the name below is only a handle for the runtime, never a device
// address: the address is looked up once per device with cudaGetSymbolAddress.
// Workspace of the look-back scan: header | one status word per tile | one per
// block of 32 tiles (+1 per segment for a partial last block; a segment has at
// least 2 tiles, so tiles/2 bounds it).
constexpr size_t scan_long_ws_bytes_for_tiles(size_t tiles) {
  return kWsHeader + tiles * 8 + (tiles / 32 + tiles / 2 + 2) * 8;
}
#if !TCU_BF16
constexpr size_t kStaticScanMaxElems = size_t(1) << 30;
constexpr size_t kStaticScanMaxTiles = kStaticScanMaxElems / kTileElems;
constexpr size_t kStaticScratchBytes = scan_long_ws_bytes_for_tiles(kStaticScanMaxTiles);
static_assert(kStaticScanMaxElems == TCU_STATIC_SCAN_MAX_ELEMENTS &&
                  kStaticScanMaxTiles == TCU_STATIC_SCAN_MAX_TILES &&
                  kStaticScratchBytes == TCU_STATIC_SCAN_SCRATCH_BYTES,
              "include/tcu_scope.h states another size for the built-in scratch");
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScratchBytes];
void* g_static_scan_scratch_addr[kMaxDevices];  // device address, per device; null = not looked up

// One-shot stalls armed by tcu_test_inject() for the next matching call.
unsigned long long g_test_skip_tile   = ~0ull;
unsigned long long g_test_ticket_from = 0;
#endif

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  return (dev >= 0 && dev < kMaxDevices) ? dev : -1;
}

int sm_count() {
  const int dev = current_device();
  if (dev < 0) return 0;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

// log2 of a power-of-two segment size >= 16, folded into the kernel classes;
// kClassGeneral for every other size; -1 for zero.
int segment_class(size_t s) {
  if (s == 0) return -1;
  if (s < 16 || (s & (s - 1)) != 0) return kClassGeneral;
  int l = 0;
  while ((size_t(1) << l) < s) ++l;
  return l <= 14 ? l : kClassLong;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool mul_overflows(size_t a, size_t b, size_t* out) {
  if (a != 0 && b > (SIZE_MAX / 2) / a) return true;  // also keeps 2*a*b representable
  *out = a * b;
  return false;
}

template <typename K>
cudaError_t ensure_smem(K kernel, bool* configured, int bytes) {
  const int dev = current_device();
  if (dev < 0) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return cudaSuccess;
}

// Launch with the programmatic-stream-serialization attribute: the kernel may be
// scheduled while its predecessor in the stream drains (see pdl_prologue()).
template <typename Params>
cudaError_t launch_pdl(void (*kernel)(Params), const Params& p, int grid, int threads,
                       size_t smem, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim          = dim3(grid);
  cfg.blockDim         = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream           = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs    = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

// Same, for the kernels that take the segment size as a second argument.
template <typename Params>
cudaError_t launch_pdl(void (*kernel)(Params, unsigned long long), const Params& p,
                       unsigned long long seg_elems, int grid, int threads, size_t smem,
                       cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim          = dim3(grid);
  cfg.blockDim         = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream           = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs    = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p, seg_elems);
}

// Multiples of 16 up to 2048 elements that are not a power of two: rows of 16 elements, 16 rows
// per warp step, a warp takes chunks of whole segments of about 256 rows.
bool rows_path(size_t segment_size) { return segment_size % 16 == 0 && segment_size <= 2048; }

RowsParams rows_params(const void* d_in, void* d_out, double* d_out_f64, size_t num_segments,
                       size_t segment_size, bool out_f32, bool exclusive) {
  RowsParams r{};
  r.in               = static_cast<const uint8_t*>(d_in);
  r.out              = d_out;
  r.out_f64          = d_out_f64;
  r.num_segments     = num_segments;
  r.rows_per_segment = unsigned(segment_size / 16);
  r.segment_bytes    = unsigned(segment_size * 2);
  // (the reduction takes any multiple of 8 elements and does not use the chunks)
  r.segs_per_chunk   = r.rows_per_segment >= 256 || r.rows_per_segment == 0 ? 1u : 256u / r.rows_per_segment;
  r.out_is_f32       = out_f32;
  r.exclusive        = exclusive;
  return r;
}

int rows_grid(const RowsParams& r, int sms) {
  const size_t chunks = (r.num_segments + r.segs_per_chunk - 1) / r.segs_per_chunk;
  const size_t ctas   = (chunks + kGeneralThreads / 32 - 1) / (kGeneralThreads / 32);
  const size_t cap    = size_t(sms) * 8;
  return int(ctas < cap ? ctas : cap);
}

// one warp per segment, eight warps per CTA, at most eight CTAs per SM
int general_grid(size_t num_segments, int sms) {
  const size_t ctas = (num_segments + kGeneralThreads / 32 - 1) / (kGeneralThreads / 32);
  const size_t cap  = size_t(sms) * 8;
  return int(ctas < cap ? ctas : cap);
}

template <int SC>
cudaError_t launch_reduce(const ReduceParams& p, int grid, cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e = ensure_smem(seg_reduce_kernel<SC, true>, configured, kDynSmemBytes);
  if (e != cudaSuccess) return e;
  return launch_pdl(seg_reduce_kernel<SC, true>, p, grid, kThreads, kDynSmemBytes, st);
}

template <int SC, bool OUT32>
cudaError_t launch_scan(const ScanParams& p, int grid, cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e = ensure_smem(seg_scan_kernel<SC, OUT32>, configured, scan_dyn_smem_bytes(SC, OUT32));
  if (e != cudaSuccess) return e;
  return launch_pdl(seg_scan_kernel<SC, OUT32>, p, grid * scan_ctas_per_sm(SC, OUT32),
                    SliceShape<scan_warps(SC, OUT32)>::kThreads, scan_dyn_smem_bytes(SC, OUT32), st);
}

// cuTensorMapEncodeTiled, looked up once through the runtime (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool looked_up   = false;
  if (!looked_up) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    looked_up = true;
  }
  return fn;
}

// 2-D view of the fp16 input for the swizzled tile loads: rows of 64 halves
// (128 bytes), one box = one tile = 256 rows.  False if the view cannot be made
// (element count not a multiple of 64, or no encoder): callers fall back to
// linear copies.  box_rows: rows per copy (256 = one 32 KiB tile, 128 = one UMMA tile).
bool make_input_tensor_map(CUtensorMap* map, const void* d_in, size_t num_elems,
                           unsigned box_rows = kTileRows) {
  if (num_elems % kSwizzleRowElems != 0) return false;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const cuuint64_t dims[2]    = {kSwizzleRowElems, num_elems / kSwizzleRowElems};
  const cuuint64_t strides[1] = {kSwizzleRowElems * 2};
  const cuuint32_t box[2]     = {kSwizzleRowElems, box_rows};
  const cuuint32_t estr[2]    = {1, 1};
  if (dims[1] >= (cuuint64_t(1) << 32)) return false;
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(d_in), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool OUT32, bool kSwz>
cudaError_t launch_scan_lookback(const ScanParams& p, const CUtensorMap& map, int grid,
                                 cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e =
      ensure_smem(scan_lookback_kernel<OUT32, kSwz>, configured, kLookbackDynSmemBytes);
  if (e != cudaSuccess) return e;
  scan_lookback_kernel<OUT32, kSwz><<<grid, kLookbackThreads, kLookbackDynSmemBytes, st>>>(p, map);
  return cudaGetLastError();
}

template <int LOG2S>
cudaError_t launch_tcgen05_reduce(const ReduceParams& p, const CUtensorMap& map, int grid,
                                  cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e = ensure_smem(tcgen05_reduce_kernel<LOG2S>, configured, kUmmaDynSmemBytes);
  if (e != cudaSuccess) return e;
  tcgen05_reduce_kernel<LOG2S><<<grid, kUmmaThreads, kUmmaDynSmemBytes, st>>>(p, map);
  return cudaGetLastError();
}

// 2-D view of a scan's output for the swizzled bulk stores: rows of 64 outputs; one box = 32
// rows x 128 bytes = what one epilogue warp stages at a time (a whole row of halves, half a
// row of floats).
bool make_output_tensor_map(CUtensorMap* map, void* d_out, size_t num_elems, bool out32) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc || num_elems % kSwizzleRowElems != 0) return false;
  const cuuint64_t rows = num_elems / kSwizzleRowElems;
  if (rows >= (cuuint64_t(1) << 31)) return false;
  const cuuint32_t estr[3] = {1, 1, 1};
  if (out32) {
    // A row of 64 floats is two swizzle spans of 128 bytes: the view {32 floats, 2 halves, rows}
    // lets one box hold whole rows (32 rows, 8 KiB contiguous in global memory).
    const cuuint64_t dims[3]    = {32, 2, rows};
    const cuuint64_t strides[2] = {128, 256};
    const cuuint32_t box[3]     = {32, 2, 32};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, d_out, dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const cuuint64_t dims[2]    = {kSwizzleRowElems, rows};
  const cuuint64_t strides[1] = {cuuint64_t(kSwizzleRowElems) * 2};
  const cuuint32_t box[2]     = {64u, 32u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, d_out, dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int LOG2S, bool OUT32, bool kExcl = false>
cudaError_t launch_tcgen05_scan(const ScanParams& p, const CUtensorMap& omap, int grid, cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e = ensure_smem(tcgen05_scan_kernel<LOG2S, OUT32, kExcl>, configured, kUscanDynSmemBytes);
  if (e != cudaSuccess) return e;
  tcgen05_scan_kernel<LOG2S, OUT32, kExcl><<<grid, kUscanThreads, kUscanDynSmemBytes, st>>>(p, omap);
  return cudaGetLastError();
}

template <int SC>
cudaError_t launch_shuffle_reduce(const ReduceParams& p, int grid, cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e = ensure_smem(seg_reduce_kernel<SC, false>, configured, kDynSmemBytes);
  if (e != cudaSuccess) return e;
  seg_reduce_kernel<SC, false><<<grid, kThreads, kDynSmemBytes, st>>>(p);
  return cudaGetLastError();
}

template <int SC, bool OUT32>
cudaError_t launch_shuffle_scan(const ScanParams& p, int grid, cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e = ensure_smem(shuffle_scan_kernel<SC, OUT32>, configured, kDynSmemBytes);
  if (e != cudaSuccess) return e;
  shuffle_scan_kernel<SC, OUT32><<<grid, kThreads, kDynSmemBytes, st>>>(p);
  return cudaGetLastError();
}

#define TCU_FOR_SHORT_CLASSES(X) X(4) X(5) X(6) X(7) X(8) X(9) X(10) X(11) X(12) X(13) X(14)

size_t reduce_long_ws_bytes() { return kWsHeader + size_t(2) * kMaxLongGrid * 16; }

size_t scan_long_tiles(size_t num_elements) { return (num_elements + kTileElems - 1) / kTileElems; }

size_t scan_long_ws_bytes(size_t num_elements) {
  return scan_long_ws_bytes_for_tiles(scan_long_tiles(num_elements));
}

int reduce_impl(const void* d_in, void* d_out, double* d_out_f64, int out_type,
                size_t num_segments, size_t segment_size, int sc, int algo, void* ws,
                size_t ws_bytes, cudaStream_t st) {
  if (out_type != TCU_OUT_F16 && out_type != TCU_OUT_F32) return TCU_ERR_UNSUPPORTED;
  if (algo != TCU_ALGO_AUTO && algo != TCU_ALGO_MMA && algo != TCU_ALGO_SHUFFLE &&
      algo != TCU_ALGO_TCGEN05)
    return TCU_ERR_UNSUPPORTED;
  if (sc == kClassGeneral && algo != TCU_ALGO_AUTO && algo != TCU_ALGO_MMA) return TCU_ERR_UNSUPPORTED;
  size_t n = 0;
  if (mul_overflows(num_segments, segment_size, &n)) return TCU_ERR_INVALID_ARG;
  // the tcgen05 variant covers 16 ... 2048-element segments of arrays it can view as 64-wide rows
  if (algo == TCU_ALGO_TCGEN05 && (sc < 4 || sc > 11 || n % kSwizzleRowElems != 0))
    return TCU_ERR_UNSUPPORTED;
  if (n == 0) return TCU_OK;
  // short classes store vectors of outputs, the long and the general class single values
  const uintptr_t out_mask = sc >= kClassLong ? 3u : 15u;
  if (!d_in || !d_out || !aligned16(d_in) || (reinterpret_cast<uintptr_t>(d_out) & out_mask) != 0)
    return TCU_ERR_INVALID_ARG;
  if (d_out_f64 && (reinterpret_cast<uintptr_t>(d_out_f64) & 7u) != 0) return TCU_ERR_INVALID_ARG;
  const int sms = sm_count();
  if (sms <= 0) return TCU_ERR_CUDA;

  ReduceParams p{};
  p.in           = static_cast<const uint8_t*>(d_in);
  p.out          = d_out;
  p.num_elems    = n;
  p.num_segments = num_segments;
  p.out_is_f32   = out_type == TCU_OUT_F32;
  p.out_f64      = d_out_f64;
  p.test_skip_tile = ~0ull;
#if !TCU_BF16
  p.test_skip_tile = g_test_skip_tile;  // one-shot stall armed by a test, see tcu_test_inject
  g_test_skip_tile = ~0ull;
#endif
  const size_t tiles = (n + kTileElems - 1) / kTileElems;
  // work units: tiles, or, for segments of 4096 ... 16384 elements, groups of eight segments
  const size_t units = sc >= 12 && sc <= 14 ? (num_segments + 7) / 8 : tiles;
  int grid           = units < size_t(sms) ? int(units) : sms;
  if (grid < 1) grid = 1;

  cudaError_t e = cudaSuccess;
  // Up to 2048 elements a warp takes 16 segments at a time: multiples of 8, whose rows start on
  // 16-byte boundaries, and -- up to 255 elements, where it measured faster than one warp per
  // segment (0.41 against 0.06 of the copy bandwidth at 50 elements, 0.31 against 0.12 at 100, a
  // tie at 255) -- any other size.
  if (sc == kClassGeneral && segment_size <= 2048 && (segment_size % 8 == 0 || segment_size <= 255)) {
    const RowsParams r = rows_params(d_in, d_out, d_out_f64, num_segments, segment_size,
                                     out_type == TCU_OUT_F32, false);
    const size_t ctas = ((num_segments + 15) / 16 + kGeneralThreads / 32 - 1) / (kGeneralThreads / 32);
    const size_t cap  = size_t(sms) * 8;
    const int rgrid   = int(ctas < cap ? ctas : cap);
    if (segment_size % 8 == 0) {  // rows start on 16-byte boundaries
      const size_t steps = (segment_size * 2 + 63) / 64;  // 64-byte steps that cover a segment
      e = steps <= 1   ? launch_pdl(seg_rowsum_kernel<1>, r, rgrid, kGeneralThreads, 0, st)
          : steps == 2 ? launch_pdl(seg_rowsum_kernel<2>, r, rgrid, kGeneralThreads, 0, st)
          : steps == 3 ? launch_pdl(seg_rowsum_kernel<3>, r, rgrid, kGeneralThreads, 0, st)
                       : launch_pdl(seg_rowsum_kernel<4>, r, rgrid, kGeneralThreads, 0, st);
    } else {  // any size: aligned loads around every piece, foreign halves cleared
      const size_t steps = (segment_size * 2 + 14 + 63) / 64;
      e = steps <= 1   ? launch_pdl(seg_rowsum_kernel<1, true>, r, rgrid, kGeneralThreads, 0, st)
          : steps == 2 ? launch_pdl(seg_rowsum_kernel<2, true>, r, rgrid, kGeneralThreads, 0, st)
          : steps == 3 ? launch_pdl(seg_rowsum_kernel<3, true>, r, rgrid, kGeneralThreads, 0, st)
                       : launch_pdl(seg_rowsum_kernel<4, true>, r, rgrid, kGeneralThreads, 0, st);
    }
    return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
  }
  if (sc == kClassGeneral) {
    // one warp per segment, or -- when that leaves SMs idle and the segments are long -- one CTA
    const bool vec   = segment_size % 8 == 0;
    const bool block = segment_size >= 8192 && num_segments < size_t(sms) * 32;
    if (block) {
      const size_t cap = size_t(sms) * 8;
      e = launch_pdl(vec ? seg_reduce_general_kernel<true, true> : seg_reduce_general_kernel<false, true>, p,
                     (unsigned long long)segment_size, int(num_segments < cap ? num_segments : cap),
                     kGeneralThreads, 0, st);
    } else {
      e = launch_pdl(vec ? seg_reduce_general_kernel<true> : seg_reduce_general_kernel<false>, p,
                     (unsigned long long)segment_size, general_grid(num_segments, sms), kGeneralThreads,
                     0, st);
    }
    return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
  }
  if (algo == TCU_ALGO_TCGEN05) {
    CUtensorMap map;
    std::memset(&map, 0, sizeof(map));
    if (!make_input_tensor_map(&map, d_in, n, kUmmaPerStage * kUmmaRows)) return TCU_ERR_CUDA;
    const size_t utiles = (n + kUmmaPerStage * kUmmaTileElems - 1) / (kUmmaPerStage * kUmmaTileElems);
    const int ugrid     = utiles < size_t(sms) ? int(utiles) : sms;
    switch (sc) {
#define X(C) case C: e = launch_tcgen05_reduce<C>(p, map, ugrid, st); break;
      X(4) X(5) X(6) X(7) X(8) X(9) X(10) X(11)
#undef X
      default: return TCU_ERR_UNSUPPORTED;
    }
    return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
  }
  p.spread_slices = sc >= 12 && sc <= 14 ? 1u << (sc - 11) : 0u;
  if (sc == kClassLong) {
    if (!ws || ws_bytes < reduce_long_ws_bytes() || !aligned16(ws)) return TCU_ERR_WORKSPACE;
    // Many long segments: eight segments per work unit, one warp per segment, like the 4096 ...
    // 16384-element classes.  Taken when the units fill the SMs evenly -- one round on 85 % of the
    // SMs or more, or several rounds with the last one at least 95 % full: measured at 2^28
    // elements, 2^15 / 2^16 / 2^18 elements per segment (1024 / 512 / 128 units), 0.94 / 0.86 /
    // 0.95 of the copy bandwidth against 0.88 / 0.91 / 0.92 for the kernel below.  The workspace
    // is then left untouched.
    if (num_segments > 1 && segment_size / kSliceElems <= (size_t(1) << 20)) {
      const size_t lunits = (num_segments + 7) / 8;
      const size_t rounds = (lunits + size_t(sms) - 1) / size_t(sms);
      if (lunits * 100 >= rounds * size_t(sms) * (rounds == 1 ? 85 : 95)) {
        p.spread_slices = unsigned(segment_size / kSliceElems);
        const int sgrid = lunits < size_t(sms) ? int(lunits) : sms;
        e = (algo == TCU_ALGO_SHUFFLE) ? launch_shuffle_reduce<14>(p, sgrid, st) : launch_reduce<14>(p, sgrid, st);
        return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
      }
    }
    if (grid > kMaxLongGrid) grid = kMaxLongGrid;
    uint8_t* w          = static_cast<uint8_t*>(ws);
    p.done_counter      = reinterpret_cast<unsigned int*>(w);
    p.bound_val         = reinterpret_cast<double*>(w + kWsHeader);
    p.bound_seg         = reinterpret_cast<long long*>(w + kWsHeader + size_t(2) * kMaxLongGrid * 8);
    // one segment (the full reduction): any multiple of 16 elements, all tiles are segment 0
    p.tiles_per_segment = num_segments == 1 ? tiles : segment_size / kTileElems;
    if (cudaMemsetAsync(w, 0, kWsHeader, st) != cudaSuccess) return TCU_ERR_CUDA;
    e = (algo == TCU_ALGO_SHUFFLE) ? launch_shuffle_reduce<kClassLong>(p, grid, st)
                                   : launch_reduce<kClassLong>(p, grid, st);
  } else if (algo == TCU_ALGO_SHUFFLE) {
    switch (sc) {
#define X(C) case C: e = launch_shuffle_reduce<C>(p, grid, st); break;
      TCU_FOR_SHORT_CLASSES(X)
#undef X
      default: return TCU_ERR_UNSUPPORTED;
    }
  } else {
    switch (sc) {
#define X(C) case C: e = launch_reduce<C>(p, grid, st); break;
      TCU_FOR_SHORT_CLASSES(X)
#undef X
      default: return TCU_ERR_UNSUPPORTED;
    }
  }
  return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
}

int scan_impl(const void* d_in, void* d_out, int out_type, size_t num_segments,
              size_t segment_size, int sc, const double* shard_totals, int shard_index, int algo,
              void* ws, size_t ws_bytes, cudaStream_t st, bool exclusive = false) {
  if (out_type != TCU_OUT_F16 && out_type != TCU_OUT_F32) return TCU_ERR_UNSUPPORTED;
  if (algo != TCU_ALGO_AUTO && algo != TCU_ALGO_MMA && algo != TCU_ALGO_SHUFFLE &&
      algo != TCU_ALGO_TCGEN05)
    return TCU_ERR_UNSUPPORTED;
  if (sc == kClassGeneral && algo != TCU_ALGO_AUTO && algo != TCU_ALGO_MMA) return TCU_ERR_UNSUPPORTED;
  size_t n = 0;
  if (mul_overflows(num_segments, segment_size, &n)) return TCU_ERR_INVALID_ARG;
  // the tcgen05 variant: inclusive scans of 16 ... 16384-element segments of arrays it can view as
  // 64-wide rows; with 16-bit outputs also whole segments of 2^15 ... 2^20 elements
  int lg = 0;  // log2 of the segment size (powers of two)
  while ((size_t(1) << lg) < segment_size) ++lg;
  const bool spread_long = sc == kClassLong && num_segments > 1 && lg <= kUscanMaxLog2 &&
                           out_type == TCU_OUT_F16 && shard_index == 0;
  if (algo == TCU_ALGO_TCGEN05 &&
      (sc < 4 || (sc > 14 && !spread_long) || n % kSwizzleRowElems != 0 || exclusive))
    return TCU_ERR_UNSUPPORTED;
  if (n == 0) return TCU_OK;
  if (!d_in || !d_out || !aligned16(d_in) || !aligned16(d_out)) return TCU_ERR_INVALID_ARG;
  if (shard_index < 0 || (shard_index > 0 && !shard_totals)) return TCU_ERR_INVALID_ARG;
  const int sms = sm_count();
  if (sms <= 0) return TCU_ERR_CUDA;

  ScanParams p{};
  p.in         = static_cast<const uint8_t*>(d_in);
  p.out        = d_out;
  p.num_elems  = n;
  p.out_is_f32 = out_type == TCU_OUT_F32;
  p.exclusive  = exclusive ? 1 : 0;
  if (exclusive && algo == TCU_ALGO_SHUFFLE) return TCU_ERR_UNSUPPORTED;  // ablation: inclusive only
  const size_t tiles = (n + kTileElems - 1) / kTileElems;
  const int grid     = tiles < size_t(sms) ? int(tiles) : sms;
  const bool f32     = out_type == TCU_OUT_F32;

  cudaError_t e = cudaSuccess;
  if (sc == kClassGeneral && rows_path(segment_size)) {
    const RowsParams r = rows_params(d_in, d_out, nullptr, num_segments, segment_size, f32, exclusive);
    e = f32 ? launch_pdl(seg_rows_kernel<true>, r, rows_grid(r, sms), kGeneralThreads, 0, st)
            : launch_pdl(seg_rows_kernel<false>, r, rows_grid(r, sms), kGeneralThreads, 0, st);
    return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
  }
  if (sc == kClassGeneral) {
    const int ggrid = general_grid(num_segments, sms);
    const bool vec  = segment_size % 4 == 0;
    const bool deep = segment_size >= 32768;  // few, long segments: three steps of loads in flight
    void (*kernel)(ScanParams, unsigned long long) =
        deep ? (f32 ? (vec ? seg_scan_general_kernel<true, true, 3> : seg_scan_general_kernel<true, false, 3>)
                    : (vec ? seg_scan_general_kernel<false, true, 3> : seg_scan_general_kernel<false, false, 3>))
             : (f32 ? (vec ? seg_scan_general_kernel<true, true> : seg_scan_general_kernel<true, false>)
                    : (vec ? seg_scan_general_kernel<false, true> : seg_scan_general_kernel<false, false>));
    e = launch_pdl(kernel, p, (unsigned long long)segment_size, ggrid, kGeneralThreads, 0, st);
    return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
  }
  // TCU_ALGO_AUTO takes the tcgen05 kernel where it measured faster than the mma.sync one:
  // 16-bit outputs of 16- and 256 ... 16384-element segments (0.96 ... 1.00 of the copy bandwidth
  // at 2^28 elements against 0.92 / 0.94 ... 0.76) and fp32 outputs of 16-element segments (0.94
  // against 0.89).  Its set-up costs 2-3 us more, so it takes over from 2^25 elements on for
  // 16-bit outputs of segments of 4096 and more (27.2 against 29.4 us at 4096) and from 2^26 on
  // for the others (16-bit: 45.8 against 47.5 us at 16 elements, 45.6 against 46.9 at 256;
  // fp32: 68.6 against 72.6 us; at 2^25 the mma.sync kernels win 20.7 ... 25.6 against 27 us).
  const bool umma_class = f32 ? sc == 4 : (sc == 4 || (sc >= 8 && sc <= 14));
  const size_t umma_from = (!f32 && sc >= 12) ? size_t(1) << 25 : size_t(1) << 26;
  // (exclusive scans: the 16-bit classes only)
  const bool umma_auto = algo == TCU_ALGO_AUTO && !(exclusive && f32) && n % kSwizzleRowElems == 0 &&
                         n >= umma_from && umma_class;
  if ((algo == TCU_ALGO_TCGEN05 && sc <= 14) || umma_auto) {
    CUtensorMap omap;
    std::memset(&omap, 0, sizeof(omap));
    const bool maps = make_output_tensor_map(&omap, d_out, n, f32);
    if (!maps && !umma_auto) return TCU_ERR_CUDA;
    if (maps) {
      // work units: single tiles, or pairs of groups of four segments of more than 2048 elements
      const size_t unit_elems = segment_size > 2048 ? 8 * segment_size : size_t(kUmmaTileElems);
      const size_t units      = (n + unit_elems - 1) / unit_elems;
      const int ugrid         = units < size_t(sms) ? int(units) : sms;
      if (exclusive) {
        switch (sc) {
#define X(C) case C: e = launch_tcgen05_scan<C, false, true>(p, omap, ugrid, st); break;
          X(4) X(8) X(9) X(10) X(11) X(12) X(13) X(14)
#undef X
          default: return TCU_ERR_UNSUPPORTED;
        }
        return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
      }
      switch (sc) {
#define X(C)                                                                              \
  case C:                                                                                 \
    e = f32 ? launch_tcgen05_scan<C, true>(p, omap, ugrid, st)                            \
            : launch_tcgen05_scan<C, false>(p, omap, ugrid, st);                          \
    break;
        X(4) X(5) X(6) X(7) X(8) X(9) X(10) X(11) X(12) X(13) X(14)
#undef X
        default: return TCU_ERR_UNSUPPORTED;
      }
      return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
    }
  }
  if (sc == kClassLong) {
    const size_t need = scan_long_ws_bytes(n);
    if (!ws || ws_bytes < need || !aligned16(ws)) return TCU_ERR_WORKSPACE;
    // 16-bit outputs of whole segments of up to 2^20 elements: the tcgen05 kernel spreads a segment
    // over tiles like the 4096 ... 16384-element ones and needs no look-back (measured 0.84 ...
    // 0.97 of the copy bandwidth at 2^28 elements where the look-back kernel reaches 0.67 ... 0.72;
    // the workspace is then left untouched).  Work units are eight segments: taken only when they
    // fill the SMs evenly enough.
    if (spread_long && !exclusive && n % kSwizzleRowElems == 0 &&
        (algo == TCU_ALGO_TCGEN05 || algo == TCU_ALGO_AUTO)) {
      const size_t units  = (num_segments + 7) / 8;
      const size_t rounds = (units + size_t(sms) - 1) / size_t(sms);
      const bool even     = units * 100 >= rounds * size_t(sms) * 85;
      CUtensorMap omap;
      std::memset(&omap, 0, sizeof(omap));
      if ((algo == TCU_ALGO_TCGEN05 || (even && n >= (size_t(1) << 26))) &&
          make_output_tensor_map(&omap, d_out, n, false)) {
        const int ugrid = units < size_t(sms) ? int(units) : sms;
        switch (lg) {
#define X(C) case C: e = launch_tcgen05_scan<C, false>(p, omap, ugrid, st); break;
          X(15) X(16) X(17) X(18) X(19) X(20)
#undef X
          default: return TCU_ERR_UNSUPPORTED;
        }
        return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
      }
      if (algo == TCU_ALGO_TCGEN05) return TCU_ERR_CUDA;
    }
    uint8_t* w          = static_cast<uint8_t*>(ws);
    p.ticket            = reinterpret_cast<unsigned int*>(w);
    p.tile_status       = reinterpret_cast<unsigned long long*>(w + kWsHeader);
    p.block_status      = p.tile_status + tiles;
    p.tiles_per_segment = num_segments == 1 ? tiles : segment_size / kTileElems;
    p.shard_totals      = shard_totals;
    p.shard_index       = shard_index;
    if (cudaMemsetAsync(w, 0, need, st) != cudaSuccess) return TCU_ERR_CUDA;
#if !TCU_BF16
    if (g_test_ticket_from != 0) {  // one-shot stall armed by a test: tiles below it are never scanned
      if (cudaMemsetAsync(w, int(g_test_ticket_from & 0xffu), 1, st) != cudaSuccess) return TCU_ERR_CUDA;
      g_test_ticket_from = 0;
    }
#endif
    const size_t want = size_t(sms) * kLookbackCtasPerSm;
    const int lgrid   = tiles < want ? int(tiles) : int(want);
    if (algo == TCU_ALGO_SHUFFLE) return TCU_ERR_UNSUPPORTED;
    CUtensorMap map;
    std::memset(&map, 0, sizeof(map));
    if (make_input_tensor_map(&map, d_in, n))
      e = f32 ? launch_scan_lookback<true, true>(p, map, lgrid, st)
              : launch_scan_lookback<false, true>(p, map, lgrid, st);
    else
      e = f32 ? launch_scan_lookback<true, false>(p, map, lgrid, st)
              : launch_scan_lookback<false, false>(p, map, lgrid, st);
  } else if (algo == TCU_ALGO_SHUFFLE) {
    switch (sc) {
#define X(C)                                                                         \
  case C:                                                                            \
    e = f32 ? launch_shuffle_scan<C, true>(p, grid, st) : launch_shuffle_scan<C, false>(p, grid, st); \
    break;
      TCU_FOR_SHORT_CLASSES(X)
#undef X
      default: return TCU_ERR_UNSUPPORTED;
    }
  } else {
    switch (sc) {
#define X(C)                                                                       \
  case C:                                                                          \
    e = f32 ? launch_scan<C, true>(p, grid, st) : launch_scan<C, false>(p, grid, st); \
    break;
      TCU_FOR_SHORT_CLASSES(X)
#undef X
      default: return TCU_ERR_UNSUPPORTED;
    }
  }
  return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
}

}  // namespace

extern "C" {

int tcu_segmented_reduce_f16(const void* d_in, void* d_out, int out_type, size_t num_segments,
                             size_t segment_size, int algo, void* d_workspace,
                             size_t workspace_bytes, void* stream) {
  const int sc = segment_class(segment_size);
  if (sc < 0) return TCU_ERR_UNSUPPORTED;
  return reduce_impl(d_in, d_out, nullptr, out_type, num_segments, segment_size, sc, algo,
                     d_workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int tcu_segmented_scan_f16(const void* d_in, void* d_out, int out_type, size_t num_segments,
                           size_t segment_size, int algo, void* d_workspace,
                           size_t workspace_bytes, void* stream) {
  const int sc = segment_class(segment_size);
  if (sc < 0) return TCU_ERR_UNSUPPORTED;
  return scan_impl(d_in, d_out, out_type, num_segments, segment_size, sc, nullptr, 0, algo,
                   d_workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int tcu_segmented_exclusive_scan_f16(const void* d_in, void* d_out, int out_type,
                                     size_t num_segments, size_t segment_size, void* d_workspace,
                                     size_t workspace_bytes, void* stream) {
  const int sc = segment_class(segment_size);
  if (sc < 0) return TCU_ERR_UNSUPPORTED;
  return scan_impl(d_in, d_out, out_type, num_segments, segment_size, sc, nullptr, 0, TCU_ALGO_AUTO,
                   d_workspace, workspace_bytes, static_cast<cudaStream_t>(stream), true);
}

int tcu_full_exclusive_scan_f16(const void* d_in, void* d_out, int out_type, size_t num_elements,
                                void* d_workspace, size_t workspace_bytes, void* stream) {
  if (num_elements % 16 != 0) return TCU_ERR_INVALID_ARG;
  return scan_impl(d_in, d_out, out_type, 1, num_elements, kClassLong, nullptr, 0, TCU_ALGO_MMA,
                   d_workspace, workspace_bytes, static_cast<cudaStream_t>(stream), true);
}

// The full operations are the long class with a single segment covering every
// tile, so any multiple of 16 elements works, not just powers of two.
int tcu_full_reduce_f16(const void* d_in, float* d_out, double* d_out_f64, size_t num_elements,
                        int algo, void* d_workspace, size_t workspace_bytes, void* stream) {
  // an empty sum has no element count to be a multiple of; reject it with the rest
  if (num_elements == 0 || num_elements % 16 != 0) return TCU_ERR_INVALID_ARG;
  return reduce_impl(d_in, d_out, d_out_f64, TCU_OUT_F32, 1, num_elements, kClassLong, algo,
                     d_workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int tcu_full_scan_f16(const void* d_in, void* d_out, int out_type, size_t num_elements,
                      const double* d_shard_totals, int shard_index, int algo,
                      void* d_workspace, size_t workspace_bytes, void* stream) {
  if (num_elements % 16 != 0) return TCU_ERR_INVALID_ARG;
  return scan_impl(d_in, d_out, out_type, 1, num_elements, kClassLong, d_shard_totals,
                   shard_index, algo, d_workspace, workspace_bytes,
                   static_cast<cudaStream_t>(stream));
}

#if !TCU_BF16
int tcu_full_scan_f16_static(const void* d_in, void* d_out, int out_type, size_t num_elements,
                             const double* d_shard_totals, int shard_index, int algo,
                             void* stream) {
  if (num_elements % 16 != 0) return TCU_ERR_INVALID_ARG;
  if (num_elements > kStaticScanMaxElems) return TCU_ERR_TOO_LARGE;
  const int dev = current_device();
  if (dev < 0) return TCU_ERR_CUDA;
  if (g_static_scan_scratch_addr[dev] == nullptr) {
    // one-time set-up for this device (it is the current one): resolve the
    // array's device address; a kernel handed the host-side name would fault
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_static_scan_scratch) != cudaSuccess || addr == nullptr)
      return TCU_ERR_CUDA;
    g_static_scan_scratch_addr[dev] = addr;
  }
  // scan_impl clears the part of the scratch this call uses (cudaMemsetAsync on
  // the stream) before the kernel; it allocates nothing.
  return scan_impl(d_in, d_out, out_type, 1, num_elements, kClassLong, d_shard_totals, shard_index,
                   algo, g_static_scan_scratch_addr[dev], kStaticScratchBytes,
                   static_cast<cudaStream_t>(stream));
}

size_t tcu_workspace_bytes(int op, size_t num_elements, size_t segment_size) {
  switch (op) {
    case TCU_OP_SEGMENTED_REDUCE:
      return segment_class(segment_size) == kClassLong ? reduce_long_ws_bytes() : 0;
    case TCU_OP_FULL_REDUCE: return reduce_long_ws_bytes();
    case TCU_OP_SEGMENTED_SCAN:
      return segment_class(segment_size) == kClassLong ? scan_long_ws_bytes(num_elements) : 0;
    case TCU_OP_FULL_SCAN: return scan_long_ws_bytes(num_elements);
    default: return 0;
  }
}

#endif  // !TCU_BF16

int tcu_fill_f16(void* d_out, size_t n, uint64_t seed, uint64_t first_index, int dist,
                 void* stream) {
  if (n == 0) return TCU_OK;
  if (!d_out || !aligned16(d_out) || n % 8 != 0) return TCU_ERR_INVALID_ARG;
  if (dist < TCU_DIST_UNIFORM_PM1 || dist > TCU_DIST_CONST_0P001) return TCU_ERR_UNSUPPORTED;
  const int sms = sm_count();
  if (sms <= 0) return TCU_ERR_CUDA;
  const size_t groups = n / 8;
  const size_t want   = (groups + 255) / 256;
  const int grid      = want < size_t(sms) * 16 ? int(want) : sms * 16;
  fill_f16_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(d_out), groups, seed, first_index, dist);
  return cudaGetLastError() == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
}

// Each of the two builds has its own device error word; this reads (and clears)
// the one of the build it is compiled in.  Not part of the public header.
#if TCU_BF16
#define tcu_error_word_of_this_build tcu_error_word_bf16_build
#else
#define tcu_error_word_of_this_build tcu_error_word_f16_build
#endif
int tcu_error_word_f16_build(unsigned int* bits, int clear);
int tcu_error_word_bf16_build(unsigned int* bits, int clear);

int tcu_error_word_of_this_build(unsigned int* bits, int clear) {
  unsigned int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return TCU_ERR_CUDA;
  if (cudaMemcpyFromSymbol(&v, g_error_word, sizeof(v)) != cudaSuccess) return TCU_ERR_CUDA;
  if (clear && v) {
    const unsigned int z = 0;
    if (cudaMemcpyToSymbol(g_error_word, &z, sizeof(z)) != cudaSuccess) return TCU_ERR_CUDA;
  }
  *bits = v;
  return TCU_OK;
}

// Likewise for the wait limits of the build this is compiled in (0 = default).
#if TCU_BF16
#define tcu_wait_limits_of_this_build tcu_wait_limits_bf16_build
#else
#define tcu_wait_limits_of_this_build tcu_wait_limits_f16_build
#endif
int tcu_wait_limits_f16_build(const unsigned int* four);
int tcu_wait_limits_bf16_build(const unsigned int* four);

int tcu_wait_limits_of_this_build(const unsigned int* four) {
  WaitLimits w = kDefaultWaitLimits;
  if (four[0]) w.barrier = four[0];
  if (four[1]) w.status = four[1];
  if (four[2]) w.flag = four[2];
  if (four[3]) w.peer = four[3];
  if (cudaDeviceSynchronize() != cudaSuccess) return TCU_ERR_CUDA;
  return cudaMemcpyToSymbol(g_wait_limits, &w, sizeof(w)) == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
}

#if !TCU_BF16
int tcu_device_error(unsigned int* bits, int clear) {
  unsigned int a = 0, b = 0;
  if (tcu_error_word_f16_build(&a, clear) != TCU_OK) return TCU_ERR_CUDA;
  if (tcu_error_word_bf16_build(&b, clear) != TCU_OK) return TCU_ERR_CUDA;
  if (bits) *bits = a | b;
  return (a | b) ? TCU_ERR_TIMEOUT : TCU_OK;
}

int tcu_test_set_wait_limits(unsigned barrier_attempts, unsigned status_polls, unsigned flag_polls,
                             unsigned peer_polls) {
  const unsigned int four[4] = {barrier_attempts, status_polls, flag_polls, peer_polls};
  if (tcu_wait_limits_f16_build(four) != TCU_OK) return TCU_ERR_CUDA;
  return tcu_wait_limits_bf16_build(four);
}

int tcu_test_inject(int what, unsigned long long arg) {
  switch (what) {
    case TCU_TEST_NONE:
      g_test_skip_tile   = ~0ull;
      g_test_ticket_from = 0;
      return TCU_OK;
    case TCU_TEST_SKIP_TILE_LOAD: g_test_skip_tile = arg; return TCU_OK;
    case TCU_TEST_LOOKBACK_TICKET:
      if (arg == 0 || arg > 255) return TCU_ERR_INVALID_ARG;
      g_test_ticket_from = arg;
      return TCU_OK;
    default: return TCU_ERR_UNSUPPORTED;
  }
}

int tcu_tile_elements(void) { return kTileElems; }

int tcu_num_sms(void) { return sm_count(); }

const char* tcu_status_string(int status) {
  switch (status) {
    case TCU_OK: return "ok";
    case TCU_ERR_INVALID_ARG: return "invalid argument (null or misaligned pointer, bad size)";
    case TCU_ERR_UNSUPPORTED: return "unsupported segment size, output type or algorithm";
    case TCU_ERR_CUDA: return "CUDA runtime error";
    case TCU_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case TCU_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case TCU_ERR_TOO_LARGE: return "input larger than the built-in scratch of the _static entry point";
    default: return "unknown status";
  }
}

#endif  // !TCU_BF16

}  // extern "C"

#if !TCU_BF16
#include "host_pipeline.inl"
#include "mgpu.inl"
#endif
