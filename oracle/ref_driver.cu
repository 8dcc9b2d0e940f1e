// Launches the REFERENCE's own WMMA kernels, compiled unmodified for sm_100a
// from where they lie (-I<reference>/src; nothing is copied).  TEST
// INFRASTRUCTURE ONLY: used (a) to pin the fp64 oracle against outputs of the
// reference itself, on inputs whose fp16 sums are exact, and (b) to time the
// reference's kernels on the same B200 beside this library.
//
// Only kernels that were checked by reading to stay inside their buffers are
// exposed: segmented_reduction_16n / _256n (src/reduction/kernel.cuh:80-125,
// 301-356) and segmented_prefixsum_16n / _256n (src/prefixsum/kernel.cuh:86-150,
// 441-506).  They have no bounds checks: num_segments must be a multiple of
// the segments one block covers, which the wrappers enforce.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <memory>

#include "init/logger.hpp"
namespace bench { namespace init { namespace logger {
std::shared_ptr<spdlog::logger> console = std::make_shared<spdlog::logger>();
}}}

#include "reduction/kernel.cuh"
#include "prefixsum/kernel.cuh"

namespace {

template <size_t S, int WPB>
int reduce_16n(const half* in, half* out, size_t segs, cudaStream_t st) {
  if (segs % (WPB * 16) != 0) return 1;
  wmma_reduction::compute_wmma_segmented_reduction_16n<S, WPB, WPB * 32>
      <<<(unsigned)(segs / (WPB * 16)), WPB * 32, 0, st>>>(in, out, segs);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

template <size_t S, int WPB>
int reduce_256n(const half* in, half* out, size_t segs, cudaStream_t st) {
  if (segs % WPB != 0) return 1;
  wmma_reduction::compute_wmma_segmented_reduction_256n<half, S, WPB, WPB * 32>
      <<<(unsigned)(segs / WPB), WPB * 32, 0, st>>>(in, out, segs);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

template <size_t S, int WPB>
int scan_16n(const half* in, half* out, size_t segs, cudaStream_t st) {
  if (segs % (WPB * 16) != 0) return 1;
  wmma_prefixsum::compute_wmma_segmented_prefixsum_16n<S, WPB, WPB * 32>
      <<<(unsigned)(segs / (WPB * 16)), WPB * 32, 0, st>>>(in, out, segs);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

template <size_t S, int WPB>
int scan_256n(const half* in, half* out, size_t segs, cudaStream_t st) {
  if (segs % WPB != 0) return 1;
  wmma_prefixsum::compute_wmma_segmented_prefixsum_256n<S, WPB, WPB * 32>
      <<<(unsigned)(segs / WPB), WPB * 32, 0, st>>>(in, out, segs);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace

#define CASE(FN, S, W) if (segment_size == S && warps_per_block == W) return FN<S, W>(in, out, num_segments, st);

// variant: 0 = 16n kernels, 1 = 256n kernels.  Returns 0 ok, 1 unsupported
// shape, 2 launch error.  Outputs are fp16 (the reference accumulates in fp16).
extern "C" int tcu_ref_segmented_reduce(const void* d_in, void* d_out, size_t num_segments,
                                        size_t segment_size, int variant, int warps_per_block,
                                        void* stream) {
  const half* in = static_cast<const half*>(d_in);
  half* out      = static_cast<half*>(d_out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (variant == 0) {
    CASE(reduce_16n, 16, 8) CASE(reduce_16n, 32, 8) CASE(reduce_16n, 64, 1) CASE(reduce_16n, 64, 8)
    CASE(reduce_16n, 256, 1) CASE(reduce_16n, 256, 8) CASE(reduce_16n, 1024, 1)
  } else {
    CASE(reduce_256n, 256, 1) CASE(reduce_256n, 256, 8) CASE(reduce_256n, 1024, 8)
    CASE(reduce_256n, 4096, 8) CASE(reduce_256n, 16384, 8)
  }
  return 1;
}

extern "C" int tcu_ref_segmented_scan(const void* d_in, void* d_out, size_t num_segments,
                                      size_t segment_size, int variant, int warps_per_block,
                                      void* stream) {
  const half* in = static_cast<const half*>(d_in);
  half* out      = static_cast<half*>(d_out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (variant == 0) {
    CASE(scan_16n, 16, 8) CASE(scan_16n, 32, 8) CASE(scan_16n, 256, 1)
  } else {
    CASE(scan_256n, 256, 8) CASE(scan_256n, 256, 4) CASE(scan_256n, 4096, 2) CASE(scan_256n, 4096, 4)
    CASE(scan_256n, 16384, 2)
  }
  return 1;
}
