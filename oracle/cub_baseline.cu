// Library baselines for the same operations: CUB (the CCCL that ships with the
// CUDA toolkit) device-wide primitives, the comparison set of the reference
// (cub::DeviceReduce::Sum, src/reduction/cub.cu:46; DeviceSegmentedReduce::Sum,
// src/reduction/seg_cub_device.cu:61; DeviceScan::InclusiveSum,
// src/prefixsum/cub.cu:44) and Thrust (thrust::reduce, src/reduction/thrust.cu;
// thrust::reduce_by_key, src/reduction/seg_thrust.cu:50; thrust::inclusive_scan,
// src/prefixsum/thrust.cu; thrust::inclusive_scan_by_key,
// src/prefixsum/seg_thrust.cu:46).  TEST / BASELINE INFRASTRUCTURE ONLY: never
// linked into the library.  Inputs are fp16 and are widened to fp32 on the fly,
// so the library calls accumulate in fp32 like the kernels they are compared with.
#include <cub/cub.cuh>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <thrust/execution_policy.h>
#include <thrust/iterator/discard_iterator.h>
#include <thrust/reduce.h>
#include <thrust/scan.h>

namespace {

struct HalfToFloat {
  __host__ __device__ float operator()(const __half& h) const { return __half2float(h); }
};
using InIt = cub::TransformInputIterator<float, HalfToFloat, const __half*>;

struct SegmentBegin {  // offset of segment i
  long long s;
  __host__ __device__ long long operator()(long long i) const { return i * s; }
};
using OffsetIt = cub::TransformInputIterator<long long, SegmentBegin, cub::CountingInputIterator<long long>>;

struct SegmentOf {  // key of element i
  long long s;
  __host__ __device__ long long operator()(long long i) const { return i / s; }
};
using KeyIt = cub::TransformInputIterator<long long, SegmentOf, cub::CountingInputIterator<long long>>;

}  // namespace

// op: 0 full reduce -> float[1]; 1 segmented reduce -> float[segs]; 2 full inclusive scan ->
// float[n]; 3 segmented inclusive scan (by key) -> float[n]; 4 the same -> half[n].
// With d_temp == nullptr only *temp_bytes is set (CUB's two-phase convention).
extern "C" int tcu_cub_run(int op, const void* d_in, void* d_out, size_t n, size_t segment_size,
                           void* d_temp, size_t* temp_bytes, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  InIt in(static_cast<const __half*>(d_in), HalfToFloat());
  cudaError_t e = cudaErrorInvalidValue;
  switch (op) {
    case 0:
      e = cub::DeviceReduce::Sum(d_temp, *temp_bytes, in, static_cast<float*>(d_out), (long long)n, st);
      break;
    case 1: {
      OffsetIt off(cub::CountingInputIterator<long long>(0), SegmentBegin{(long long)segment_size});
      e = cub::DeviceSegmentedReduce::Sum(d_temp, *temp_bytes, in, static_cast<float*>(d_out),
                                          (int)(n / segment_size), off, off + 1, st);
      break;
    }
    case 2:
      e = cub::DeviceScan::InclusiveSum(d_temp, *temp_bytes, in, static_cast<float*>(d_out), (long long)n, st);
      break;
    case 3: {
      KeyIt keys(cub::CountingInputIterator<long long>(0), SegmentOf{(long long)segment_size});
      e = cub::DeviceScan::InclusiveSumByKey(d_temp, *temp_bytes, keys, in, static_cast<float*>(d_out),
                                             (long long)n, cub::Equality(), st);
      break;
    }
    case 4: {
      KeyIt keys(cub::CountingInputIterator<long long>(0), SegmentOf{(long long)segment_size});
      e = cub::DeviceScan::InclusiveSumByKey(d_temp, *temp_bytes, keys, in, static_cast<__half*>(d_out),
                                             (long long)n, cub::Equality(), st);
      break;
    }
    default: break;
  }
  return e == cudaSuccess ? 0 : (int)e;
}

// The Thrust forms of the same operations (Thrust allocates its own temporary storage per
// call, as it does in the reference's drivers).  op: 0 thrust::reduce -> float[1] (the value
// comes back through the host, as the reference uses it); 1 thrust::reduce_by_key ->
// float[segs]; 2 thrust::inclusive_scan -> float[n]; 3 thrust::inclusive_scan_by_key -> float[n].
extern "C" int tcu_thrust_run(int op, const void* d_in, void* d_out, size_t n, size_t segment_size,
                              void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  InIt in(static_cast<const __half*>(d_in), HalfToFloat());
  auto pol = thrust::cuda::par.on(st);
  KeyIt keys(cub::CountingInputIterator<long long>(0), SegmentOf{(long long)segment_size});
  try {
    switch (op) {
      case 0: {
        const float total = thrust::reduce(pol, in, in + n, 0.0f);
        return cudaMemcpyAsync(d_out, &total, sizeof(total), cudaMemcpyHostToDevice, st) == cudaSuccess &&
                       cudaStreamSynchronize(st) == cudaSuccess
                   ? 0
                   : 1;
      }
      case 1:
        thrust::reduce_by_key(pol, keys, keys + n, in, thrust::make_discard_iterator(),
                              static_cast<float*>(d_out));
        return 0;
      case 2: thrust::inclusive_scan(pol, in, in + n, static_cast<float*>(d_out)); return 0;
      case 3:
        thrust::inclusive_scan_by_key(pol, keys, keys + n, in, static_cast<float*>(d_out));
        return 0;
      default: return (int)cudaErrorInvalidValue;
    }
  } catch (...) {
    cudaGetLastError();
    return 2;
  }
}
