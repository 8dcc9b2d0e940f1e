// tcu_bench -- the reference's benchmark surface over this library.
//
// c3sr/tcu_scope is one Google-Benchmark binary; every operator is a registered
// benchmark whose NAME (template arguments and "/arg_name:value" suffixes
// included) is what its plot specs select on (figures/spec/*.yml, parsed by
// tools/plot.py:117-165).  This runner registers the same names with the same
// argument sweeps (src/reduction/args.hpp:38-146) for the tensor-core reduce /
// scan families, times them the same way (CUDA events around the call, manual
// time, src/reduction/seg_wmma_16n.cu:57-73), reports the same counters
// (:75-81, "flops" = elements per second) and writes the same JSON schema, so
// the reference's tooling reads its output unchanged.  Google Benchmark itself
// is not needed.
//
// The WARPS_PER_BLOCK / SEGMENTS_PER_WARP / SEGMENT_SIZE template arguments of
// the reference's names select launch shapes of its kernels.  This library picks
// its launch shape itself, per segment class (persistent CTAs of 8 or 16
// consumer warps, one or two per SM), so those arguments are INERT here: they
// are kept in the name so that result files keep their names, reported as
// "warps_per_block" like the reference does, and every result carries a
// "label" saying so.  The same goes for the CUDA_UNSAFE_WMMA_* names
// (src/unsafe_reduction, src/unsafe_prefixsum): their one difference in the
// reference -- the constant matrix is written straight into fragment registers
// instead of being staged through shared memory -- is how every kernel of this
// library builds its constant operand.
//
//   tcu_bench --benchmark_filter='SEGMENTED_REDUCTION_16N<8>.*segment_size:16/' \
//             --benchmark_out=results.json --benchmark_out_format=json
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <regex>
#include <string>
#include <vector>

#include "../../include/tcu_scope.h"

namespace {

struct Options {
  std::string filter = ".*";
  std::string out_path;
  bool list_only    = false;
  double min_time   = 0.2;  // seconds of measured GPU time per benchmark
  int device        = 0;    // the reference defaults to 1 and falls back to 0 (src/init/flags.cpp:4)
  uint64_t seed     = 2024;
  bool const_fill   = false;  // the reference's constant 0.001 fill instead of seeded uniform
  bool validate     = false;
  bool cold_cache   = true;   // rotate over buffers until the working set exceeds 2x L2
  int algo          = TCU_ALGO_AUTO;
  int out_type      = -1;     // -1: fp32 for reductions and the full scan, fp16 for segmented scans
  int min_log2 = 12, max_log2 = 30;  // src/reduction/args.hpp:39-40
  int num_gpus = 1;  // > 1: the array is cut into one contiguous shard per device (whole segments)
};

struct Benchmark {
  std::string name;
  int op;
  size_t num_segments, segment_size, num_elements;
  int warps_per_block;
  std::vector<std::pair<std::string, long long>> extra_counters;
};

struct Result {
  std::string name;
  bool error = false;
  std::string error_message;
  long long iterations = 0;
  std::string label;
  double real_time_ns = 0, cpu_time_ns = 0;
  std::vector<std::pair<std::string, double>> counters;
};

#define CHECK_CUDA(x)                                                          \
  do {                                                                         \
    cudaError_t e_ = (x);                                                      \
    if (e_ != cudaSuccess) throw std::string(#x ": ") + cudaGetErrorString(e_); \
  } while (0)

void check_tcu(int st, const char* what) {
  if (st != TCU_OK) throw std::string(what) + ": " + tcu_status_string(st);
}

// ---------------------------------------------------------------- registry
const int kWarpsPerBlock[] = {1, 2, 4, 8, 16};

std::string seg_name(const std::string& base, int wpb, size_t segs, size_t s, size_t n) {
  return base + "<" + std::to_string(wpb) + ">/num_segments:" + std::to_string(segs) +
         "/segment_size:" + std::to_string(s) + "/num_elements:" + std::to_string(n) + "/manual_time";
}

void add_segmented(std::vector<Benchmark>& out, const Options& o, const std::string& base, int op,
                   std::initializer_list<size_t> sizes) {
  for (size_t s : sizes)  // ArgsParamsSegmented<S>, src/reduction/args.hpp:50-62
    for (int wpb : kWarpsPerBlock)
      for (int l = o.min_log2; l <= o.max_log2; ++l) {
        const size_t n = size_t(1) << l;
        if (n < s) continue;
        out.push_back({seg_name(base, wpb, n / s, s, n), op, n / s, s, n, wpb, {}});
      }
}

void add_tune(std::vector<Benchmark>& out, const std::string& base, int op, size_t base_seg,
              int max_log2) {
  // TuningArgs<BASE, LOG2MAX>, src/reduction/args.hpp:82-96
  const size_t n = size_t(1) << max_log2;
  for (int wpb : kWarpsPerBlock)
    for (size_t segs = n / base_seg; segs >= 1; segs /= 2) {
      const size_t s = n / segs;
      std::string name = base + "<" + std::to_string(wpb) + ">/num_segments:" +
                         std::to_string(segs) + "/segment_size:" + std::to_string(s) +
                         "/base_segment_size:" + std::to_string(base_seg) +
                         "/max_elements_log2:" + std::to_string(max_log2) + "/manual_time";
      out.push_back({name, op, segs, s, n, wpb,
                     {{"base_segment_size", (long long)base_seg}, {"max_elements_log2", max_log2}}});
      if (segs == 1) break;
    }
}

// Fixed-size kernels carry two template arguments, <SEGMENTS_PER_WARP, WARPS_PER_BLOCK>
// (src/reduction/seg_wmma_16.cu:132-147, seg_wmma_256.cu; same in src/prefixsum).
void add_fixed(std::vector<Benchmark>& out, const Options& o, const std::string& base, int op,
               size_t s) {
  for (int spw : {1, 2, 4, 8})
    for (int wpb : {1, 2, 4, 8})
      for (int l = o.min_log2; l <= o.max_log2; ++l) {
        const size_t n = size_t(1) << l;
        if (n < s) continue;
        out.push_back({base + "<" + std::to_string(spw) + ", " + std::to_string(wpb) +
                           ">/num_segments:" + std::to_string(n / s) + "/segment_size:" +
                           std::to_string(s) + "/num_elements:" + std::to_string(n) + "/manual_time",
                       op, n / s, s, n, wpb, {}});
      }
}

void add_full(std::vector<Benchmark>& out, const Options& o, const std::string& base, int op,
              int max_mult) {
  // BENCHMARK_TEMPLATE(name, SEGMENT_SIZE, WARPS_PER_BLOCK)->ARGS(): the template
  // arguments appear in the name as written, e.g. "<64 * 256, 8>"
  for (int mult = 1; mult <= max_mult; mult *= 2)
    for (int wpb : kWarpsPerBlock)
      for (int l = o.min_log2; l <= o.max_log2; ++l) {
        const size_t n = size_t(1) << l;
        if (n < size_t(mult) * 256) continue;  // "num_elements must be multiples of SEGMENT_SIZE"
        const std::string seg = mult == 1 ? "256" : std::to_string(mult) + " * 256";
        out.push_back({base + "<" + seg + ", " + std::to_string(wpb) + ">/num_elements:" +
                           std::to_string(n) + "/manual_time",
                       op, 1, n, n, wpb, {{"segment_size", (long long)mult * 256}}});
      }
}

void add_family(std::vector<Benchmark>& b, const Options& o, const std::string& prefix);

std::vector<Benchmark> registry(const Options& o) {
  std::vector<Benchmark> b;
  add_family(b, o, "CUDA_WMMA_");
  // src/unsafe_reduction/seg_wmma_16n.cu:183-229, src/unsafe_prefixsum/seg_wmma_16n.cu:188-194
  // and their siblings: the same registrations under the CUDA_UNSAFE_WMMA_ prefix
  add_family(b, o, "CUDA_UNSAFE_WMMA_");
  return b;
}

void add_family(std::vector<Benchmark>& b, const Options& o, const std::string& prefix) {
  const bool unsafe = prefix.find("UNSAFE") != std::string::npos;
  const std::initializer_list<size_t> k16n  = {16, 32, 64, 128, 256, 512, 1024};
  const std::initializer_list<size_t> k256n = {256, 512, 1024, 2048, 4096, 8192, 16384};
  // Every variant name of the reference maps onto the one kernel family of this
  // library (warps per block, segments per warp, _OPT / _BLOCK are tuning knobs of
  // kernels that no longer exist), so result files keep their names.
  // src/reduction/seg_wmma_16n.cu:215-221, seg_wmma_16n_opt.cu:209-221, seg_wmma_16n_block.cu:213-235,
  // seg_wmma_256n.cu:223-229, seg_wmma_256n_block.cu, seg_wmma_16.cu:132-147, seg_wmma_256.cu
  for (const char* v : {"", "_OPT", "_BLOCK"}) {
    add_segmented(b, o, (prefix + "SEGMENTED_REDUCTION_16N") + v, TCU_OP_SEGMENTED_REDUCE, k16n);
    add_tune(b, (prefix + "TUNE_SEGMENTED_REDUCTION_16N") + v, TCU_OP_SEGMENTED_REDUCE, 16, 30);
  }
  for (const char* v : {"", "_BLOCK"}) {
    add_segmented(b, o, (prefix + "SEGMENTED_REDUCTION_256N") + v, TCU_OP_SEGMENTED_REDUCE, k256n);
    add_tune(b, (prefix + "TUNE_SEGMENTED_REDUCTION_256N") + v, TCU_OP_SEGMENTED_REDUCE, 256, 22);
    add_tune(b, (prefix + "TUNE_SEGMENTED_REDUCTION_256N") + v, TCU_OP_SEGMENTED_REDUCE, 256, 30);
  }
  add_fixed(b, o, prefix + "SEGMENTED_REDUCTION_16", TCU_OP_SEGMENTED_REDUCE, 16);
  add_fixed(b, o, prefix + "SEGMENTED_REDUCTION_256", TCU_OP_SEGMENTED_REDUCE, 256);
  // src/reduction/wmma_2kers.cu:172-194, wmma_2kers_block.cu:173-198, wmma_cg.cu:171-195,
  // wmma_atomic.cu:163-185
  add_full(b, o, prefix + "FULL_REDUCTION_2KERS_BASE_16", TCU_OP_FULL_REDUCE, 16);
  add_full(b, o, prefix + "FULL_REDUCTION_2KERS_BASE_256", TCU_OP_FULL_REDUCE, 16);
  add_full(b, o, prefix + "FULL_REDUCTION_2KERS_BLOCK_BASE_16", TCU_OP_FULL_REDUCE, 256);
  add_full(b, o, prefix + "FULL_REDUCTION_2KERS_BLOCK_BASE_256", TCU_OP_FULL_REDUCE, 256);
  add_full(b, o, prefix + "FULL_REDUCTION_CG", TCU_OP_FULL_REDUCE, 1024);
  // the unsafe tree registers these two without the underscore after WMMA
  // (src/unsafe_reduction/wmma_atomic.cu:166,172); the name is kept as it is there
  const std::string atomic_prefix = unsafe ? "CUDA_UNSAFE_WMMA" : prefix;
  add_full(b, o, atomic_prefix + "FULL_REDUCTION_ATOMIC_W_ATOMIC_BALLOT", TCU_OP_FULL_REDUCE, 16);
  add_full(b, o, atomic_prefix + "FULL_REDUCTION_ATOMIC_W_BLOCK_SYNC", TCU_OP_FULL_REDUCE, 16);
  // src/prefixsum/seg_wmma_16n.cu:217-223, seg_wmma_16n_opt.cu:211-223, seg_wmma_16n_block.cu:216-238,
  // seg_wmma_256n.cu:216-222, seg_wmma_256n_block.cu:211-233, seg_wmma_16.cu, seg_wmma_256.cu
  for (const char* v : {"", "_OPT", "_BLOCK"}) {
    add_segmented(b, o, (prefix + "SEGMENTED_PREFIXSUM_16N") + v, TCU_OP_SEGMENTED_SCAN, k16n);
    add_tune(b, (prefix + "TUNE_SEGMENTED_PREFIXSUM_16N") + v, TCU_OP_SEGMENTED_SCAN, 16, 30);
  }
  for (const char* v : {"", "_BLOCK"}) {
    add_segmented(b, o, (prefix + "SEGMENTED_PREFIXSUM_256N") + v, TCU_OP_SEGMENTED_SCAN, k256n);
    add_tune(b, (prefix + "TUNE_SEGMENTED_PREFIXSUM_256N") + v, TCU_OP_SEGMENTED_SCAN, 256, 30);
  }
  add_fixed(b, o, prefix + "SEGMENTED_PREFIXSUM_16", TCU_OP_SEGMENTED_SCAN, 16);
  add_fixed(b, o, prefix + "SEGMENTED_PREFIXSUM_256", TCU_OP_SEGMENTED_SCAN, 256);
  // src/prefixsum/wmma_3kers.cu:161-183, wmma_3kers_block.cu:175-185, wmma_cg.cu:183-207,
  // wmma_atomic.cu:176-200
  add_full(b, o, prefix + "FULL_PREFIXSUM_3KERS", TCU_OP_FULL_SCAN, 16);
  add_full(b, o, prefix + "FULL_PREFIXSUM_3KERS_BLOCK", TCU_OP_FULL_SCAN, 256);
  add_full(b, o, prefix + "FULL_PREFIXSUM_CG", TCU_OP_FULL_SCAN, 1024);
  add_full(b, o, prefix + "FULL_PREFIXSUM_ATOMIC_W_ATOMIC_BALLOT", TCU_OP_FULL_SCAN, 1024);
  add_full(b, o, prefix + "FULL_PREFIXSUM_ATOMIC_W_BLOCK_SYNC", TCU_OP_FULL_SCAN, 1024);
}

// ------------------------------------------------------------- validation
// The sequential check the reference's drivers carry but compile out
// (src/reduction/seg_wmma_16n.cu:82-109, src/prefixsum/wmma_3kers.cu:92-129),
// in double, with the tolerances of this build: fp32 1e-3 relative / 1e-5
// absolute, fp16 two representable halves.
double half_to_double(uint16_t h) {
  const int sign = h >> 15, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
  double v = exp == 0 ? std::ldexp((double)man, -24)
                      : (exp == 31 ? (man ? NAN : INFINITY) : std::ldexp((double)(man | 0x400), exp - 25));
  return sign ? -v : v;
}

bool close_enough(double got, double ref, bool f32) {
  if (!(got == got)) return false;
  if (f32) return std::fabs(got - ref) <= std::max(1e-3 * std::fabs(ref), 1e-5);
  if (std::fabs(ref) >= 65520.0) return std::isinf(got) && (got > 0) == (ref > 0);  // half overflows
  // fp16: |got - ref| within 2 half-ULP of ref (+ half an ULP for ref's own rounding)
  const double mag = std::max(std::fabs(ref), std::ldexp(1.0, -14));
  const double ulp = std::ldexp(1.0, (int)std::floor(std::log2(mag)) - 10);
  return std::fabs(got - ref) <= 2.5 * ulp;
}

std::string validate(const Benchmark& b, bool f32, const void* d_in, const void* d_out) {
  // first and last few segments (all of it when small)
  const size_t S = b.segment_size, segs = b.num_segments;
  const bool scan = b.op == TCU_OP_SEGMENTED_SCAN || b.op == TCU_OP_FULL_SCAN;
  const size_t max_elems = size_t(1) << 22;
  std::vector<size_t> check;
  if (S > max_elems && scan) return "";  // a running sum from the start is needed; skip huge scans
  const size_t per_side = std::max<size_t>(1, std::min<size_t>(segs, max_elems / std::max<size_t>(S, 1)) / 2);
  for (size_t j = 0; j < std::min(per_side, segs); ++j) check.push_back(j);
  for (size_t j = segs > per_side ? segs - per_side : 0; j < segs; ++j)
    if (j >= per_side) check.push_back(j);
  std::vector<uint16_t> in(S);
  const size_t osz = f32 ? 4 : 2;
  std::vector<uint8_t> out(scan ? S * osz : osz);
  for (size_t j : check) {
    CHECK_CUDA(cudaMemcpy(in.data(), (const uint8_t*)d_in + j * S * 2, S * 2, cudaMemcpyDeviceToHost));
    const size_t ocount = scan ? S : 1;
    CHECK_CUDA(cudaMemcpy(out.data(), (const uint8_t*)d_out + (scan ? j * S : j) * osz, ocount * osz,
                          cudaMemcpyDeviceToHost));
    double acc = 0.0;
    for (size_t i = 0; i < S; ++i) {
      acc += half_to_double(in[i]);
      if (scan || i + 1 == S) {
        const size_t k = scan ? i : 0;
        const double got = f32 ? (double)((const float*)out.data())[k]
                               : half_to_double(((const uint16_t*)out.data())[k]);
        if (!close_enough(got, acc, f32)) {
          char msg[160];
          std::snprintf(msg, sizeof msg, "validation failed: segment %zu element %zu expected %.9g got %.9g",
                        j, i, acc, got);
          return msg;
        }
      }
    }
  }
  return "";
}

// ------------------------------------------------------------------ runner
Result run_one(const Benchmark& b, const Options& o) {
  Result r;
  r.name = b.name;
  const bool reduce = b.op == TCU_OP_SEGMENTED_REDUCE || b.op == TCU_OP_FULL_REDUCE;
  const int out_type = b.op == TCU_OP_FULL_REDUCE ? TCU_OUT_F32
                       : (o.out_type >= 0 ? o.out_type
                                          : (reduce || b.op == TCU_OP_FULL_SCAN ? TCU_OUT_F32 : TCU_OUT_F16));
  const size_t osz = out_type == TCU_OUT_F32 ? 4 : 2;
  const size_t n = b.num_elements;
  const size_t in_bytes = n * 2, out_bytes = (reduce ? b.num_segments : n) * osz;
  // cold cache: enough buffer sets that the working set exceeds twice the 126 MB L2
  int sets = 1;
  if (o.cold_cache) sets = (int)std::min<size_t>(64, std::max<size_t>(1, (size_t(256) << 20) / (in_bytes + out_bytes) + 1));
  std::vector<void*> d_in(sets, nullptr), d_out(sets, nullptr);
  void* d_ws = nullptr;
  double* d_f64 = nullptr;
  cudaEvent_t start = nullptr, stop = nullptr;
  auto cleanup = [&]() {
    for (void* p : d_in) if (p) cudaFree(p);
    for (void* p : d_out) if (p) cudaFree(p);
    if (d_ws) cudaFree(d_ws);
    if (d_f64) cudaFree(d_f64);
    if (start) cudaEventDestroy(start);
    if (stop) cudaEventDestroy(stop);
  };
  try {
    const size_t ws_bytes = tcu_workspace_bytes(b.op, n, b.segment_size);
    if (ws_bytes) CHECK_CUDA(cudaMalloc(&d_ws, ws_bytes));
    CHECK_CUDA(cudaMalloc((void**)&d_f64, 8));
    const bool full = b.op == TCU_OP_FULL_REDUCE || b.op == TCU_OP_FULL_SCAN;
    const int dist = o.const_fill ? TCU_DIST_CONST_0P001 : (full ? TCU_DIST_UNIFORM_01 : TCU_DIST_UNIFORM_PM1);
    for (int k = 0; k < sets; ++k) {
      CHECK_CUDA(cudaMalloc(&d_in[k], in_bytes));
      CHECK_CUDA(cudaMalloc(&d_out[k], std::max<size_t>(out_bytes, 16)));
      check_tcu(tcu_fill_f16(d_in[k], n, o.seed + k, 0, dist, nullptr), "tcu_fill_f16");
    }
    CHECK_CUDA(cudaEventCreate(&start));
    CHECK_CUDA(cudaEventCreate(&stop));
    auto call = [&](int k) {
      switch (b.op) {
        case TCU_OP_SEGMENTED_REDUCE:
          return tcu_segmented_reduce_f16(d_in[k], d_out[k], out_type, b.num_segments, b.segment_size,
                                          o.algo, d_ws, ws_bytes, nullptr);
        case TCU_OP_SEGMENTED_SCAN:
          return tcu_segmented_scan_f16(d_in[k], d_out[k], out_type, b.num_segments, b.segment_size,
                                        o.algo, d_ws, ws_bytes, nullptr);
        case TCU_OP_FULL_REDUCE:
          return tcu_full_reduce_f16(d_in[k], (float*)d_out[k], d_f64, n, o.algo, d_ws, ws_bytes, nullptr);
        default:
          return tcu_full_scan_f16(d_in[k], d_out[k], out_type, n, nullptr, 0,
                                   o.algo == TCU_ALGO_SHUFFLE ? TCU_ALGO_AUTO : o.algo, d_ws, ws_bytes, nullptr);
      }
    };
    for (int w = 0; w < 3; ++w) check_tcu(call(w % sets), "warm-up");
    CHECK_CUDA(cudaDeviceSynchronize());
    double total_ms = 0.0;
    long long iters = 0;
    const auto host_t0 = std::chrono::steady_clock::now();
    while ((total_ms < o.min_time * 1e3 && iters < 100000) || iters < 3) {
      const int k = (int)(iters % sets);
      CHECK_CUDA(cudaEventRecord(start));
      check_tcu(call(k), "call");
      CHECK_CUDA(cudaEventRecord(stop));
      CHECK_CUDA(cudaEventSynchronize(stop));
      float ms = 0.f;
      CHECK_CUDA(cudaEventElapsedTime(&ms, start, stop));
      total_ms += ms;
      ++iters;
    }
    const double host_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - host_t0).count();
    unsigned int bits = 0;
    check_tcu(tcu_device_error(&bits, 1), "device error word");
    if (o.validate) {
      const std::string msg = validate(b, out_type == TCU_OUT_F32, d_in[(iters - 1) % sets], d_out[(iters - 1) % sets]);
      if (!msg.empty()) throw msg;
    }
    r.iterations   = iters;
    r.label        = "template arguments are inert: the library picks its launch shape per segment class";
    r.real_time_ns = total_ms * 1e6 / iters;
    r.cpu_time_ns  = host_ms * 1e6 / iters;
    const double secs = total_ms * 1e-3;
    const double bytes_alg = (double)in_bytes + (double)out_bytes;
    r.counters = {{"num_segments", (double)b.num_segments},
                  {"segment_size", (double)b.segment_size},
                  {"num_elements", (double)n},
                  {"warps_per_block", (double)b.warps_per_block},
                  {"flops", (double)iters * (double)n / secs},  // elements per second
                  {"bytes_algorithmic", bytes_alg},
                  {"gbytes_per_s", (double)iters * bytes_alg / secs / 1e9},
                  {"cold_cache_buffer_sets", (double)sets}};
    for (auto& kv : b.extra_counters) {
      bool have = false;
      for (auto& c : r.counters) if (c.first == kv.first) { c.second = (double)kv.second; have = true; }
      if (!have) r.counters.push_back({kv.first, (double)kv.second});
    }
  } catch (const std::string& e) {  // the reference's SkipWithError (seg_wmma_16n.cu:126-134)
    r.error = true;
    r.error_message = e;
    cudaGetLastError();
  }
  cleanup();
  return r;
}

// --num_gpus=G: one array, G contiguous shards of whole segments, one per device, driven by
// this one host thread (the reference is single-device, src/init/cuda.cpp:45).  Segmented
// operations need no communication; the full reduction and the full scan go through
// tcu_mgpu_* (the shard totals are stored by the kernels into every device's memory).  The
// time of an iteration is the longest of the devices' own event intervals; "flops" counts
// the elements of all shards.
Result run_one_multi(const Benchmark& b, const Options& o) {
  Result r;
  r.name = b.name;
  const int G = o.num_gpus;
  const bool reduce = b.op == TCU_OP_SEGMENTED_REDUCE || b.op == TCU_OP_FULL_REDUCE;
  const bool full   = b.op == TCU_OP_FULL_REDUCE || b.op == TCU_OP_FULL_SCAN;
  const int out_type = b.op == TCU_OP_FULL_REDUCE ? TCU_OUT_F32
                       : (o.out_type >= 0 ? o.out_type
                                          : (reduce || b.op == TCU_OP_FULL_SCAN ? TCU_OUT_F32 : TCU_OUT_F16));
  const size_t osz = out_type == TCU_OUT_F32 ? 4 : 2;
  struct Dev {
    void *in = nullptr, *out = nullptr, *ws = nullptr;
    cudaStream_t st = nullptr;
    cudaEvent_t start = nullptr, stop = nullptr;
    tcu_mgpu_ctx* ctx = nullptr;
    size_t first = 0, elems = 0, units = 0;  // shard: first element, elements, segments
    size_t ws_bytes = 0;
  };
  std::vector<Dev> dev(G);
  auto cleanup = [&]() {
    for (int d = 0; d < G; ++d) {
      cudaSetDevice(d);
      cudaDeviceSynchronize();
    }
    for (int d = 0; d < G; ++d) {  // every device is idle: nobody stores into a peer any more
      cudaSetDevice(d);
      Dev& v = dev[d];
      if (v.ctx) tcu_mgpu_ctx_destroy(v.ctx);
      if (v.in) cudaFree(v.in);
      if (v.out) cudaFree(v.out);
      if (v.ws) cudaFree(v.ws);
      if (v.start) cudaEventDestroy(v.start);
      if (v.stop) cudaEventDestroy(v.stop);
      if (v.st) cudaStreamDestroy(v.st);
    }
    cudaSetDevice(o.device);
  };
  try {
    // units of sharding: whole segments, or groups of 16 elements for the full operations
    const size_t unit = full ? 16 : b.segment_size;
    const size_t units = b.num_elements / unit;
    const int dist = o.const_fill ? TCU_DIST_CONST_0P001 : (full ? TCU_DIST_UNIFORM_01 : TCU_DIST_UNIFORM_PM1);
    std::vector<tcu_mgpu_ctx*> group(G, nullptr);
    for (int d = 0; d < G; ++d) {
      CHECK_CUDA(cudaSetDevice(d));
      Dev& v = dev[d];
      const size_t ub = units * d / G, ue = units * (d + 1) / G;
      v.first = ub * unit;
      v.elems = (ue - ub) * unit;
      v.units = ue - ub;
      CHECK_CUDA(cudaStreamCreateWithFlags(&v.st, cudaStreamNonBlocking));
      CHECK_CUDA(cudaEventCreate(&v.start));
      CHECK_CUDA(cudaEventCreate(&v.stop));
      CHECK_CUDA(cudaMalloc(&v.in, std::max<size_t>(v.elems * 2, 16)));
      CHECK_CUDA(cudaMalloc(&v.out, std::max<size_t>((reduce ? (full ? 1 : v.units) : v.elems) * osz, 16)));
      v.ws_bytes = full ? 0 : tcu_workspace_bytes(b.op, v.elems, b.segment_size);
      if (v.ws_bytes) CHECK_CUDA(cudaMalloc(&v.ws, v.ws_bytes));
      check_tcu(tcu_fill_f16(v.in, v.elems, o.seed, v.first, dist, v.st), "tcu_fill_f16");
      if (full) {
        check_tcu(tcu_mgpu_ctx_create(&v.ctx, d, G, nullptr), "tcu_mgpu_ctx_create");
        group[d] = v.ctx;
      }
    }
    if (full)
      for (int d = 0; d < G; ++d) check_tcu(tcu_mgpu_ctx_connect_local(dev[d].ctx, group.data()), "tcu_mgpu_ctx_connect_local");
    auto call = [&](int d) {
      Dev& v = dev[d];
      switch (b.op) {
        case TCU_OP_SEGMENTED_REDUCE:
          return tcu_segmented_reduce_f16(v.in, v.out, out_type, v.units, b.segment_size, o.algo, v.ws, v.ws_bytes, v.st);
        case TCU_OP_SEGMENTED_SCAN:
          return tcu_segmented_scan_f16(v.in, v.out, out_type, v.units, b.segment_size, o.algo, v.ws, v.ws_bytes, v.st);
        case TCU_OP_FULL_REDUCE: return tcu_mgpu_full_reduce_f16(v.ctx, v.in, (float*)v.out, nullptr, v.elems, v.st);
        default: return tcu_mgpu_full_scan_f16(v.ctx, v.in, v.out, out_type, v.elems, v.st);
      }
    };
    auto round = [&](bool timed) {
      for (int d = 0; d < G; ++d) {
        CHECK_CUDA(cudaSetDevice(d));
        if (timed) CHECK_CUDA(cudaEventRecord(dev[d].start, dev[d].st));
        check_tcu(call(d), "call");
        if (timed) CHECK_CUDA(cudaEventRecord(dev[d].stop, dev[d].st));
      }
      float worst = 0.f;
      for (int d = 0; d < G; ++d) {
        CHECK_CUDA(cudaSetDevice(d));
        CHECK_CUDA(cudaStreamSynchronize(dev[d].st));
        if (timed) {
          float ms = 0.f;
          CHECK_CUDA(cudaEventElapsedTime(&ms, dev[d].start, dev[d].stop));
          worst = std::max(worst, ms);
        }
      }
      return worst;
    };
    for (int w = 0; w < 3; ++w) round(false);
    double total_ms = 0.0;
    long long iters = 0;
    const auto host_t0 = std::chrono::steady_clock::now();
    while ((total_ms < o.min_time * 1e3 && iters < 100000) || iters < 3) {
      total_ms += round(true);
      ++iters;
    }
    const double host_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - host_t0).count();
    for (int d = 0; d < G; ++d) {
      CHECK_CUDA(cudaSetDevice(d));
      unsigned int bits = 0;
      check_tcu(tcu_device_error(&bits, 1), "device error word");
    }
    if (o.validate) {
      // every shard against the sequential sum of ITS segments; the full scan against the
      // running sum continued from the earlier shards (their totals summed on the host)
      double carry = 0.0;
      for (int d = 0; d < G; ++d) {
        CHECK_CUDA(cudaSetDevice(d));
        const Dev& v = dev[d];
        if (!full) {
          Benchmark sb = b;
          sb.num_segments = v.units;
          sb.num_elements = v.elems;
          const std::string msg = validate(sb, out_type == TCU_OUT_F32, v.in, v.out);
          if (!msg.empty()) throw "device " + std::to_string(d) + ": " + msg;
          continue;
        }
        std::vector<uint16_t> in(v.elems);
        CHECK_CUDA(cudaMemcpy(in.data(), v.in, v.elems * 2, cudaMemcpyDeviceToHost));
        std::vector<uint8_t> out(b.op == TCU_OP_FULL_SCAN ? v.elems * osz : 0);
        if (!out.empty()) CHECK_CUDA(cudaMemcpy(out.data(), v.out, out.size(), cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < v.elems; ++i) {
          carry += half_to_double(in[i]);
          if (b.op != TCU_OP_FULL_SCAN) continue;
          const double got = out_type == TCU_OUT_F32 ? (double)((const float*)out.data())[i]
                                                     : half_to_double(((const uint16_t*)out.data())[i]);
          if (!close_enough(got, carry, out_type == TCU_OUT_F32))
            throw "validation failed: device " + std::to_string(d) + " element " + std::to_string(i);
        }
      }
      if (b.op == TCU_OP_FULL_REDUCE)
        for (int d = 0; d < G; ++d) {  // every device holds the sum over all shards
          CHECK_CUDA(cudaSetDevice(d));
          float got = 0.f;
          CHECK_CUDA(cudaMemcpy(&got, dev[d].out, 4, cudaMemcpyDeviceToHost));
          if (!close_enough(got, carry, true)) throw "validation failed: total on device " + std::to_string(d);
        }
    }
    r.iterations   = iters;
    r.label        = "template arguments are inert: the library picks its launch shape per segment class";
    r.real_time_ns = total_ms * 1e6 / iters;
    r.cpu_time_ns  = host_ms * 1e6 / iters;
    const double secs = total_ms * 1e-3;
    const double n = (double)b.num_elements;
    const double bytes_alg = n * 2 + (reduce ? (double)b.num_segments : n) * osz;
    r.counters = {{"num_segments", (double)b.num_segments},
                  {"segment_size", (double)b.segment_size},
                  {"num_elements", n},
                  {"warps_per_block", (double)b.warps_per_block},
                  {"flops", (double)iters * n / secs},
                  {"bytes_algorithmic", bytes_alg},
                  {"gbytes_per_s", (double)iters * bytes_alg / secs / 1e9},
                  {"num_gpus", (double)G}};
    for (auto& kv : b.extra_counters) {
      bool have = false;
      for (auto& c : r.counters) if (c.first == kv.first) { c.second = (double)kv.second; have = true; }
      if (!have) r.counters.push_back({kv.first, (double)kv.second});
    }
  } catch (const std::string& e) {
    r.error = true;
    r.error_message = e;
    cudaGetLastError();
  }
  cleanup();
  return r;
}

std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') o += '\\';
    o += c;
  }
  return o;
}

void write_json(const std::string& path, const std::vector<Result>& results, const Options& o) {
  FILE* f = std::fopen(path.c_str(), "w");
  if (!f) { std::fprintf(stderr, "cannot open %s\n", path.c_str()); return; }
  cudaDeviceProp prop{};
  cudaGetDeviceProperties(&prop, o.device);
  std::fprintf(f, "{\n  \"context\": {\n    \"executable\": \"tcu_bench\",\n    \"gpu\": \"%s\",\n"
                  "    \"num_sms\": %d,\n    \"library_build_type\": \"release\"\n  },\n  \"benchmarks\": [\n",
               prop.name, prop.multiProcessorCount);
  for (size_t i = 0; i < results.size(); ++i) {
    const Result& r = results[i];
    std::fprintf(f, "    {\n      \"name\": \"%s\",\n", json_escape(r.name).c_str());
    if (r.error) {
      std::fprintf(f, "      \"error_occurred\": true,\n      \"error_message\": \"%s\",\n",
                   json_escape(r.error_message).c_str());
    }
    std::fprintf(f, "      \"iterations\": %lld,\n      \"real_time\": %.6e,\n      \"cpu_time\": %.6e,\n"
                    "      \"time_unit\": \"ns\"",
                 r.iterations, r.real_time_ns, r.cpu_time_ns);
    if (!r.label.empty()) std::fprintf(f, ",\n      \"label\": \"%s\"", json_escape(r.label).c_str());
    for (auto& c : r.counters) std::fprintf(f, ",\n      \"%s\": %.6e", c.first.c_str(), c.second);
    std::fprintf(f, "\n    }%s\n", i + 1 < results.size() ? "," : "");
  }
  std::fprintf(f, "  ]\n}\n");
  std::fclose(f);
}

bool flag_value(const char* arg, const char* name, std::string* value) {
  const size_t n = std::strlen(name);
  if (std::strncmp(arg, name, n) != 0) return false;
  if (arg[n] == '=') { *value = arg + n + 1; return true; }
  if (arg[n] == '\0') { *value = "true"; return true; }
  return false;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    std::string v;
    if (flag_value(argv[i], "--benchmark_filter", &v)) o.filter = v;
    else if (flag_value(argv[i], "--benchmark_out_format", &v)) { /* json only */ }
    else if (flag_value(argv[i], "--benchmark_out", &v)) o.out_path = v;
    else if (flag_value(argv[i], "--benchmark_list_tests", &v)) o.list_only = v != "false";
    else if (flag_value(argv[i], "--benchmark_min_time", &v)) o.min_time = std::atof(v.c_str());
    else if (flag_value(argv[i], "--benchmark_counters_tabular", &v)) { /* accepted, as src/main.cpp:44 adds it */ }
    else if (flag_value(argv[i], "--cuda_device_id", &v)) o.device = std::atoi(v.c_str());
    else if (flag_value(argv[i], "--seed", &v)) o.seed = std::strtoull(v.c_str(), nullptr, 10);
    else if (flag_value(argv[i], "--fill", &v)) o.const_fill = v == "const";
    else if (flag_value(argv[i], "--validate", &v)) o.validate = v != "false";
    else if (flag_value(argv[i], "--cold_cache", &v)) o.cold_cache = v != "false" && v != "0";
    else if (flag_value(argv[i], "--algo", &v)) o.algo = v == "shuffle" ? TCU_ALGO_SHUFFLE : v == "tcgen05" ? TCU_ALGO_TCGEN05 : TCU_ALGO_MMA;
    else if (flag_value(argv[i], "--out_type", &v)) o.out_type = v == "f32" ? TCU_OUT_F32 : TCU_OUT_F16;
    else if (flag_value(argv[i], "--min_log2", &v)) o.min_log2 = std::atoi(v.c_str());
    else if (flag_value(argv[i], "--max_log2", &v)) o.max_log2 = std::atoi(v.c_str());
    else if (flag_value(argv[i], "--num_gpus", &v)) o.num_gpus = std::atoi(v.c_str());
    else {
      std::printf("usage: tcu_bench [--benchmark_filter=REGEX] [--benchmark_list_tests] "
                  "[--benchmark_out=FILE] [--benchmark_min_time=S]\n"
                  "                 [--cuda_device_id=N] [--seed=N] [--fill=uniform|const] [--validate] "
                  "[--cold_cache=0|1]\n"
                  "                 [--algo=mma|shuffle|tcgen05] [--out_type=f16|f32] [--min_log2=N] [--max_log2=N]\n");
      return std::strcmp(argv[i], "-h") == 0 || std::strcmp(argv[i], "--help") == 0 ? 0 : 1;
    }
  }
  std::regex re;
  try {
    re = std::regex(o.filter);
  } catch (const std::regex_error&) {
    std::fprintf(stderr, "bad --benchmark_filter\n");
    return 1;
  }
  std::vector<Benchmark> all = registry(o), selected;
  for (auto& b : all)
    if (std::regex_search(b.name, re)) selected.push_back(b);
  if (o.list_only) {
    for (auto& b : selected) std::printf("%s\n", b.name.c_str());
    return 0;
  }
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    std::fprintf(stderr, "no CUDA device\n");
    return 1;
  }
  if (o.device >= count) o.device = 0;  // as src/init/cuda.cpp:41-43
  if (o.num_gpus < 1 || o.num_gpus > count || o.num_gpus > TCU_MGPU_MAX_RANKS) {
    std::fprintf(stderr, "--num_gpus=%d: this machine has %d device(s)\n", o.num_gpus, count);
    return 1;
  }
  if (o.num_gpus > 1) o.device = 0;  // shards go to devices 0 .. G-1
  cudaSetDevice(o.device);
  std::printf("%-100s %14s %12s %16s\n", "Benchmark", "Time(ns)", "Iterations", "Gelem/s");
  std::vector<Result> results;
  for (auto& b : selected) {
    Result r = o.num_gpus > 1 ? run_one_multi(b, o) : run_one(b, o);
    if (r.error) {
      std::printf("%-100s ERROR OCCURRED: '%s'\n", r.name.c_str(), r.error_message.c_str());
    } else {
      double flops = 0;
      for (auto& c : r.counters) if (c.first == "flops") flops = c.second;
      std::printf("%-100s %14.0f %12lld %16.2f\n", r.name.c_str(), r.real_time_ns, r.iterations, flops / 1e9);
    }
    results.push_back(r);
  }
  if (!o.out_path.empty()) write_json(o.out_path, results, o);
  return 0;
}
