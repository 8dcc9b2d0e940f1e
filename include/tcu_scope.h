/*
 * tcu_scope.h -- C ABI of the B200 (sm_100a) segmented / full reduce and
 * inclusive-scan library for fp16 arrays.
 *
 * The reference project (c3sr/tcu_scope) has no FFI; its operator surface is
 * a set of header-only kernel templates
 *     compute_wmma_<op>_<variant><SEGMENT_SIZE, WARPS_PER_BLOCK, ...>
 *         (const half* d_in, OUT* d_out, [half* partial_sums,] size_t num_segments)
 * launched by one Google-Benchmark driver per variant.  Each entry point below
 * names the kernels / drivers it stands in for.  Conventions shared by all of
 * them, taken from those call sites:
 *   - the caller owns every device buffer (the drivers cudaMalloc them,
 *     src/reduction/seg_wmma_16n.cu:35-36); nothing here allocates or frees;
 *   - segment j occupies in[j*segment_size, (j+1)*segment_size)
 *     (src/reduction/seg_wmma_16n.cu:14-25);
 *   - work is queued on the given stream and the call returns at once;
 *   - the return value is a tcu_status; nothing throws, nothing resets the
 *     device (the reference does both, src/utils/error.hpp:28-46).
 * Pointers are plain device pointers (void*), streams are cudaStream_t passed
 * as void*; there are no C++ or torch types in any signature.
 */
#ifndef TCU_SCOPE_H_
#define TCU_SCOPE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TCU_OK              = 0,
  TCU_ERR_INVALID_ARG = 1, /* null / misaligned pointer, size overflow                  */
  TCU_ERR_UNSUPPORTED = 2, /* segment size 0, unknown algo/type, algo without that size   */
  TCU_ERR_CUDA        = 3, /* a CUDA runtime call failed (see cudaGetLastError)         */
  TCU_ERR_TIMEOUT     = 4, /* a bounded device-side wait ran out (tcu_device_error)     */
  TCU_ERR_WORKSPACE   = 5, /* workspace missing or smaller than tcu_workspace_bytes()   */
  TCU_ERR_TOO_LARGE   = 6  /* more elements than TCU_STATIC_SCAN_MAX_ELEMENTS           */
} tcu_status;

typedef enum {
  TCU_ALGO_AUTO    = 0, /* the fastest tensor-core kernel for the size: mma.sync, or
                           tcgen05 for large scans with 16-bit outputs                  */
  TCU_ALGO_MMA     = 1, /* TMA ring + mma.sync m16n8k16 against ones / triangular ones  */
  TCU_ALGO_SHUFFLE = 2, /* same pipeline, CUDA-core adds + warp shuffles: the ablation  */
  TCU_ALGO_TCGEN05 = 3  /* tcgen05.mma, accumulators in tensor memory; powers of two,
                           num_elements % 64 == 0: segmented reduction of 16 ... 2048
                           elements (plain fp32 accumulation), inclusive segmented scan
                           of 16 ... 16384 elements (exact parts, like TCU_ALGO_MMA),
                           with 16-bit outputs of up to 2^20 elements (2 segments or more) */
} tcu_algo;

typedef enum { TCU_OUT_F16 = 0, TCU_OUT_F32 = 1 } tcu_out_type;

typedef enum {
  TCU_OP_SEGMENTED_REDUCE = 0,
  TCU_OP_SEGMENTED_SCAN   = 1,
  TCU_OP_FULL_REDUCE      = 2,
  TCU_OP_FULL_SCAN        = 3
} tcu_op;

/* Input distributions of tcu_fill_f16 (bit-identical to the CPU oracle's). */
typedef enum {
  TCU_DIST_UNIFORM_PM1 = 0, /* uniform in [-1, 1)                                       */
  TCU_DIST_UNIFORM_01  = 1, /* uniform in [0, 1)                                        */
  TCU_DIST_SMALL_INT   = 2, /* integers -2..2 (every sum exact in any precision)        */
  TCU_DIST_CONST_0P001 = 3  /* half(0.001f): the reference's fill,
                               src/reduction/seg_wmma_16n.cu:38                          */
} tcu_dist;

/*
 * Segmented sum reduction: out[j] = sum of segment j.
 * Replaces compute_wmma_segmented_reduction_16n (src/reduction/kernel.cuh:80-125),
 * ..._256n (:301-356) and ..._256n_block (:418-485) and their drivers
 * CUDA_WMMA_SEGMENTED_REDUCTION_16N / _256N / _256N_BLOCK
 * (src/reduction/seg_wmma_16n.cu:137-221, seg_wmma_256n.cu:149-229).
 * segment_size: any size >= 1.  Powers of two >= 16 (the sizes of the
 * reference's dispatch table, seg_wmma_16n.cu:146-172, and of all its
 * benchmarks) run the tiled kernels at HBM speed; the other multiples of 16
 * the reference accepts run kernels that give a warp 16 segments (reduction,
 * also for multiples of 8 and for any size up to 255) or 16 rows of 16
 * elements (scan) at a time, up to 2048 elements; every other size (tails
 * masked) runs a one-warp-per-segment kernel (TCU_ALGO_AUTO or TCU_ALGO_MMA
 * only).
 * d_out: num_segments floats or halves.
 * A workspace is needed only when segment_size > 16384.
 */
int tcu_segmented_reduce_f16(const void* d_in, void* d_out, int out_type, size_t num_segments,
                             size_t segment_size, int algo, void* d_workspace,
                             size_t workspace_bytes, void* stream);

/*
 * Segmented inclusive prefix sum: out[j*S + i] = in[j*S] + ... + in[j*S + i].
 * Replaces compute_wmma_segmented_prefixsum_16n (src/prefixsum/kernel.cuh:86-150),
 * ..._256n (:441-506), ..._256n_block (:586-678) and their drivers
 * CUDA_WMMA_SEGMENTED_PREFIXSUM_16N / _256N (src/prefixsum/seg_wmma_16n.cu:139-223,
 * seg_wmma_256n.cu:143-222).  d_out: num_segments*segment_size halves or floats.
 * A workspace is needed only when segment_size > 16384.
 */
int tcu_segmented_scan_f16(const void* d_in, void* d_out, int out_type, size_t num_segments,
                           size_t segment_size, int algo, void* d_workspace,
                           size_t workspace_bytes, void* stream);

/*
 * Sum of all num_elements inputs (a multiple of 16) into *d_out (float) and,
 * if d_out_f64 is not null, into *d_out_f64 (double; what a multi-GPU caller
 * gathers).  Replaces CUDA_WMMA_FULL_REDUCTION_2KERS[_BLOCK]_BASE_{16,256}
 * (src/reduction/wmma_2kers.cu:17-193): segmented kernel + cub::DeviceReduce.
 * Always needs a workspace.
 */
int tcu_full_reduce_f16(const void* d_in, float* d_out, double* d_out_f64, size_t num_elements,
                        int algo, void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * Inclusive prefix sum over all num_elements inputs (a multiple of 16).
 * Replaces CUDA_WMMA_FULL_PREFIXSUM_3KERS[_BLOCK] (src/prefixsum/wmma_3kers.cu:14-177):
 * ..._256n_ps + cub::DeviceScan::ExclusiveSum + add_partial_sums, here one pass.
 * For a scan sharded over several GPUs, d_shard_totals points at the gathered
 * per-shard totals (device memory, doubles) and shard_index is this GPU's
 * position: the sum of the earlier shards' totals seeds the scan.  Pass NULL
 * and 0 on one GPU.  Always needs a workspace.
 */
int tcu_full_scan_f16(const void* d_in, void* d_out, int out_type, size_t num_elements,
                      const double* d_shard_totals, int shard_index, int algo,
                      void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * Exclusive variants: out[i] = sum of the elements of the segment BEFORE i (0 for
 * the first).  The reference has inclusive scans only (U has ones on its
 * diagonal, src/prefixsum/kernel.cuh:60); callers that turn counts into offsets
 * need this form, and on the tensor core it is the same product with the
 * diagonal of U removed.  Arguments as for the inclusive entry points; always
 * the tensor-core algorithm.
 */
int tcu_segmented_exclusive_scan_f16(const void* d_in, void* d_out, int out_type,
                                     size_t num_segments, size_t segment_size, void* d_workspace,
                                     size_t workspace_bytes, void* stream);
int tcu_full_exclusive_scan_f16(const void* d_in, void* d_out, int out_type, size_t num_elements,
                                void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * bfloat16 inputs.  Same operations, arguments, status codes, workspace sizes
 * and segment sizes as the *_f16 entry points of the same name; d_in holds
 * bfloat16 values and out_type TCU_OUT_F16 means "16-bit outputs in the type
 * of the input", i.e. bfloat16.  No counterpart in the reference, which is
 * fp16 only (half everywhere in src/reduction/kernel.cuh and
 * src/prefixsum/kernel.cuh); the step next to it that mixed-precision callers
 * need first.  Same kernels, compiled a second time with the bf16 form of the
 * MMA, of the constant matrices and of the exact hi/lo split.  algo:
 * TCU_ALGO_AUTO / _MMA / _SHUFFLE / _TCGEN05 as for fp16.
 */
int tcu_segmented_reduce_bf16(const void* d_in, void* d_out, int out_type, size_t num_segments,
                              size_t segment_size, int algo, void* d_workspace,
                              size_t workspace_bytes, void* stream);
int tcu_segmented_scan_bf16(const void* d_in, void* d_out, int out_type, size_t num_segments,
                            size_t segment_size, int algo, void* d_workspace,
                            size_t workspace_bytes, void* stream);
int tcu_segmented_exclusive_scan_bf16(const void* d_in, void* d_out, int out_type,
                                      size_t num_segments, size_t segment_size, void* d_workspace,
                                      size_t workspace_bytes, void* stream);
int tcu_full_exclusive_scan_bf16(const void* d_in, void* d_out, int out_type, size_t num_elements,
                                 void* d_workspace, size_t workspace_bytes, void* stream);
int tcu_full_reduce_bf16(const void* d_in, float* d_out, double* d_out_f64, size_t num_elements,
                         int algo, void* d_workspace, size_t workspace_bytes, void* stream);
int tcu_full_scan_bf16(const void* d_in, void* d_out, int out_type, size_t num_elements,
                       const double* d_shard_totals, int shard_index, int algo,
                       void* d_workspace, size_t workspace_bytes, void* stream);
/* tcu_fill_f16 rounding the same values to bfloat16 instead. */
int tcu_fill_bf16(void* d_out, size_t n, uint64_t seed, uint64_t first_index, int dist,
                  void* stream);

/*
 * tcu_full_scan_f16 for callers that must not allocate device memory.  It has
 * no counterpart in the reference, whose drivers cudaMalloc whatever they need.
 *
 * Who needs it: code that runs where cudaMalloc / cudaFree are off limits or
 * too expensive -- a plugin that was handed its input and output buffers and
 * nothing else by a host framework that owns all device memory, a service
 * loop with a latency budget (cudaMalloc and cudaFree synchronise the whole
 * device), or a step that sits between other asynchronous work and must not
 * stall it.  Such a caller cannot produce the workspace tcu_full_scan_f16 asks
 * for, so this variant brings its own: a fixed array in the library's device
 * image, TCU_STATIC_SCAN_SCRATCH_BYTES (about 0.8 MiB) on every GPU the
 * library is loaded on, held until the process exits.
 *
 * Same arguments and results as tcu_full_scan_f16 minus the workspace.  Limits
 * and rules that come with the shared array:
 *   - num_elements <= TCU_STATIC_SCAN_MAX_ELEMENTS (2^30), else TCU_ERR_TOO_LARGE
 *     and nothing is launched;
 *   - the first call on each device looks up the array's device address (with
 *     that device current); make that first call outside any stream capture;
 *   - every call uses the same array and clears the part it needs on `stream`
 *     before its kernel, so calls in one stream are fine back to back, but two
 *     calls that can run at the same time on one GPU (different streams,
 *     different host threads) race on it: serialise them, or give the second
 *     one a workspace and use tcu_full_scan_f16;
 *   - no cudaMalloc, cudaFree or allocating library routine is called.
 */
#define TCU_STATIC_SCAN_MAX_ELEMENTS ((size_t)1 << 30)
#define TCU_STATIC_SCAN_MAX_TILES (TCU_STATIC_SCAN_MAX_ELEMENTS / 16384)
#define TCU_STATIC_SCAN_SCRATCH_BYTES \
  (256 + TCU_STATIC_SCAN_MAX_TILES * 8 + (TCU_STATIC_SCAN_MAX_TILES / 32 + TCU_STATIC_SCAN_MAX_TILES / 2 + 2) * 8)
int tcu_full_scan_f16_static(const void* d_in, void* d_out, int out_type, size_t num_elements,
                             const double* d_shard_totals, int shard_index, int algo,
                             void* stream);

/* Bytes of device workspace the operation needs (0 = none).  The workspace
 * needs no initialisation; one workspace must not be shared by calls that can
 * run at the same time. */
size_t tcu_workspace_bytes(int op, size_t num_elements, size_t segment_size);

/*
 * Seeded input fill, element i = f(seed, first_index + i): the build's
 * replacement for cuda_memory_set / setFP16 (src/utils/cuda_helpers.cuh:123-181).
 * Shards of one logical array are filled independently by passing their
 * first global index.  n must be a multiple of 8.
 */
int tcu_fill_f16(void* d_out, size_t n, uint64_t seed, uint64_t first_index, int dist,
                 void* stream);

/*
 * Same operations with HOST buffers: input is copied to the device in chunks
 * of whole segments that overlap with the kernels, results are copied back.
 * h_in / h_out should be pinned for full copy bandwidth.  The context owns
 * its staging buffers and streams (created once; this is the only place the
 * library allocates).  op selects the operation; for the full operations
 * segment_size is ignored.  The call returns when h_out is complete.
 */
typedef struct tcu_host_ctx tcu_host_ctx;
int tcu_host_ctx_create(tcu_host_ctx** ctx, size_t chunk_elements);
void tcu_host_ctx_destroy(tcu_host_ctx* ctx);
int tcu_host_run_f16(tcu_host_ctx* ctx, int op, const void* h_in, void* h_out, int out_type,
                     size_t num_elements, size_t segment_size, int algo);

/*
 * The reference's segment-size sweep (one array, many segment sizes:
 * SEG_16_ARGS ... SEG_16384_ARGS over the same element counts,
 * src/reduction/args.hpp:64-75) for an array in HOST memory: every chunk is
 * copied to the device once and reduced at all num_sizes segment sizes while
 * the next chunk is on its way; h_outs[i] receives num_elements /
 * segment_sizes[i] sums.  Saves num_sizes - 1 of num_sizes host-to-device
 * passes compared with num_sizes calls of tcu_host_run_f16.
 */
int tcu_host_segmented_reduce_sweep_f16(tcu_host_ctx* ctx, const void* h_in, size_t num_elements,
                                        int num_sizes, const size_t* segment_sizes,
                                        void* const* h_outs, int out_type, int algo);

/*
 * Full reduction and full scan of ONE array sharded contiguously over the GPUs
 * of a node: rank r holds elements [begin_r, end_r) in its own device memory
 * and keeps its part of the output.  The reference is single-device
 * (src/init/cuda.cpp:45 selects one GPU and nothing in src/ talks to another),
 * so these entry points have no counterpart there; they are what its full
 * operations (src/reduction/wmma_2kers.cu:65-81, src/prefixsum/wmma_3kers.cu:63-70)
 * become when the array does not live on one GPU.
 *
 * One context per GPU.  The GPUs exchange one double each per call -- the
 * shard totals -- which the reduction kernel's last thread block stores
 * straight into a small slot array in every rank's memory; the scan kernel of
 * rank r waits (bounded) for the totals of ranks < r in its own memory.  No
 * library collective runs per call.  Set-up:
 *   - one process per GPU: every rank calls tcu_mgpu_ctx_create, which fills
 *     handle_out (TCU_MGPU_HANDLE_BYTES bytes, a CUDA IPC handle of its slot
 *     array); the ranks exchange the handles by any means they have (one
 *     all-gather at start-up) and pass all of them, in rank order, to
 *     tcu_mgpu_ctx_connect;
 *   - one process driving several devices: create one context per device (with
 *     that device current; handle_out may be NULL) and call
 *     tcu_mgpu_ctx_connect_local on each with the array of all contexts.
 * Rules: every rank makes the same sequence of tcu_mgpu_full_* calls, each on
 * one stream of its own GPU, and the calls of one context do not overlap;
 * a rank whose peers never make the matching call gives up after about two
 * seconds and reports TCU_ERR_TIMEOUT through tcu_device_error (bit 2).
 * Destroy a context only after EVERY rank has finished its last call
 * (synchronise, then meet at a host barrier): peers store into its memory.
 *
 * tcu_mgpu_full_reduce_f16: *d_out (and *d_out_f64 if not NULL) receive the
 * sum over all ranks' shards, on every rank.
 * tcu_mgpu_full_scan_f16: d_out[i] = (sum of all earlier ranks' shards) +
 * in[0] + ... + in[i]; two passes over the shard (reduce, then scan).
 * num_elements: this rank's shard, a multiple of 16, may be 0.
 * tcu_mgpu_ctx_set_l2_keep_bytes: how much of the shard the first pass asks
 * L2 to keep for the second (default 64 MiB; 0 = nothing).
 */
#define TCU_MGPU_HANDLE_BYTES 64
#define TCU_MGPU_MAX_RANKS 16
typedef struct tcu_mgpu_ctx tcu_mgpu_ctx;
int tcu_mgpu_ctx_create(tcu_mgpu_ctx** ctx, int rank, int world, void* handle_out);
int tcu_mgpu_ctx_connect(tcu_mgpu_ctx* ctx, const void* handles);
int tcu_mgpu_ctx_connect_local(tcu_mgpu_ctx* ctx, tcu_mgpu_ctx* const* group);
int tcu_mgpu_ctx_set_l2_keep_bytes(tcu_mgpu_ctx* ctx, size_t bytes);
void tcu_mgpu_ctx_destroy(tcu_mgpu_ctx* ctx);
int tcu_mgpu_full_reduce_f16(tcu_mgpu_ctx* ctx, const void* d_in, float* d_out, double* d_out_f64,
                             size_t num_elements, void* stream);
int tcu_mgpu_full_scan_f16(tcu_mgpu_ctx* ctx, const void* d_in, void* d_out, int out_type,
                           size_t num_elements, void* stream);

/* Reads (and optionally clears) the device-side error word of the current
 * device: bit 0 = an mbarrier wait ran out, bit 1 = a tile-status poll ran
 * out, bit 2 = a wait for another GPU's total ran out.  Synchronises the
 * device.  Returns TCU_ERR_TIMEOUT if any bit is set. */
int tcu_device_error(unsigned int* bits, int clear);

/*
 * Test hooks for the bounded waits (the reference has none: its one
 * device-side spin barrier is disabled as a dead lock,
 * src/prefixsum/wmma_atomic.cu:189).  Every device-side wait of the library
 * gives up after a limit and raises a bit of the error word instead of
 * hanging; these two calls let a test see that happen within a millisecond.
 * tcu_test_set_wait_limits: attempts before an mbarrier wait, a tile-status
 * poll, a shared-memory flag poll and a peer-total poll give up, on the
 * current device; 0 restores that limit's default.
 * tcu_test_inject: arms ONE stall for the next matching call on this host
 * thread's library state -- TCU_TEST_SKIP_TILE_LOAD: the next segmented or
 * full reduction never loads tile `arg` of CTA 0's tiles (its consumers'
 * barrier is never armed); TCU_TEST_LOOKBACK_TICKET: the next look-back scan
 * hands out tiles starting at `arg` instead of 0 (tile `arg` polls status
 * words nobody publishes).  Nothing faults or traps: the waits run out, the
 * kernels return, the outputs of that call are wrong and flagged.
 */
typedef enum { TCU_TEST_NONE = 0, TCU_TEST_SKIP_TILE_LOAD = 1, TCU_TEST_LOOKBACK_TICKET = 2 } tcu_test_stall;
int tcu_test_set_wait_limits(unsigned barrier_attempts, unsigned status_polls, unsigned flag_polls,
                             unsigned peer_polls);
int tcu_test_inject(int what, unsigned long long arg);

/* Geometry the kernels were built with, for callers that size experiments. */
int tcu_tile_elements(void);
int tcu_num_sms(void);

const char* tcu_status_string(int status);

#ifdef __cplusplus
}
#endif
#endif /* TCU_SCOPE_H_ */
