// Multi-GPU entry points: full reduction and full scan of an array sharded
// contiguously over the GPUs of one node, one context per GPU (one process per
// GPU, or one process driving several devices).  The only thing the GPUs
// exchange is one double each, stored by the kernels themselves into small slot
// arrays that every rank maps from every other rank (see shard_kernels.cuh);
// the contexts own those arrays, which is the one allocation this file makes,
// once, at set-up.

struct tcu_mgpu_ctx {
  int rank, world, device;
  uint8_t* local;                        // this rank's block: slots | counters | per-CTA totals
  void* peers[tcu::kMaxRanks];           // slot arrays of all ranks, as mapped here
  bool opened[tcu::kMaxRanks];           // mapped through an IPC handle (to be closed)
  bool connected;
  size_t l2_keep_bytes;
};

namespace {

constexpr size_t kMgpuSlotBytes    = size_t(tcu::kSlotEpochs) * tcu::kMaxRanks * sizeof(tcu::PeerSlot);
constexpr size_t kMgpuCounterOff   = 1024;  // CTAs done with pass 1 (wraps to zero by itself)
constexpr size_t kMgpuSeqOff       = 1032;  // calls made so far (advanced by pass 1)
constexpr size_t kMgpuCtaTotalsOff = 2048;
constexpr int kMaxShardGrid        = 1024;
constexpr size_t kMgpuBlockBytes   = kMgpuCtaTotalsOff + size_t(kMaxShardGrid) * 8;
constexpr size_t kDefaultL2Keep    = size_t(64) << 20;
static_assert(kMgpuSlotBytes <= kMgpuCounterOff, "slots overlap the counter");
static_assert(sizeof(cudaIpcMemHandle_t) == TCU_MGPU_HANDLE_BYTES, "handle size");
static_assert(tcu::kMaxRanks == TCU_MGPU_MAX_RANKS, "rank limit");

template <typename... Args>
cudaError_t launch_pdl_n(void (*kernel)(Args...), int grid, int threads, size_t smem,
                         cudaStream_t st, Args... args) {
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
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <bool OUT32>
cudaError_t launch_shard_scan(const tcu::ShardParams& p, int grid, cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e = ensure_smem(tcu::shard_scan_kernel<OUT32>, configured, kDynSmemBytes);
  if (e != cudaSuccess) return e;
  return launch_pdl_n(tcu::shard_scan_kernel<OUT32>, grid, tcu::kThreads, size_t(kDynSmemBytes), st, p);
}

// Fills the parts of ShardParams both passes share.
int shard_params(tcu_mgpu_ctx* c, const void* d_in, size_t n, tcu::ShardParams* p, int* grid) {
  if (!c || !c->connected) return TCU_ERR_INVALID_ARG;
  if (n % 16 != 0 || (n != 0 && (!d_in || !aligned16(d_in)))) return TCU_ERR_INVALID_ARG;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != c->device) return TCU_ERR_INVALID_ARG;
  const int sms = sm_count();
  if (sms <= 0) return TCU_ERR_CUDA;
  const size_t tiles = (n + tcu::kTileElems - 1) / tcu::kTileElems;
  int g              = tiles < size_t(sms) ? int(tiles) : sms;
  if (g < 1) g = 1;  // an empty shard still has a total to publish
  if (g > kMaxShardGrid) g = kMaxShardGrid;
  *grid = g;
  *p    = tcu::ShardParams{};
  p->in           = static_cast<const uint8_t*>(d_in);
  p->num_elems    = n;
  p->keep_tiles   = int(c->l2_keep_bytes / (size_t(g) * tcu::kTileBytes));
  p->cta_total    = reinterpret_cast<double*>(c->local + kMgpuCtaTotalsOff);
  p->done_counter = reinterpret_cast<unsigned int*>(c->local + kMgpuCounterOff);
  for (int r = 0; r < c->world; ++r) p->x.slots[r] = static_cast<tcu::PeerSlot*>(c->peers[r]);
  p->x.rank        = c->rank;
  p->x.world       = c->world;
  p->x.seq_counter = reinterpret_cast<unsigned long long*>(c->local + kMgpuSeqOff);
  return TCU_OK;
}

cudaError_t launch_shard_reduce(const tcu::ShardParams& p, int grid, cudaStream_t st) {
  static bool configured[kMaxDevices];
  cudaError_t e = ensure_smem(tcu::shard_reduce_kernel, configured, kDynSmemBytes);
  if (e != cudaSuccess) return e;
  return launch_pdl_n(tcu::shard_reduce_kernel, grid, tcu::kThreads, size_t(kDynSmemBytes), st, p);
}

void mgpu_ctx_free(tcu_mgpu_ctx* c) {
  if (!c) return;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(c->device);
  for (int r = 0; r < tcu::kMaxRanks; ++r)
    if (c->opened[r] && c->peers[r]) cudaIpcCloseMemHandle(c->peers[r]);
  if (c->local) cudaFree(c->local);
  if (prev >= 0) cudaSetDevice(prev);
  delete c;
}

}  // namespace

extern "C" {

int tcu_mgpu_ctx_create(tcu_mgpu_ctx** out, int rank, int world, void* handle_out) {
  if (!out) return TCU_ERR_INVALID_ARG;
  *out = nullptr;
  if (world < 1 || world > tcu::kMaxRanks || rank < 0 || rank >= world) return TCU_ERR_INVALID_ARG;
  const int dev = current_device();
  if (dev < 0) return TCU_ERR_CUDA;
  tcu_mgpu_ctx* c = new (std::nothrow) tcu_mgpu_ctx();
  if (!c) return TCU_ERR_CUDA;
  c->rank          = rank;
  c->world         = world;
  c->device        = dev;
  c->l2_keep_bytes = kDefaultL2Keep;
  bool ok = cudaMalloc(reinterpret_cast<void**>(&c->local), kMgpuBlockBytes) == cudaSuccess;
  ok      = ok && cudaMemset(c->local, 0, kMgpuBlockBytes) == cudaSuccess;
  ok      = ok && cudaDeviceSynchronize() == cudaSuccess;
  if (ok && handle_out) {
    cudaIpcMemHandle_t h;
    ok = cudaIpcGetMemHandle(&h, c->local) == cudaSuccess;
    if (ok) std::memcpy(handle_out, &h, sizeof(h));
  }
  if (!ok) {
    cudaGetLastError();
    mgpu_ctx_free(c);
    return TCU_ERR_CUDA;
  }
  c->peers[rank] = c->local;
  if (world == 1) c->connected = true;
  *out = c;
  return TCU_OK;
}

int tcu_mgpu_ctx_connect(tcu_mgpu_ctx* c, const void* handles) {
  if (!c || !handles) return TCU_ERR_INVALID_ARG;
  if (c->connected) return TCU_OK;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != c->device) return TCU_ERR_INVALID_ARG;
  const uint8_t* h = static_cast<const uint8_t*>(handles);
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t handle;
    std::memcpy(&handle, h + size_t(r) * TCU_MGPU_HANDLE_BYTES, sizeof(handle));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || !p) {
      cudaGetLastError();
      return TCU_ERR_CUDA;
    }
    c->peers[r]  = p;
    c->opened[r] = true;
  }
  c->connected = true;
  return TCU_OK;
}

int tcu_mgpu_ctx_connect_local(tcu_mgpu_ctx* c, tcu_mgpu_ctx* const* group) {
  if (!c || !group) return TCU_ERR_INVALID_ARG;
  if (c->connected) return TCU_OK;
  int prev = -1;
  if (cudaGetDevice(&prev) != cudaSuccess) return TCU_ERR_CUDA;
  if (cudaSetDevice(c->device) != cudaSuccess) return TCU_ERR_CUDA;
  int status = TCU_OK;
  for (int r = 0; r < c->world && status == TCU_OK; ++r) {
    const tcu_mgpu_ctx* o = group[r];
    if (!o || o->rank != r || o->world != c->world) {
      status = TCU_ERR_INVALID_ARG;
      break;
    }
    if (o->device != c->device) {
      const cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) status = TCU_ERR_CUDA;
      cudaGetLastError();
    }
    c->peers[r] = o->local;
  }
  cudaSetDevice(prev);
  if (status == TCU_OK) c->connected = true;
  return status;
}

int tcu_mgpu_ctx_set_l2_keep_bytes(tcu_mgpu_ctx* c, size_t bytes) {
  if (!c) return TCU_ERR_INVALID_ARG;
  c->l2_keep_bytes = bytes;
  return TCU_OK;
}

void tcu_mgpu_ctx_destroy(tcu_mgpu_ctx* c) { mgpu_ctx_free(c); }

int tcu_mgpu_full_reduce_f16(tcu_mgpu_ctx* c, const void* d_in, float* d_out, double* d_out_f64,
                             size_t num_elements, void* stream) {
  if (!d_out || (reinterpret_cast<uintptr_t>(d_out) & 3u) != 0) return TCU_ERR_INVALID_ARG;
  if (d_out_f64 && (reinterpret_cast<uintptr_t>(d_out_f64) & 7u) != 0) return TCU_ERR_INVALID_ARG;
  tcu::ShardParams p;
  int grid         = 0;
  const int status = shard_params(c, d_in, num_elements, &p, &grid);
  if (status != TCU_OK) return status;
  p.keep_tiles = 0;  // nothing reads the shard again
  p.total_f32  = d_out;
  p.total_f64  = d_out_f64;
  p.wait_all   = 1;
  return launch_shard_reduce(p, grid, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? TCU_OK
             : TCU_ERR_CUDA;
}

int tcu_mgpu_full_scan_f16(tcu_mgpu_ctx* c, const void* d_in, void* d_out, int out_type,
                           size_t num_elements, void* stream) {
  if (out_type != TCU_OUT_F16 && out_type != TCU_OUT_F32) return TCU_ERR_UNSUPPORTED;
  if (num_elements != 0 && (!d_out || !aligned16(d_out))) return TCU_ERR_INVALID_ARG;
  tcu::ShardParams p;
  int grid         = 0;
  const int status = shard_params(c, d_in, num_elements, &p, &grid);
  if (status != TCU_OK) return status;
  p.out        = d_out;
  p.out_is_f32 = out_type == TCU_OUT_F32;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (launch_shard_reduce(p, grid, st) != cudaSuccess) return TCU_ERR_CUDA;
  if (num_elements == 0) return TCU_OK;
  const cudaError_t e = out_type == TCU_OUT_F32 ? launch_shard_scan<true>(p, grid, st)
                                                : launch_shard_scan<false>(p, grid, st);
  return e == cudaSuccess ? TCU_OK : TCU_ERR_CUDA;
}

}  // extern "C"
