// Host-buffer entry points: the same four operations for callers whose data
// lives in host memory.  The input is cut into chunks of whole segments; two
// streams alternate so that the copy of one chunk overlaps the kernel and the
// copy-back of the other.  This is the only part of the library that owns
// device memory, and it allocates it once, in tcu_host_ctx_create.

struct tcu_host_ctx {
  size_t chunk_elems;
  void* d_in[2];
  void* d_out[2];
  void* d_ws[2];
  size_t ws_bytes;
  cudaStream_t st[2];
  cudaEvent_t ev_total[2];
  double* d_totals;   // per-chunk totals (full reduce / full scan)
  float* d_scratch;   // per-chunk float results nobody reads
  double* h_totals;   // pinned
  size_t max_chunks;
};

namespace {

constexpr size_t kHostMaxChunks = 1 << 16;

void host_ctx_free(tcu_host_ctx* c) {
  if (!c) return;
  for (int k = 0; k < 2; ++k) {
    if (c->d_in[k]) cudaFree(c->d_in[k]);
    if (c->d_out[k]) cudaFree(c->d_out[k]);
    if (c->d_ws[k]) cudaFree(c->d_ws[k]);
    if (c->st[k]) cudaStreamDestroy(c->st[k]);
    if (c->ev_total[k]) cudaEventDestroy(c->ev_total[k]);
  }
  if (c->d_totals) cudaFree(c->d_totals);
  if (c->d_scratch) cudaFree(c->d_scratch);
  if (c->h_totals) cudaFreeHost(c->h_totals);
  delete c;
}

}  // namespace

extern "C" {

int tcu_host_ctx_create(tcu_host_ctx** out, size_t chunk_elements) {
  if (!out) return TCU_ERR_INVALID_ARG;
  *out = nullptr;
  if (chunk_elements < size_t(tcu::kTileElems)) chunk_elements = tcu::kTileElems;
  chunk_elements = (chunk_elements + tcu::kTileElems - 1) / tcu::kTileElems * tcu::kTileElems;
  tcu_host_ctx* c = new (std::nothrow) tcu_host_ctx();
  if (!c) return TCU_ERR_CUDA;
  c->chunk_elems = chunk_elements;
  c->max_chunks  = kHostMaxChunks;
  const size_t ws_scan = scan_long_ws_bytes(chunk_elements), ws_red = reduce_long_ws_bytes();
  c->ws_bytes          = ws_scan > ws_red ? ws_scan : ws_red;
  bool ok              = true;
  for (int k = 0; k < 2 && ok; ++k) {
    ok = ok && cudaMalloc(&c->d_in[k], chunk_elements * 2) == cudaSuccess;
    ok = ok && cudaMalloc(&c->d_out[k], chunk_elements * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&c->d_ws[k], c->ws_bytes) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&c->st[k], cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&c->ev_total[k], cudaEventDisableTiming) == cudaSuccess;
  }
  ok = ok && cudaMalloc(reinterpret_cast<void**>(&c->d_totals), c->max_chunks * 8) == cudaSuccess;
  ok = ok && cudaMalloc(reinterpret_cast<void**>(&c->d_scratch), c->max_chunks * 4) == cudaSuccess;
  ok = ok && cudaMallocHost(reinterpret_cast<void**>(&c->h_totals), c->max_chunks * 8) == cudaSuccess;
  if (!ok) {
    host_ctx_free(c);
    return TCU_ERR_CUDA;
  }
  *out = c;
  return TCU_OK;
}

void tcu_host_ctx_destroy(tcu_host_ctx* ctx) { host_ctx_free(ctx); }

int tcu_host_run_f16(tcu_host_ctx* c, int op, const void* h_in, void* h_out, int out_type,
                     size_t num_elements, size_t segment_size, int algo) {
  if (!c || !h_in || !h_out) return TCU_ERR_INVALID_ARG;
  if (out_type != TCU_OUT_F16 && out_type != TCU_OUT_F32) return TCU_ERR_UNSUPPORTED;
  const bool segmented = op == TCU_OP_SEGMENTED_REDUCE || op == TCU_OP_SEGMENTED_SCAN;
  if (!segmented && op != TCU_OP_FULL_REDUCE && op != TCU_OP_FULL_SCAN) return TCU_ERR_UNSUPPORTED;
  if (num_elements == 0) return segmented ? TCU_OK : TCU_ERR_INVALID_ARG;
  size_t chunk = c->chunk_elems;
  if (segmented) {
    if (segment_class(segment_size) < 0) return TCU_ERR_UNSUPPORTED;
    if (num_elements % segment_size != 0) return TCU_ERR_INVALID_ARG;
    if (segment_size > chunk) return TCU_ERR_UNSUPPORTED;  // a segment must fit one staging buffer
    chunk = chunk / segment_size * segment_size;
  } else {
    if (num_elements % 16 != 0) return TCU_ERR_INVALID_ARG;
    if (op == TCU_OP_FULL_REDUCE) out_type = TCU_OUT_F32;
  }
  const size_t num_chunks = (num_elements + chunk - 1) / chunk;
  if (!segmented && num_chunks > c->max_chunks) return TCU_ERR_UNSUPPORTED;
  const size_t out_elem = out_type == TCU_OUT_F32 ? 4 : 2;
  const uint8_t* src    = static_cast<const uint8_t*>(h_in);
  uint8_t* dst          = static_cast<uint8_t*>(h_out);

  int status = TCU_OK;
  for (size_t ci = 0; ci < num_chunks && status == TCU_OK; ++ci) {
    const int k         = int(ci & 1);
    const size_t first  = ci * chunk;
    const size_t elems  = num_elements - first < chunk ? num_elements - first : chunk;
    cudaStream_t st     = c->st[k];
    if (cudaMemcpyAsync(c->d_in[k], src + first * 2, elems * 2, cudaMemcpyHostToDevice, st) !=
        cudaSuccess) {
      status = TCU_ERR_CUDA;
      break;
    }
    switch (op) {
      case TCU_OP_SEGMENTED_REDUCE: {
        const size_t segs = elems / segment_size;
        status = tcu_segmented_reduce_f16(c->d_in[k], c->d_out[k], out_type, segs, segment_size,
                                          algo, c->d_ws[k], c->ws_bytes, st);
        if (status == TCU_OK &&
            cudaMemcpyAsync(dst + first / segment_size * out_elem, c->d_out[k], segs * out_elem,
                            cudaMemcpyDeviceToHost, st) != cudaSuccess)
          status = TCU_ERR_CUDA;
        break;
      }
      case TCU_OP_SEGMENTED_SCAN: {
        status = tcu_segmented_scan_f16(c->d_in[k], c->d_out[k], out_type, elems / segment_size,
                                        segment_size, algo, c->d_ws[k], c->ws_bytes, st);
        if (status == TCU_OK &&
            cudaMemcpyAsync(dst + first * out_elem, c->d_out[k], elems * out_elem,
                            cudaMemcpyDeviceToHost, st) != cudaSuccess)
          status = TCU_ERR_CUDA;
        break;
      }
      case TCU_OP_FULL_REDUCE:
        status = tcu_full_reduce_f16(c->d_in[k], c->d_scratch + ci, c->d_totals + ci, elems, algo,
                                     c->d_ws[k], c->ws_bytes, st);
        break;
      case TCU_OP_FULL_SCAN: {
        // total of this chunk first: the next chunk's scan (on the other
        // stream) needs it, and this chunk's scan needs the previous one's
        status = tcu_full_reduce_f16(c->d_in[k], c->d_scratch + ci, c->d_totals + ci, elems, algo,
                                     c->d_ws[k], c->ws_bytes, st);
        if (status != TCU_OK) break;
        if (cudaEventRecord(c->ev_total[k], st) != cudaSuccess ||
            (ci > 0 && cudaStreamWaitEvent(st, c->ev_total[k ^ 1], 0) != cudaSuccess)) {
          status = TCU_ERR_CUDA;
          break;
        }
        status = tcu_full_scan_f16(c->d_in[k], c->d_out[k], out_type, elems, c->d_totals, int(ci),
                                   algo == TCU_ALGO_SHUFFLE ? TCU_ALGO_MMA : algo, c->d_ws[k],
                                   c->ws_bytes, st);
        if (status == TCU_OK &&
            cudaMemcpyAsync(dst + first * out_elem, c->d_out[k], elems * out_elem,
                            cudaMemcpyDeviceToHost, st) != cudaSuccess)
          status = TCU_ERR_CUDA;
        break;
      }
      default: status = TCU_ERR_UNSUPPORTED;
    }
  }
  // drain both streams even after an error: the staging buffers are reused
  const bool s0 = cudaStreamSynchronize(c->st[0]) == cudaSuccess;
  const bool s1 = cudaStreamSynchronize(c->st[1]) == cudaSuccess;
  if (status != TCU_OK) return status;
  if (!s0 || !s1) return TCU_ERR_CUDA;

  if (op == TCU_OP_FULL_REDUCE) {
    if (cudaMemcpy(c->h_totals, c->d_totals, num_chunks * 8, cudaMemcpyDeviceToHost) != cudaSuccess)
      return TCU_ERR_CUDA;
    double total = 0.0;
    for (size_t ci = 0; ci < num_chunks; ++ci) total += c->h_totals[ci];
    *static_cast<float*>(h_out) = static_cast<float>(total);
  }
  return TCU_OK;
}

int tcu_host_segmented_reduce_sweep_f16(tcu_host_ctx* c, const void* h_in, size_t num_elements,
                                        int num_sizes, const size_t* segment_sizes,
                                        void* const* h_outs, int out_type, int algo) {
  if (!c || !h_in || !segment_sizes || !h_outs || num_sizes <= 0 || num_sizes > 32)
    return TCU_ERR_INVALID_ARG;
  if (out_type != TCU_OUT_F16 && out_type != TCU_OUT_F32) return TCU_ERR_UNSUPPORTED;
  if (num_elements == 0) return TCU_OK;
  // every chunk must hold whole segments of EVERY size: a multiple of their least common
  // multiple (for the powers of two of the reference's sweep that is the largest size)
  size_t unit = 1;
  for (int i = 0; i < num_sizes; ++i) {
    if (!h_outs[i]) return TCU_ERR_INVALID_ARG;
    if (segment_class(segment_sizes[i]) < 0) return TCU_ERR_UNSUPPORTED;
    if (num_elements % segment_sizes[i] != 0) return TCU_ERR_INVALID_ARG;
    size_t a = unit, b = segment_sizes[i];
    while (b != 0) {
      const size_t r = a % b;
      a = b;
      b = r;
    }
    const size_t step = segment_sizes[i] / a;  // unit * step = lcm(unit, size)
    if (step > c->chunk_elems / unit) return TCU_ERR_UNSUPPORTED;  // no chunk holds whole segments of all sizes
    unit *= step;
  }
  const size_t chunk    = c->chunk_elems / unit * unit;
  const size_t out_elem = out_type == TCU_OUT_F32 ? 4 : 2;
  // all outputs of one chunk share the staging buffer (chunk * 4 bytes): with every
  // size >= 16 and at most 32 sizes they need at most 32 * chunk/16 * 4 bytes -- check anyway
  size_t need = 0;
  for (int i = 0; i < num_sizes; ++i) need += (chunk / segment_sizes[i] * out_elem + 255) / 256 * 256;
  if (need > c->chunk_elems * 4) return TCU_ERR_UNSUPPORTED;
  const uint8_t* src = static_cast<const uint8_t*>(h_in);
  const size_t num_chunks = (num_elements + chunk - 1) / chunk;
  int status = TCU_OK;
  for (size_t ci = 0; ci < num_chunks && status == TCU_OK; ++ci) {
    const int k        = int(ci & 1);
    const size_t first = ci * chunk;
    const size_t elems = num_elements - first < chunk ? num_elements - first : chunk;
    cudaStream_t st    = c->st[k];
    if (cudaMemcpyAsync(c->d_in[k], src + first * 2, elems * 2, cudaMemcpyHostToDevice, st) !=
        cudaSuccess) {
      status = TCU_ERR_CUDA;
      break;
    }
    size_t off = 0;
    for (int i = 0; i < num_sizes && status == TCU_OK; ++i) {
      const size_t s = segment_sizes[i], segs = elems / s;
      uint8_t* d_out = static_cast<uint8_t*>(c->d_out[k]) + off;
      status = tcu_segmented_reduce_f16(c->d_in[k], d_out, out_type, segs, s, algo, c->d_ws[k],
                                        c->ws_bytes, st);
      if (status == TCU_OK &&
          cudaMemcpyAsync(static_cast<uint8_t*>(h_outs[i]) + first / s * out_elem, d_out,
                          segs * out_elem, cudaMemcpyDeviceToHost, st) != cudaSuccess)
        status = TCU_ERR_CUDA;
      off += (chunk / s * out_elem + 255) / 256 * 256;
    }
  }
  const bool s0 = cudaStreamSynchronize(c->st[0]) == cudaSuccess;
  const bool s1 = cudaStreamSynchronize(c->st[1]) == cudaSuccess;
  if (status != TCU_OK) return status;
  return s0 && s1 ? TCU_OK : TCU_ERR_CUDA;
}


}  // extern "C"
