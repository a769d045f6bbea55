// C ABI of the stand-alone quantised weight: upload, read-back, dequantise, product. The
// counterpart of ferrum_wgpu::ops::quant's public functions (ferrum_wgpu/src/ops/quant.rs).
#include "common.cuh"

int k_qgemm_tc(FcDevice* dev, FcQWeight* w, const float* x_dev, uint32_t m, float* y_dev); // model_tc.cu
int tc_check_errors(FcDevice* dev);                                                            // gemm_tc.cu

FC_API size_t fc_block_bytes(int kind, size_t n_elems) {
  if (kind == FC_F32) return n_elems * 4;
  if (kind == FC_Q2_K) return n_elems % QK_K ? 0 : n_elems / QK_K * 84;
  if (n_elems % QK) return 0;
  if (kind_byte_blocks(kind)) return n_elems / QK * 34;
  if (kind == FC_Q4_0) return n_elems / QK * 18;
  if (kind == FC_MXFP4) return n_elems / QK * 17;
  if (kind == FC_F16) return n_elems * 2;
  return 0;
}

FC_API int fc_qweight_create(FcDevice* dev, int kind, const float* w_in_out, uint32_t k, uint32_t n, FcQWeight** out) {
  if (!dev || !out) return FC_ERR_ARG;
  *out = nullptr;
  cudaSetDevice(dev->ordinal);
  if (!w_in_out) return fc_fail(dev, FC_ERR_ARG, "fc_qweight_create: NULL weights");
  if (!kind_known(kind)) return fc_fail(dev, FC_ERR_ARG, "unknown weight kind %d", kind);
  if (k == 0 || n == 0 || (kind != FC_F32 && k % QK))
    return fc_fail(dev, FC_ERR_SHAPE, "cannot quantise %llu elements as a %u x %u weight in whole 32-blocks",
                   (unsigned long long)k * n, k, n);
  return qweight_from_f32(dev, kind, w_in_out, k, n, out);
}

FC_API int fc_qweight_create_from_blocks(FcDevice* dev, int kind, const uint8_t* blocks, size_t n_bytes, uint32_t k,
                                         uint32_t n, FcQWeight** out) {
  if (!dev || !out) return FC_ERR_ARG;
  *out = nullptr;
  cudaSetDevice(dev->ordinal);
  if (!blocks) return fc_fail(dev, FC_ERR_ARG, "fc_qweight_create_from_blocks: NULL blocks");
  if (!kind_known(kind) || kind == FC_F32) return fc_fail(dev, FC_ERR_ARG, "block upload takes a block format or F16, not kind %d", kind);
  if (k == 0 || n == 0 || k % kind_block_elems(kind))
    return fc_fail(dev, FC_ERR_SHAPE, "a %u x %u weight is not whole %u-element blocks", k, n, kind_block_elems(kind));
  const size_t want = fc_block_bytes(kind, (size_t)k * n);
  if (n_bytes != want)
    return fc_fail(dev, FC_ERR_SHAPE, "%zu bytes is not the %zu a %u x %u weight needs", n_bytes, want, k, n);
  FcQWeight* w = new FcQWeight();
  w->dev = dev;
  const size_t qs_bytes = qmat_qs_bytes(kind, k, n), sc_bytes = qmat_sc_bytes(kind, k, n);
  uint8_t* stage = nullptr;
  cudaError_t e = cudaMalloc(&w->qs_alloc, qs_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&w->sc_alloc, sc_bytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&stage, n_bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    qweight_free(w);
    if (stage) cudaFree(stage);
    return fc_fail(dev, FC_ERR_OOM, "cannot allocate a %u x %u weight: %s", k, n, cudaGetErrorString(e));
  }
  w->m.kind = kind, w->m.k = k, w->m.n = n;
  w->m.qs = (const uint8_t*)w->qs_alloc;
  w->m.sc = (const __half*)w->sc_alloc;
  w->bytes = qs_bytes + sc_bytes;
  int rc = FC_OK;
  if (cudaMemcpyAsync(stage, blocks, n_bytes, cudaMemcpyHostToDevice, dev->stream) != cudaSuccess)
    rc = fc_fail(dev, FC_ERR_DEVICE, "block upload failed");
  if (rc == FC_OK) rc = k_repack_blocks(dev, kind, stage, k, n, (uint8_t*)w->qs_alloc, (__half*)w->sc_alloc);
  if (rc == FC_OK && cudaStreamSynchronize(dev->stream) != cudaSuccess) {
    dev->lost = true;
    rc = fc_fail(dev, FC_ERR_DEVICE, "block repack failed: %s", cudaGetErrorString(cudaGetLastError()));
  }
  cudaFree(stage);
  if (rc != FC_OK) {
    qweight_free(w);
    return rc;
  }
  *out = w;
  return FC_OK;
}

FC_API int fc_qweight_destroy(FcQWeight* w) {
  if (!w) return FC_ERR_ARG;
  cudaSetDevice(w->dev->ordinal);
  cudaStreamSynchronize(w->dev->stream);
  if (w->tc_cache) cudaFree(w->tc_cache);
  if (w->mma_scratch) cudaFree(w->mma_scratch);
  qweight_free(w);
  return FC_OK;
}

FC_API int fc_qweight_info(const FcQWeight* w, int* kind, uint32_t* k, uint32_t* n, uint64_t* dev_bytes) {
  if (!w) return FC_ERR_ARG;
  if (kind) *kind = w->m.kind;
  if (k) *k = w->m.k;
  if (n) *n = w->m.n;
  if (dev_bytes) *dev_bytes = w->bytes;
  return FC_OK;
}

FC_API int fc_qweight_blocks(FcQWeight* w, uint8_t* out, size_t out_bytes) {
  if (!w || !out) return FC_ERR_ARG;
  FcDevice* dev = w->dev;
  cudaSetDevice(dev->ordinal);
  if (w->m.kind == FC_F32) return fc_fail(dev, FC_ERR_UNSUPPORTED, "an f32 weight has no block form");
  const size_t want = fc_block_bytes(w->m.kind, (size_t)w->m.k * w->m.n);
  if (out_bytes != want) return fc_fail(dev, FC_ERR_SHAPE, "output holds %zu bytes, the blocks are %zu", out_bytes, want);
  uint8_t* d = nullptr;
  FC_CUDA(dev, cudaMalloc((void**)&d, want));
  int rc = k_export_blocks(dev, w->m, d);
  if (rc == FC_OK && cudaMemcpyAsync(out, d, want, cudaMemcpyDeviceToHost, dev->stream) != cudaSuccess)
    rc = fc_fail(dev, FC_ERR_DEVICE, "block read-back failed");
  if (rc == FC_OK && cudaStreamSynchronize(dev->stream) != cudaSuccess) rc = fc_fail(dev, FC_ERR_DEVICE, "block read-back failed");
  cudaFree(d);
  return rc;
}

FC_API int fc_dequant(FcQWeight* w, float* out, size_t out_elems) {
  if (!w || !out) return FC_ERR_ARG;
  FcDevice* dev = w->dev;
  cudaSetDevice(dev->ordinal);
  const size_t want = (size_t)w->m.k * w->m.n;
  if (out_elems != want) return fc_fail(dev, FC_ERR_SHAPE, "output holds %zu elements, the weight has %zu", out_elems, want);
  float* d = nullptr;
  FC_CUDA(dev, cudaMalloc((void**)&d, want * 4));
  int rc = k_dequant(dev, w->m, d);
  if (rc == FC_OK && cudaMemcpyAsync(out, d, want * 4, cudaMemcpyDeviceToHost, dev->stream) != cudaSuccess)
    rc = fc_fail(dev, FC_ERR_DEVICE, "dequant read-back failed");
  if (rc == FC_OK && cudaStreamSynchronize(dev->stream) != cudaSuccess) rc = fc_fail(dev, FC_ERR_DEVICE, "dequant read-back failed");
  cudaFree(d);
  return rc;
}

FC_API int fc_qmatmul_dev(FcQWeight* w, const float* x_dev, uint32_t m, float* y_dev, int mode) {
  if (!w || !x_dev || !y_dev) return FC_ERR_ARG;
  FcDevice* dev = w->dev;
  // the kernels read x and write y in 16-byte pieces: a pointer into the middle of a buffer is refused here,
  // before any launch
  if ((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(y_dev)) & 15)
    return fc_fail(dev, FC_ERR_ARG, "x_dev and y_dev must be 16-byte aligned");
  cudaSetDevice(dev->ordinal);
  if (mode == FC_EXACT_F32) {
    Epilogue ep;
    if (qmatvec_mma_supports(w->m, m)) { // 1..64 rows: the decode tensor product needs scratch
      if (!w->mma_scratch) FC_CUDA(dev, cudaMalloc(&w->mma_scratch, qmatvec_mma_scratch_bytes(w->m.k, w->m.n)));
      ep.scratch = w->mma_scratch;
    }
    return k_qlinear_f32(dev, w->m, x_dev, m, y_dev, ep);
  }
  if (mode == FC_TENSOR_F16) return k_qgemm_tc(dev, w, x_dev, m, y_dev);
  return fc_fail(dev, FC_ERR_ARG, "unknown arithmetic mode %d", mode);
}

FC_API int fc_qmatmul(FcQWeight* w, const float* x, uint32_t m, float* y, int mode) {
  if (!w || !x || !y) return FC_ERR_ARG;
  FcDevice* dev = w->dev;
  cudaSetDevice(dev->ordinal);
  if (m == 0) return FC_OK;
  float *dx = nullptr, *dy = nullptr;
  cudaError_t e = cudaMalloc((void**)&dx, (size_t)m * w->m.k * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&dy, (size_t)m * w->m.n * 4);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (dx) cudaFree(dx);
    return fc_fail(dev, FC_ERR_OOM, "cannot allocate product buffers: %s", cudaGetErrorString(e));
  }
  int rc = FC_OK;
  if (cudaMemcpyAsync(dx, x, (size_t)m * w->m.k * 4, cudaMemcpyHostToDevice, dev->stream) != cudaSuccess)
    rc = fc_fail(dev, FC_ERR_DEVICE, "upload of x failed");
  if (rc == FC_OK) rc = fc_qmatmul_dev(w, dx, m, dy, mode);
  if (rc == FC_OK && mode == FC_TENSOR_F16) rc = tc_check_errors(dev);
  if (rc == FC_OK && cudaMemcpyAsync(y, dy, (size_t)m * w->m.n * 4, cudaMemcpyDeviceToHost, dev->stream) != cudaSuccess)
    rc = fc_fail(dev, FC_ERR_DEVICE, "read-back of y failed");
  if (rc == FC_OK && cudaStreamSynchronize(dev->stream) != cudaSuccess) {
    dev->lost = true;
    rc = fc_fail(dev, FC_ERR_DEVICE, "product failed: %s", cudaGetErrorString(cudaGetLastError()));
  }
  cudaFree(dx);
  cudaFree(dy);
  return rc;
}
