// Device handle, error reporting, launch accounting / host-side fault injection, weight upload.
// The CUDA counterpart of ferrum_wgpu::device (ferrum_wgpu/src/device/{mod,runtime,tensor}.rs):
// errors are values, a failed CUDA call makes the handle report "lost" from then on, and the
// fault hook refuses the k-th launch before it reaches the device.
#include <cstring>
#include <mutex>

#include "common.cuh"

static std::string g_no_device_error;
static std::mutex g_err_mutex;

int fc_fail(FcDevice* dev, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (dev) {
    dev->last_error = buf;
  } else {
    std::lock_guard<std::mutex> lock(g_err_mutex);
    g_no_device_error = buf;
  }
  return code;
}

int fc_pre_launch(FcDevice* dev, const char* what) {
  if (dev->lost) return fc_fail(dev, FC_ERR_DEVICE, "device lost: %s refused after an earlier CUDA failure", what);
  if (dev->fail_after == 0) return fc_fail(dev, FC_ERR_INJECTED, "injected fault: launch of %s refused", what);
  if (dev->fail_after > 0) dev->fail_after--;
  dev->launches++;
  if (dev->profiling) {
    FcDevice::ProfSpan s{what, nullptr, nullptr};
    for (cudaEvent_t* ev : {&s.t0, &s.t1}) {
      if (!dev->event_pool.empty()) {
        *ev = dev->event_pool.back();
        dev->event_pool.pop_back();
      } else if (cudaEventCreate(ev) != cudaSuccess) {
        return fc_fail(dev, FC_ERR_DEVICE, "cannot create a timing event");
      }
    }
    cudaEventRecord(s.t0, dev->stream);
    dev->spans.push_back(s);
  }
  return FC_OK;
}

int fc_post_launch(FcDevice* dev, const char* what) {
  if (dev->profiling && !dev->spans.empty()) cudaEventRecord(dev->spans.back().t1, dev->stream);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    dev->lost = true;
    return fc_fail(dev, FC_ERR_DEVICE, "launch of %s failed: %s", what, cudaGetErrorString(e));
  }
  return FC_OK;
}

int fc_pinned(FcDevice* dev, size_t bytes, void** out) {
  if (bytes > dev->pinned_bytes) {
    if (dev->pinned) {
      FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
      cudaFreeHost(dev->pinned);
      dev->pinned = nullptr;
      dev->pinned_bytes = 0;
    }
    size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
    FC_CUDA(dev, cudaMallocHost(&dev->pinned, want));
    dev->pinned_bytes = want;
  }
  *out = dev->pinned;
  return FC_OK;
}

FC_API int fc_device_open(int ordinal, FcDevice** out) {
  if (!out) return fc_fail(nullptr, FC_ERR_ARG, "fc_device_open: out is NULL");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return fc_fail(nullptr, FC_ERR_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  if (ordinal < 0 || ordinal >= count)
    return fc_fail(nullptr, FC_ERR_ARG, "no CUDA device %d (%d present)", ordinal, count);
  FcDevice* dev = new FcDevice();
  dev->ordinal = ordinal;
  if ((e = cudaSetDevice(ordinal)) != cudaSuccess || (e = cudaGetDeviceProperties(&dev->prop, ordinal)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&dev->stream, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaMalloc(&dev->d_flag, sizeof(int))) != cudaSuccess) {
    int rc = fc_fail(nullptr, FC_ERR_DEVICE, "cannot open CUDA device %d: %s", ordinal, cudaGetErrorString(e));
    delete dev;
    return rc;
  }
  if (dev->prop.major != 10) {
    int rc = fc_fail(nullptr, FC_ERR_UNSUPPORTED, "device %d (%s, sm_%d%d) is not sm_100: this library is built for B200 only",
                     ordinal, dev->prop.name, dev->prop.major, dev->prop.minor);
    cudaStreamDestroy(dev->stream);
    cudaFree(dev->d_flag);
    delete dev;
    return rc;
  }
  cudaMemsetAsync(dev->d_flag, 0, sizeof(int), dev->stream);
  *out = dev;
  return FC_OK;
}

FC_API int fc_device_close(FcDevice* dev) {
  if (!dev) return FC_ERR_ARG;
  cudaSetDevice(dev->ordinal);
  cudaStreamSynchronize(dev->stream);
  if (dev->pinned) cudaFreeHost(dev->pinned);
  if (dev->d_flag) cudaFree(dev->d_flag);
  for (auto& s : dev->spans) {
    cudaEventDestroy(s.t0);
    cudaEventDestroy(s.t1);
  }
  for (cudaEvent_t e : dev->event_pool) cudaEventDestroy(e);
  cudaStreamDestroy(dev->stream);
  delete dev;
  return FC_OK;
}

FC_API int fc_device_name(FcDevice* dev, char* buf, size_t buf_len) {
  if (!dev || !buf || buf_len == 0) return FC_ERR_ARG;
  snprintf(buf, buf_len, "%s (CUDA device %d, sm_%d%d, %d SMs)", dev->prop.name, dev->ordinal, dev->prop.major,
           dev->prop.minor, dev->prop.multiProcessorCount);
  return FC_OK;
}

FC_API int fc_device_props(FcDevice* dev, int* sm_count, uint64_t* total_mem_bytes) {
  if (!dev) return FC_ERR_ARG;
  if (sm_count) *sm_count = dev->prop.multiProcessorCount;
  if (total_mem_bytes) *total_mem_bytes = dev->prop.totalGlobalMem;
  return FC_OK;
}

FC_API const char* fc_last_error(FcDevice* dev) {
  if (dev) return dev->last_error.c_str();
  std::lock_guard<std::mutex> lock(g_err_mutex);
  return g_no_device_error.c_str();
}

FC_API void* fc_device_stream(FcDevice* dev) { return dev ? (void*)dev->stream : nullptr; }

// Also the place where a caller of the device-pointer entry points learns that a kernel gave up a bounded wait:
// the status word the kernels raise is read with the synchronisation and cleared.
FC_API int fc_device_sync(FcDevice* dev) {
  if (!dev) return FC_ERR_ARG;
  cudaSetDevice(dev->ordinal);
  int flag = 0;
  if (dev->d_flag) FC_CUDA(dev, cudaMemcpyAsync(&flag, dev->d_flag, sizeof(int), cudaMemcpyDeviceToHost, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (flag != 0) {
    cudaMemsetAsync(dev->d_flag, 0, sizeof(int), dev->stream);
    return fc_fail(dev, FC_ERR_TIMEOUT, "a kernel gave up a bounded wait (status %d): results since the last synchronisation are incomplete", flag);
  }
  return FC_OK;
}

// Test hook: raise the status word the way a kernel that gave up a wait does (no kernel has to time out).
FC_API int fc_debug_raise_status(FcDevice* dev, int value) {
  if (!dev || !dev->d_flag) return FC_ERR_ARG;
  cudaSetDevice(dev->ordinal);
  FC_CUDA(dev, cudaMemcpyAsync(dev->d_flag, &value, sizeof(int), cudaMemcpyHostToDevice, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return FC_OK;
}

FC_API uint64_t fc_device_launch_count(FcDevice* dev) { return dev ? dev->launches : 0; }

FC_API int fc_debug_fail_after(FcDevice* dev, int64_t n_launches) {
  if (!dev) return FC_ERR_ARG;
  dev->fail_after = n_launches < 0 ? -1 : n_launches;
  return FC_OK;
}

FC_API int fc_debug_matvec_kernel(FcDevice* dev, int choice) {
  if (!dev || choice < 0 || choice > 2) return FC_ERR_ARG;
  dev->matvec_choice = choice;
  return FC_OK;
}

FC_API int fc_debug_profile(FcDevice* dev, int enable) {
  if (!dev) return FC_ERR_ARG;
  cudaSetDevice(dev->ordinal);
  dev->profiling = enable != 0;
  return FC_OK;
}

// JSON object {"kernel name": {"launches": n, "ms": total}, ...} of every launch timed since the last
// report; synchronises the stream, then forgets the spans.
FC_API int fc_debug_profile_report(FcDevice* dev, char* buf, size_t buf_len) {
  if (!dev || !buf || buf_len < 3) return FC_ERR_ARG;
  cudaSetDevice(dev->ordinal);
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  struct Acc {
    const char* name;
    uint64_t n;
    double ms;
  };
  std::vector<Acc> acc;
  for (auto& s : dev->spans) {
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, s.t0, s.t1);
    Acc* a = nullptr;
    for (auto& e : acc)
      if (e.name == s.name || std::string(e.name) == s.name) a = &e;
    if (!a) {
      acc.push_back({s.name, 0, 0.0});
      a = &acc.back();
    }
    a->n++;
    a->ms += ms;
    dev->event_pool.push_back(s.t0);
    dev->event_pool.push_back(s.t1);
  }
  dev->spans.clear();
  std::string out = "{";
  for (size_t i = 0; i < acc.size(); i++) {
    char line[256];
    snprintf(line, sizeof line, "%s\"%s\": {\"launches\": %llu, \"ms\": %.6f}", i ? ", " : "", acc[i].name,
             (unsigned long long)acc[i].n, acc[i].ms);
    out += line;
  }
  out += "}";
  if (out.size() + 1 > buf_len) return fc_fail(dev, FC_ERR_SHAPE, "the profile report needs %zu bytes", out.size() + 1);
  memcpy(buf, out.c_str(), out.size() + 1);
  return FC_OK;
}

// ---- weight upload -------------------------------------------------------------------------------

void qweight_free(FcQWeight* w) {
  if (!w) return;
  if (w->qs_alloc) cudaFree(w->qs_alloc);
  if (w->sc_alloc) cudaFree(w->sc_alloc);
  delete w;
}

// Build one device weight of n = sum(ns) output rows from `count` host tensors that share the input width k (q, k
// and v, or gate and up, become one weight). A part of kind FC_F32 is an f32 `[k, ns[i]]` matrix and is quantised
// to `kind` on the device; a part of a block kind is the GGUF bytes of the tensor (ns[i] rows of k / 32 blocks)
// and is repacked as it is (ferrum_gguf/src/io/reader.rs:L298 hands exactly these bytes) - no dequantise /
// transpose / requantise round trip, and bit-identical to it by the reference's identity test
// (ferrum_wgpu/src/ops/quant/tests.rs:L89-L104). All parts must come out as the same stored format.
int qweight_from_parts(FcDevice* dev, int kind, const WeightSrc* parts, const uint32_t* ns, int count, uint32_t k,
                       FcQWeight** out) {
  *out = nullptr;
  uint64_t n_total = 0;
  size_t stage_bytes = 0;
  kind = effective_kind(kind, k);              // Q2_K on a width of whole 32s only: Q4_0 (ops/quant.rs:L134-L144)
  if (kind != FC_F32 && k % QK) kind = FC_F32; // ineligible width stays f32 (ops/quant.rs:L125-L134, lin.rs:L54-L61)
  int stored = -1;
  for (int i = 0; i < count; i++) {
    n_total += ns[i];
    if (!parts[i].p) return fc_fail(dev, FC_ERR_ARG, "a weight tensor is missing");
    const int pk = parts[i].kind == FC_F32 ? kind : parts[i].kind;
    if (!kind_known(pk)) return fc_fail(dev, FC_ERR_ARG, "unknown weight kind %d", pk);
    if (parts[i].kind != FC_F32 && k % kind_block_elems(pk))
      return fc_fail(dev, FC_ERR_SHAPE, "a width of %u is not whole %u-element blocks", k, kind_block_elems(pk));
    if (stored >= 0 && pk != stored)
      return fc_fail(dev, FC_ERR_UNSUPPORTED, "the tensors of one stacked weight are stored in different formats (%d and %d)", stored, pk);
    stored = pk;
    const size_t b = parts[i].kind == FC_F32 ? (size_t)k * ns[i] * 4 : fc_block_bytes(pk, (size_t)k * ns[i]);
    stage_bytes = b > stage_bytes ? b : stage_bytes;
  }
  if (k == 0 || n_total == 0 || n_total > 0x7fffffffu) return fc_fail(dev, FC_ERR_SHAPE, "empty or oversized weight");
  kind = stored;
  const uint32_t n = (uint32_t)n_total;
  FcQWeight* w = new FcQWeight();
  w->dev = dev;
  const size_t qs_bytes = qmat_qs_bytes(kind, k, n), sc_bytes = qmat_sc_bytes(kind, k, n);
  uint8_t* stage = nullptr;
  cudaError_t e = cudaMalloc(&w->qs_alloc, qs_bytes);
  if (e == cudaSuccess && sc_bytes) e = cudaMalloc(&w->sc_alloc, sc_bytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&stage, stage_bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    qweight_free(w);
    if (stage) cudaFree(stage);
    return fc_fail(dev, FC_ERR_OOM, "cannot allocate a %u x %u weight: %s", k, n, cudaGetErrorString(e));
  }
  w->m.kind = kind;
  w->m.k = k;
  w->m.n = n;
  w->m.qs = (const uint8_t*)w->qs_alloc;
  w->m.sc = (const __half*)w->sc_alloc;
  w->bytes = qs_bytes + sc_bytes;
  int rc = FC_OK;
  size_t row0 = 0;
  for (int i = 0; i < count && rc == FC_OK; i++) {
    const bool f32 = parts[i].kind == FC_F32;
    const size_t bytes = f32 ? (size_t)k * ns[i] * 4 : fc_block_bytes(kind, (size_t)k * ns[i]);
    e = cudaMemcpyAsync(stage, parts[i].p, bytes, cudaMemcpyHostToDevice, dev->stream);
    if (e != cudaSuccess) {
      rc = fc_fail(dev, FC_ERR_DEVICE, "weight upload failed: %s", cudaGetErrorString(e));
      break;
    }
    uint8_t* qs = (uint8_t*)w->qs_alloc + qmat_qs_bytes(kind, k, row0);
    __half* sc = w->sc_alloc ? (__half*)((uint8_t*)w->sc_alloc + qmat_sc_bytes(kind, k, row0)) : nullptr;
    if (!f32)
      rc = k_repack_blocks(dev, kind, stage, k, ns[i], qs, sc);
    else
      rc = kind == FC_F32 ? k_transpose_kn(dev, (const float*)stage, k, ns[i], (float*)qs)
                          : k_quantise_kn(dev, kind, (const float*)stage, k, ns[i], qs, sc);
    if (rc == FC_OK && cudaStreamSynchronize(dev->stream) != cudaSuccess) {
      dev->lost = true;
      rc = fc_fail(dev, FC_ERR_DEVICE, "weight upload failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    row0 += ns[i];
  }
  cudaFree(stage);
  if (rc != FC_OK) {
    qweight_free(w);
    return rc;
  }
  *out = w;
  return FC_OK;
}

// The same from f32 `[k, ns[i]]` matrices only.
int qweight_from_f32_concat(FcDevice* dev, int kind, const float* const* mats, const uint32_t* ns, int count,
                            uint32_t k, FcQWeight** out) {
  std::vector<WeightSrc> parts(count);
  for (int i = 0; i < count; i++) parts[i] = WeightSrc{mats[i], FC_F32};
  return qweight_from_parts(dev, kind, parts.data(), ns, count, k, out);
}

int qweight_from_f32(FcDevice* dev, int kind, const float* w_host, uint32_t k, uint32_t n, FcQWeight** out) {
  return qweight_from_f32_concat(dev, kind, &w_host, &n, 1, k, out);
}
