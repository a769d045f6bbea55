// A product entry point that allocates nothing.
//
// fc_qmatmul_dev in tensor-core mode needs scratch: the f32 activations are first rounded to an fp16
// copy that the TMA loads of the product read, and that copy normally lives in a buffer the library
// cudaMalloc's (and grows) per weight. Some callers cannot let that happen: code running between
// cudaStreamBeginCapture and EndCapture on another stream of the same context, a host whose memory
// plan was fixed and checked before the first request (the reference refuses a model whose plan does
// not fit *before* allocating, models/llama/mod.rs:L241-L243, and then expects no further growth), or
// a latency-critical loop that must not meet the implicit device-wide synchronisation of cudaMalloc /
// cudaFree. For them the scratch here is a fixed array in the library's own device image: it exists
// on every GPU that loads the library, from load to exit, whether or not this entry point is used.
#include "gemm_tc.cuh"

// The fp16 copy of x: FC_NOALLOC_MAX_ELEMS activations (8 MiB).
constexpr size_t NOALLOC_MAX_ELEMS = (size_t)4 << 20;
static __device__ __align__(256) __half g_x_scratch[NOALLOC_MAX_ELEMS];

namespace {
constexpr int MAX_DEVICES = 64;
__half* g_scratch_ptr[MAX_DEVICES] = {}; // device address of g_x_scratch on each ordinal, resolved once
} // namespace

FC_API int fc_qmatmul_dev_noalloc(FcQWeight* w, const float* x_dev, uint32_t m, float* y_dev) {
  if (!w || !x_dev || !y_dev) return FC_ERR_ARG;
  FcDevice* dev = w->dev;
  if ((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(y_dev)) & 15)
    return fc_fail(dev, FC_ERR_ARG, "x_dev and y_dev must be 16-byte aligned"); // (the kernels move 16-byte pieces)
  cudaSetDevice(dev->ordinal);
  if (m == 0) return FC_OK;
  if ((size_t)m * w->m.k > NOALLOC_MAX_ELEMS)
    return fc_fail(dev, FC_ERR_SHAPE, "fc_qmatmul_dev_noalloc: %u rows of %u inputs exceed the fixed scratch of %zu elements",
                   m, w->m.k, NOALLOC_MAX_ELEMS);
  if (dev->ordinal < 0 || dev->ordinal >= MAX_DEVICES) return fc_fail(dev, FC_ERR_UNSUPPORTED, "device ordinal %d", dev->ordinal);
  // In host code `g_x_scratch` is only a handle for the symbol, not an address a kernel can use: the
  // device address is looked up once per device, with that device current. This first call on a
  // device should therefore come before any stream capture.
  if (!g_scratch_ptr[dev->ordinal]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_x_scratch);
    if (e != cudaSuccess || !p)
      return fc_fail(dev, FC_ERR_DEVICE, "cannot resolve the fixed scratch on device %d: %s", dev->ordinal, cudaGetErrorString(e));
    g_scratch_ptr[dev->ordinal] = (__half*)p;
  }
  __half* a = g_scratch_ptr[dev->ordinal];
  // the copy overwrites exactly the m * k elements the product reads; nothing has to start at zero
  FC_TRY(k_f32_to_f16(dev, x_dev, (size_t)m * w->m.k, a));
  TcArgs t;
  t.m = m;
  t.out_f32 = y_dev;
  t.ldo = w->m.n;
  return k_qgemm_tc_f16(dev, w->m, a, EPI_F32, t);
}
