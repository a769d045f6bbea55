// Shared host-side plumbing of libferrum_cuda: device handle, status/error helpers, launch
// accounting with host-side fault injection, and the packed-weight descriptor every kernel takes.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/ferrum_cuda.h"

#define FC_API extern "C" __attribute__((visibility("default")))

constexpr int QK = 32; // elements per quantisation block (ferrum_gguf/src/lib.rs:L55)

struct FcDevice {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  cudaDeviceProp prop{};
  std::string last_error;
  bool lost = false;       // a CUDA call failed: sticky, like the reference's device-lost health
  uint64_t launches = 0;   // kernels launched by this library on this device
  int64_t fail_after = -1; // fault injection: launches left before every launch is refused
  void* pinned = nullptr;  // pinned host staging for results and small inputs
  size_t pinned_bytes = 0;
  int* d_flag = nullptr;   // device int for kernels that report a status
  int matvec_choice = 0;   // fc_debug_matvec_kernel: which kernel multiplies 1..8 rows (0: the library's rule)
  // per-kernel timing (off by default): one event pair per launch, summed by name on report
  bool profiling = false;
  struct ProfSpan {
    const char* name;
    cudaEvent_t t0, t1;
  };
  std::vector<ProfSpan> spans;
  std::vector<cudaEvent_t> event_pool;
};

// Record a message and hand back the status code.
int fc_fail(FcDevice* dev, int code, const char* fmt, ...);

// Counts one kernel launch; refuses it (before it reaches the device) when the injection hook
// has run out. Every launch in the library goes through FC_LAUNCH.
int fc_pre_launch(FcDevice* dev, const char* what);
int fc_post_launch(FcDevice* dev, const char* what);

#define FC_TRY(expr)            \
  do {                          \
    int _rc = (expr);           \
    if (_rc != FC_OK) return _rc; \
  } while (0)

#define FC_CUDA(dev, expr)                                                                   \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess) {                                                                 \
      (dev)->lost = _e != cudaErrorMemoryAllocation;                                         \
      return fc_fail((dev), _e == cudaErrorMemoryAllocation ? FC_ERR_OOM : FC_ERR_DEVICE,    \
                     "%s: %s", #expr, cudaGetErrorString(_e));                               \
    }                                                                                        \
  } while (0)

#define FC_LAUNCH(dev, what, ...)         \
  do {                                    \
    FC_TRY(fc_pre_launch((dev), (what))); \
    __VA_ARGS__;                          \
    FC_TRY(fc_post_launch((dev), (what))); \
  } while (0)

// A kernel's attributes (dynamic shared memory limit) are set per device: a once-flag per device ordinal, one
// static instance per kernel instantiation.
struct OncePerDevice {
  bool done[64] = {};
  bool first(int ordinal) {
    if (ordinal < 0 || ordinal >= 64) return true; // (out of the table: set the attribute every time)
    if (done[ordinal]) return false;
    done[ordinal] = true;
    return true;
  }
  void again(int ordinal) { // the set-up did not complete: the next call repeats it
    if (ordinal >= 0 && ordinal < 64) done[ordinal] = false;
  }
};

// Pinned staging buffer of at least `bytes` (grown on demand).
int fc_pinned(FcDevice* dev, size_t bytes, void** out);

// A weight matrix as the kernels see it: `n` output rows of `k` inputs.
//  FC_Q8_0: qs = int8 [n][k];            sc = f16 [n][k/32]
//  FC_Q4_0: qs = u8   [n][k/2], 16 bytes (four u32 words) per block; word w holds elements
//           8w..8w+7 of the block, element j in nibble position (j>>1) + 4*(j&1), so that the
//           mask pairs (p, p+4) of one word unpack to consecutive elements; sc as above
//  FC_F32:  qs = f32  [n][k];            sc = nullptr
//  FC_F16:  qs = f16  [n][k];            sc = nullptr
//  FC_FP8_E4M3 / FC_FP8_E5M2: Q8_0's planes, the bytes being FP8 codes instead of int8 quants
//  FC_Q2_K: super-blocks of 256 (k a multiple of 256). qs = u8 [n][k/4], 2 bits per element in element
//           order (64 bytes per super-block; 32-bit word j is sub-block j, 16 elements); sc = 20-byte
//           records [n][k/256]: the 16 scale/min bytes of the sub-blocks in element order, then d and dmin (f16)
//  FC_MXFP4: qs = u8 [n][k/2], 16 bytes per block in element order (byte i: element 2i in the low nibble,
//           2i+1 in the high one), each nibble an E2M1 code; sc = u16 [n][k/32], the bf16 bit pattern
//           of the block's power-of-two scale 2^(e-127) (all 255 scale bytes fit: the smallest is a
//           bf16 subnormal), so a kernel gets the f32 scale with one shift
struct QMat {
  int kind = FC_F32;
  uint32_t k = 0, n = 0;
  const uint8_t* qs = nullptr;
  const __half* sc = nullptr;
};

struct FcQWeight {
  FcDevice* dev = nullptr;
  QMat m;
  void* qs_alloc = nullptr;
  void* sc_alloc = nullptr;
  uint64_t bytes = 0;
  // bf16 GEMM operand descriptors are built lazily by the tensor path
  void* tc_cache = nullptr;
  size_t tc_cache_bytes = 0;
  void* mma_scratch = nullptr; // scratch of the batched-decode product for stand-alone use
};

__host__ __device__ constexpr bool kind_is_fp8(int kind) { return kind == FC_FP8_E4M3 || kind == FC_FP8_E5M2; }
// one byte per element and an f16 scale per 32: Q8_0 and the FP8 formats share planes, loads and addressing
__host__ __device__ constexpr bool kind_byte_blocks(int kind) { return kind == FC_Q8_0 || kind_is_fp8(kind); }
// half a byte per element, 16 bytes per block: Q4_0 and MXFP4 share addressing (not the nibble order)
__host__ __device__ constexpr bool kind_nibble_blocks(int kind) { return kind == FC_Q4_0 || kind == FC_MXFP4; }
__host__ __device__ constexpr bool kind_has_scales(int kind) { return kind_byte_blocks(kind) || kind_nibble_blocks(kind); }
static inline bool kind_known(int kind) { return kind >= FC_F32 && kind <= FC_Q2_K; }
constexpr uint32_t QK_K = 256; // elements of a Q2_K super-block
static inline uint32_t kind_block_elems(int kind) { return kind == FC_Q2_K ? QK_K : QK; }
// ops/quant.rs:L134-L144 (`effective`): Q2_K on a width of whole 32s but not whole 256s is stored as Q4_0
static inline int effective_kind(int kind, uint64_t k) {
  return (kind == FC_Q2_K && k % QK_K != 0 && k > 0 && k % QK == 0) ? FC_Q4_0 : kind;
}

static inline size_t qmat_qs_bytes(int kind, size_t k, size_t n) {
  return kind_byte_blocks(kind)     ? k * n
         : kind_nibble_blocks(kind) ? k * n / 2
         : kind == FC_Q2_K          ? k * n / 4
         : kind == FC_F16           ? k * n * 2
                                    : k * n * 4;
}
static inline size_t qmat_sc_bytes(int kind, size_t k, size_t n) {
  return kind == FC_Q2_K ? (k / QK_K) * n * 20 : kind_has_scales(kind) ? (k / QK) * n * 2 : 0;
}

#ifdef __CUDACC__
// Two FP8 codes (the low 16 bits of `two`) as two fp16 values, low byte in the low half. Exact: every
// E4M3 and E5M2 value, infinities and NaNs included, is an fp16 value.
template <int KIND>
__device__ __forceinline__ uint32_t fp8x2_to_f16x2(uint32_t two) {
  uint32_t r;
  const unsigned short v = (unsigned short)two;
  if (KIND == FC_FP8_E4M3)
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  else
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}
// The eight E2M1 codes of one word of an MXFP4 block (byte i: elements 2i, 2i+1) as four fp16 pairs in
// element order. Exact: the values are 0, 0.5, 1, 1.5, 2, 3, 4, 6 and their negatives.
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t (&o)[4]) {
  asm("{\n.reg .b8 b0, b1, b2, b3;\nmov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\ncvt.rn.f16x2.e2m1x2 %1, b1;\ncvt.rn.f16x2.e2m1x2 %2, b2;\ncvt.rn.f16x2.e2m1x2 %3, b3;\n}"
      : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3])
      : "r"(w));
}
// The f32 scale of a block from its 16-bit slot: an f16 for the GGUF integer / FP8 formats, the bf16 bits
// of a power of two for MXFP4.
template <int KIND>
__device__ __forceinline__ float block_scale_f32(__half raw) {
  return KIND == FC_MXFP4 ? __uint_as_float((uint32_t)__half_as_ushort(raw) << 16) : __half2float(raw);
}
// One code as f32 (exact).
template <int KIND>
__device__ __forceinline__ float fp8_to_f32(uint32_t code) {
  const uint32_t h2 = fp8x2_to_f16x2<KIND>(code & 0xffu);
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
}
#endif

// Epilogue of a matrix product: y = act(x W + bias) (+ resid). All pointers device, nullable.
enum { ACT_NONE = 0, ACT_GELU = 1 };
// A 9..64-row product whose split-K partial sums have not been combined yet: the consumer of its result
// (the norm + split launch of the next product) adds them up, applies bias and residual, writes y and
// carries on - one launch instead of two on a step that is bound by its launch chain.
struct DeferredReduce {
  const float* partial = nullptr; // [splits][m][n]
  uint32_t splits = 0;            // 0: nothing pending
  uint32_t m = 0, n = 0;
  const float* bias = nullptr;
  const float* resid = nullptr;
  float* y = nullptr;
};

struct Epilogue {
  const float* bias = nullptr;  // [n]
  const float* resid = nullptr; // [m][n]; may alias y
  int act = ACT_NONE;
  // device scratch of at least qmatvec_mma_scratch_bytes(k, n): lets products of 9..64 rows run on the
  // tensor-core batched-decode kernel; without it they take the tiled f32 kernel
  void* scratch = nullptr;
  // "x is the raw residual stream: normalise each row first" (NORM_RMS: y = x / sqrt(mean(x^2) + eps) * g,
  // NORM_LAYER: (x - mean) / sqrt(var + 1e-5) * g + b). The one-row FMA matvec does it while it stages x
  // in shared memory (one launch less per product); the other kernels run the norm kernel into
  // `norm_tmp` ([m][k] floats) first.
  int norm = 0;
  const float* norm_g = nullptr;
  const float* norm_b = nullptr;
  float norm_eps = 0.0f;
  float* norm_tmp = nullptr;
  // the producer of x has already written its two fp16 terms where the 9..64-row tensor-core product
  // stages them (qmatvec_mma_split_ptrs): the product skips its split launch and ignores `x`
  bool presplit = false;
  // leave this product's split-K reduce to the consumer (filled in when the product did split)
  DeferredReduce* defer_out = nullptr;
  // where a deferring product puts its partial sums, when the place behind its own x terms would be
  // overwritten by the consumer (nullable: that default place)
  float* partial_at = nullptr;
  // finish this pending reduce first: its y is this product's x (same buffer, raw residual stream)
  const DeferredReduce* pending = nullptr;
};
enum { NORM_NONE = 0, NORM_RMS = 1, NORM_LAYER = 2 };

// matvec_mma.cu: 9 <= m <= 64 rows at f32-class accuracy on mma.sync
bool qmatvec_mma_supports(const QMat& w, uint32_t m);
size_t qmatvec_mma_scratch_bytes(uint32_t k, uint32_t n);
int k_qmatvec_mma(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep, void* scratch);
// Whether k_qlinear_f32 will take the 9..64-row tensor-core product for (w, m) with this scratch, and where
// that product expects the two fp16 terms of x ([mp][k] each, rows >= m zero).
bool qlinear_takes_wide_mma(const QMat& w, uint32_t m, const void* scratch);
int k_flush_deferred(FcDevice* dev, const DeferredReduce& d);
void qmatvec_mma_split_ptrs(void* scratch, uint32_t m, uint32_t k, __half** xh, __half** xl, uint32_t* mp);

// ---- kernels' host entry points (each enqueues on dev->stream) --------------------------------
// codec.cu
int k_quantise_kn(FcDevice* dev, int kind, const float* w_kn_dev, uint32_t k, uint32_t n, uint8_t* qs, __half* sc);
int k_transpose_kn(FcDevice* dev, const float* w_kn_dev, uint32_t k, uint32_t n, float* out_nk);
int k_repack_blocks(FcDevice* dev, int kind, const uint8_t* blocks_dev, uint32_t k, uint32_t n, uint8_t* qs, __half* sc);
int k_export_blocks(FcDevice* dev, const QMat& m, uint8_t* blocks_dev);
int k_dequant(FcDevice* dev, const QMat& m, float* out_nk_dev);
// matvec.cu: m <= 8 rows
int k_qmatvec(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep);
// matvec1.cu: one row of a block format, streamed through shared memory onto mma.sync
// gemm_tc.cu: the exact-class tcgen05 product of 2..64 rows of x (x as its two fp16 terms)
bool qgemm_tx_takes(const FcDevice* dev, const QMat& w, uint32_t m, bool deferring);
int k_qgemm_tx(FcDevice* dev, const QMat& w, const __half* xh, const __half* xl, uint32_t mp, uint32_t m, float* y,
               const Epilogue& ep);
bool qmatvec1_supports(const FcDevice* dev, const QMat& w);
int k_qmatvec1(FcDevice* dev, const QMat& w, const float* x, float* y, const Epilogue& ep);
// gemm_f32.cu: any m
int k_qgemm_f32(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep);
// The exact-f32 product of any m: picks matvec or tiled GEMM.
int k_qlinear_f32(FcDevice* dev, const QMat& w, const float* x, uint32_t m, float* y, const Epilogue& ep);

// Upload helpers (runtime.cu)
// One host tensor of a weight: kind FC_F32 = an f32 `[in, out]` matrix (the reference's host layout), a block kind =
// the GGUF bytes of the `[out, in]` tensor.
struct WeightSrc {
  const void* p;
  int kind;
};
int qweight_from_parts(FcDevice* dev, int kind, const WeightSrc* parts, const uint32_t* ns, int count, uint32_t k,
                       FcQWeight** out);
int qweight_from_f32(FcDevice* dev, int kind, const float* w_in_out_host, uint32_t k, uint32_t n, FcQWeight** out);
int qweight_from_f32_concat(FcDevice* dev, int kind, const float* const* mats_host, const uint32_t* ns, int count,
                            uint32_t k, FcQWeight** out);
void qweight_free(FcQWeight* w);
