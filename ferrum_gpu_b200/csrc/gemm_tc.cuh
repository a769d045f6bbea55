// Host interface of the bf16 tensor-core product (gemm_tc.cu) and its companions (ops_tc.cu).
#pragma once
#include <cuda.h>

#include "common.cuh"

// What the epilogue does with the 128 x 128 f32 accumulator tile.
enum {
  EPI_F32 = 0,    // out_f32[m][ldo]  = acc + bias
  EPI_BF16 = 1,   // out_bf16[m][ldo] = bf16(act(acc + bias))
  EPI_RESID = 2,  // out_f32[m][ldo] += acc + bias          (residual stream, in place)
  EPI_SWIGLU = 3, // out_bf16[m][n/2] = bf16(silu(gate) * up); weight rows interleaved 64 gate / 64 up
  EPI_LSE = 4     // partial[tile][m][4] = (max, sum exp, target logit | -inf, first argmax)
};

struct TcArgs {
  uint32_t m = 0, n = 0, k = 0;
  const float* bias = nullptr;
  float* out_f32 = nullptr;
  __nv_bfloat16* out_bf16 = nullptr;
  uint32_t ldo = 0;
  int act = ACT_NONE;
  const int32_t* targets = nullptr;
  uint32_t v0 = 0;
  float* partial = nullptr;
  int* err_flag = nullptr;
};

constexpr uint32_t TC_BM = 256, TC_BN = 128, TC_BK = 64; // output tile of one CTA step, K slice

// y = a[m][k] (bf16, row-major, device) . W^T with the epilogue `epi`. k % 64 == 0.
int k_qgemm_tc_bf16(FcDevice* dev, const QMat& w, const __nv_bfloat16* a, int epi, TcArgs args);
// Reads and clears the device-side error word the tensor kernels report bounded-wait failures in.
int tc_check_errors(FcDevice* dev);

// ops_tc.cu
int k_f32_to_bf16(FcDevice* dev, const float* x, size_t n, __nv_bfloat16* y);
int k_norm_bf16(FcDevice* dev, bool layernorm, const float* x, const float* g, const float* b, uint32_t rows, uint32_t d,
                float eps, __nv_bfloat16* y);
int k_rope_bf16(FcDevice* dev, __nv_bfloat16* qkv, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                const float* cos, const float* sin, uint32_t rope_dim, uint32_t type, const int32_t* positions);
int k_attn_causal_bf16(FcDevice* dev, const __nv_bfloat16* qkv, uint32_t n_seqs, uint32_t t, uint32_t heads,
                       uint32_t kv_heads, uint32_t hd, __nv_bfloat16* out);
int k_partial_merge(FcDevice* dev, const float* tiles, uint32_t n_tiles, uint32_t rows, float* out);
int k_permute_rows(FcDevice* dev, const uint8_t* src, uint8_t* dst, uint32_t rows, uint32_t row_bytes, uint32_t half,
                   uint32_t group);
